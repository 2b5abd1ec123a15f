"""The oracle against the fixtures made from the reference's own PyTorch functions (CPU)."""
import pytest
import torch

from _util import GOLDEN_CASES, golden_inputs, load_golden, make_golden, oracle_output
from oracle import pa_oracle


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_oracle_matches_reference_golden(name):
    torch.set_num_threads(1)
    gold = load_golden(name)
    inp = golden_inputs(name)
    # the inputs must be the ones the fixture was made from, else a mismatch means nothing
    assert make_golden.input_digest(inp) == gold["digest"], "seeded inputs differ from the fixture's"
    assert torch.equal(inp.context_lens, gold["context_lens"])
    out = oracle_output(inp)
    assert out.dtype == torch.bfloat16 and out.shape == gold["out"].shape
    # same torch ops in the same order as the reference: bit-exact
    assert torch.equal(out.view(torch.int16), gold["out"].view(torch.int16))


@pytest.mark.parametrize("name", ["cfg1_small", "mtp2_g8", "mtp4_g2_pertoken", "partition512", "bs64_g5"])
def test_split_kv_statement_agrees_with_full_attention(name):
    """merge(partition triples) == unsplit attention: pins the split-KV restatement."""
    inp = golden_inputs(name)
    c = inp.cfg
    ks, vs = inp.flat_scales()
    m, l, o = pa_oracle.split_kv_partials(inp.query, inp.key_cache, inp.value_cache, inp.block_tables,
                                          inp.context_lens, c.query_len, inp.softmax_scale, c.partition_size, ks, vs)
    merged = pa_oracle.merge_partials(m, l, o)                     # [S, Hkv, eqG, D]
    from triton_op_b200.inputs import unpack_mtp
    merged = unpack_mtp(merged.reshape(c.num_seqs, -1, c.head_size), c.num_seqs, c.query_len, c.kv_heads)
    ref = load_golden(name)["out"].float()
    assert torch.allclose(merged, ref, atol=4e-3, rtol=8e-3)  # fp32 vs the bf16-rounded golden


def test_merge_triples_is_associative():
    torch.manual_seed(0)
    m = torch.randn(4, 50) * 3
    l = torch.rand(4, 50) + 0.1
    o = torch.randn(4, 50, 128)
    l[1, :10] = 0  # an empty shard for some rows
    m[1, :10] = float("-inf")
    full = pa_oracle.merge_triples(m, l, o)
    # merging two halves first, then the halves, gives the same answer
    def half(sl):
        M = torch.where(l[sl] > 0, m[sl], torch.full_like(m[sl], float("-inf"))).max(0).values
        w = torch.where(l[sl] > 0, l[sl] * torch.exp(m[sl] - M), torch.zeros_like(l[sl]))
        return M, w.sum(0), pa_oracle.merge_triples(m[sl], l[sl], o[sl])
    ma, la, oa = half(slice(0, 2))
    mb, lb, ob = half(slice(2, 4))
    two = pa_oracle.merge_triples(torch.stack([ma, mb]), torch.stack([la, lb]), torch.stack([oa, ob]))
    assert torch.allclose(full, two, atol=1e-5, rtol=1e-5)


def test_compare_arrays_metrics():
    import numpy as np
    a = np.array([[1.0, 2.0], [3.0, 4.5]], dtype=np.float32)
    b = np.array([[1.0, 2.5], [3.0, 4.0]], dtype=np.float32)
    r = pa_oracle.compare_arrays(a, b, k=2)
    assert r["max_abs_diff"] == pytest.approx(0.5)
    assert r["max_diff_thr"] == pytest.approx(0.5 / 3.5)
    assert r["top_k_diff"][0]["value"] == pytest.approx(0.5)
    assert sum(s["count"] for s in r["threshold_stats"]) == 4
    with pytest.raises(ValueError):
        pa_oracle.compare_arrays(a, b[:1])


# ----------------------------------------------------------------------------- fixtures run by the reference's Triton path
import importlib.util as _ilu
import os as _os

import numpy as _np

_spec = _ilu.spec_from_file_location("make_golden_triton", _os.path.join(_os.path.dirname(__file__), "golden", "make_golden_triton.py"))
make_golden_triton = _ilu.module_from_spec(_spec)
_spec.loader.exec_module(make_golden_triton)


def load_triton_golden(name):
    z = _np.load(_os.path.join(_os.path.dirname(__file__), "golden", name + ".npz"))
    g = {k: torch.from_numpy(z[k].copy()) for k in ("out", "tmp_output", "exp_sums", "max_logits", "alibi_slopes", "context_lens")}
    g["digest"] = dict(zip(z["digest_keys"].tolist(), z["digest_vals"].tolist()))
    return g


# The reference computed these in fp16 (scaled query, probabilities, partial and final outputs all
# rounded to fp16, fp32 accumulation); the oracle is fp32 throughout.  Tolerances are fp16-level.
TRITON_OUT_TOL = dict(atol=3e-3, rtol=1e-2)
TRITON_LOGIT_TOL = dict(atol=1e-2, rtol=2e-3)
TRITON_SUM_TOL = dict(atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("name", sorted(make_golden_triton.CASES))
def test_oracle_alibi_and_split_kv_match_the_reference_triton_run(name):
    """Outputs and split-KV intermediates of pa_decode_triton.paged_attention_decode (run on CPU under
    the Triton interpreter, with and without alibi_slopes) against the oracle: pins the oracle's ALiBi
    bias (slope * (key position - (context - 1)), per query head) and its (max, sum, normalised
    output) statement per 256-token partition to something the reference itself executed."""
    gold = load_triton_golden(name)
    inp, slopes = make_golden_triton.case_inputs(name)
    assert make_golden.input_digest(inp) == gold["digest"], "seeded inputs differ from the fixture's"
    c = inp.cfg
    if slopes is not None:
        assert torch.equal(slopes, gold["alibi_slopes"])
    out = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables, inp.context_lens,
                                    inp.query_indptr(), None, None, alibi_slopes=slopes).float()
    assert torch.allclose(out, gold["out"], **TRITON_OUT_TOL), float((out - gold["out"]).abs().max())
    m, l, o = pa_oracle.split_kv_partials(inp.query, inp.key_cache, inp.value_cache, inp.block_tables, inp.context_lens,
                                          1, inp.softmax_scale, 256, None, None, alibi_slopes=slopes)
    for s in range(c.num_seqs):
        np_s = (int(inp.context_lens[s]) + 255) // 256
        assert torch.allclose(m[s, :, :np_s], gold["max_logits"][s, :, :np_s], **TRITON_LOGIT_TOL)
        assert torch.allclose(l[s, :, :np_s], gold["exp_sums"][s, :, :np_s], **TRITON_SUM_TOL)
        assert torch.allclose(o[s, :, :np_s], gold["tmp_output"][s, :, :np_s], **TRITON_OUT_TOL)
    if slopes is not None:      # the bias matters on these cases: without it the oracle is far off
        plain = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables,
                                          inp.context_lens, inp.query_indptr(), None, None).float()
        assert (plain - gold["out"]).abs().max() > 0.1
