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
