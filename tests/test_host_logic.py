"""CPU-only checks: the library loads and exports the header's symbols, argument validation of
the Python entry point and of the C ABI (error paths that return before any CUDA call)."""
import ctypes as C
import os
import re

import pytest
import torch

import triton_op_b200
from triton_op_b200 import PaArgumentError, _lib
from triton_op_b200 import build as pa_build
from triton_op_b200.inputs import DecodeConfig, make_inputs, pack_mtp, unpack_mtp
from triton_op_b200.pa_decode import build_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    pa_build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "pa_decode_sm100.h")).read()
    declared = set(re.findall(r"^\s*(?:int|int64_t|const char\*)\s+(pa_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.pa_abi_version() == _lib.PA_ABI_VERSION
    assert lib.pa_strerror(0) == b"ok" and b"NULL" in lib.pa_strerror(-1)


def test_struct_mirror_matches_header_field_order():
    header = open(os.path.join(ROOT, "include", "pa_decode_sm100.h")).read()
    start = header.index("typedef struct PaDecodeParams {") + len("typedef struct PaDecodeParams {")
    body = header[start:header.index("} PaDecodeParams;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        decl = re.sub(r"^(const\s+)?(void|float|int32_t|uint32_t|int64_t|uint64_t)\s*\*?\s*", "", decl)
        names += [n.strip().lstrip("*") for n in decl.split(",")]
    assert names == [f[0] for f in _lib.PaDecodeParams._fields_]


def _args(inp, **over):
    c = inp.cfg
    a = dict(output=torch.empty_like(inp.query), query=inp.query, key_cache=inp.key_cache,
             value_cache=inp.value_cache, sequence_lengths=inp.context_lens, block_tables=inp.block_tables,
             softmax_scale=inp.softmax_scale, query_sequence_length=c.query_len,
             max_sequence_length=inp.max_context, compute_type=torch.bfloat16, query_scale=None,
             key_scale=inp.key_scale, value_scale=inp.value_scale, alibi_slopes=None,
             partition_size=c.partition_size, exp_sums=None, max_logits=None, tmp_output=None,
             status=None, tune=None)
    a.update(over)
    return a


@pytest.fixture(scope="module")
def small():
    return make_inputs(DecodeConfig("t", 3, 8, 2, 16, 2, ("uniform", 5, 300)), seed=1)


def test_param_block_is_filled_from_the_tensors(small):
    p, keep = build_params(**_args(small))
    assert p.struct_size == C.sizeof(_lib.PaDecodeParams)
    assert (p.num_seqs, p.num_kv_heads, p.query_group_size, p.query_len) == (3, 2, 4, 2)
    assert p.block_size == 16 and p.head_size == 128 and p.partition_size == 256
    assert p.max_partitions == (small.max_context + 255) // 256
    assert p.kv_quant_mode == _lib.PA_QUANT_PER_TENSOR and p.q_quant_mode == _lib.PA_QUANT_NONE
    assert p.k_stride_head == 2048 and p.k_stride_block == 2 * 2048
    assert p.key_cache == small.key_cache.data_ptr()


def test_reference_asserts_are_reproduced(small):
    with pytest.raises(AssertionError, match="output tensor only support dtype"):
        build_params(**_args(small, output=torch.empty_like(small.query, dtype=torch.float16)))
    with pytest.raises(ValueError, match="Expected 3D query"):
        build_params(**_args(small, query=small.query[0]))
    with pytest.raises(PaArgumentError, match="Expected 5D key_cache"):
        build_params(**_args(small, key_cache=small.key_cache[0]))
    with pytest.raises(RuntimeError, match="Unsupported value cache shape"):
        build_params(**_args(small, value_cache=small.value_cache[0]))
    with pytest.raises(PaArgumentError, match="QUERY_SEQ_LEN"):
        build_params(**_args(small, query_sequence_length=8))
    with pytest.raises(PaArgumentError, match="same shape"):
        build_params(**_args(small, value_scale=torch.ones(4, 2, 16, 1)))
    with pytest.raises(PaArgumentError, match="only support dtype == torch.float32"):
        build_params(**_args(small, key_scale=small.key_scale.double(), value_scale=small.value_scale.double()))
    big = make_inputs(DecodeConfig("g", 1, 40, 1, 16, 2, ("fixed", 20)), seed=0)   # eqG = 80 > 64
    with pytest.raises(PaArgumentError, match="exceeds maximum of 64"):
        build_params(**_args(big))
    kc = torch.zeros(4, 2, 8, 32, 16, dtype=torch.float8_e4m3fn)                   # block size 32
    with pytest.raises(PaArgumentError, match="not in"):
        build_params(**_args(small, key_cache=kc, value_cache=torch.zeros(4, 2, 128, 32, dtype=torch.float8_e4m3fn)))


def test_cpu_tensors_are_refused_not_emulated(small, lib):
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        a = _args(small)
        triton_op_b200.paged_attention_decode(
            a["output"], a["query"], a["key_cache"], a["value_cache"], a["sequence_lengths"], a["block_tables"],
            a["softmax_scale"], a["query_sequence_length"], a["max_sequence_length"], a["compute_type"],
            None, a["key_scale"], a["value_scale"])


def test_c_abi_rejects_bad_blocks_before_touching_cuda(small, lib):
    p, keep = build_params(**_args(small))
    assert lib.pa_decode_sm100(None, None) == -1
    q = _lib.PaDecodeParams.from_buffer_copy(p)
    q.struct_size = 8
    assert lib.pa_decode_sm100(C.byref(q), None) == -6
    q = _lib.PaDecodeParams.from_buffer_copy(p)
    q.key_cache = None
    assert lib.pa_partition_sm100(C.byref(q), None) == -1
    q = _lib.PaDecodeParams.from_buffer_copy(p)
    q.head_size = 64
    assert lib.pa_decode_sm100(C.byref(q), None) == -3
    q = _lib.PaDecodeParams.from_buffer_copy(p)
    q.num_kv_heads = 0
    assert lib.pa_decode_sm100(C.byref(q), None) == -2
    q = _lib.PaDecodeParams.from_buffer_copy(p)
    q.tmp_stride_row = 3
    assert lib.pa_reduce_sm100(C.byref(q), None, None, None, None) == -4
    assert lib.pa_reduce_sm100(C.byref(p), C.c_void_p(16), None, None, None) == -1  # partial triple
    assert lib.pa_merge_triples_sm100(None, 128, None, None, None, 2, 4, 128, None) == -1
    assert lib.pa_merge_triples_sm100(C.c_void_p(64), 128, C.c_void_p(64), C.c_void_p(64), C.c_void_p(64),
                                      2, 4, 64, None) == -3


def test_mtp_row_permutation_round_trip():
    x = torch.arange(3 * 2 * 8 * 4, dtype=torch.float32).reshape(3 * 2, 8, 4)
    packed = pack_mtp(x, 3, 2, 2)          # S=3, L=2, Hkv=2, G=4
    assert packed.shape == (3, 16, 4)
    # row r = t*G + g of kv head h is token t, head h*G+g
    s, h, t, g = 1, 1, 1, 2
    assert torch.equal(packed[s, h * 8 + t * 4 + g], x[s * 2 + t, h * 4 + g])
    assert torch.equal(unpack_mtp(packed, 3, 2, 2), x)


def test_subset_inputs_keeps_every_kept_sequence_bit_for_bit():
    """``subset_inputs`` (what the benchmark's parity check moves to the host) renumbers the pages of the
    kept sequences only: the oracle on the subset equals the oracle's rows of the full batch."""
    from oracle import pa_oracle
    from triton_op_b200.inputs import DecodeConfig, make_inputs, subset_inputs
    for cfg in (DecodeConfig("s1", 6, 8, 2, 16, 2, ("uniform", 2, 300), quant="per_token"),
                DecodeConfig("s2", 5, 4, 1, 64, 1, ("uniform", 1, 500))):
        inp = make_inputs(cfg, seed=5)
        ks, vs = inp.flat_scales()
        full = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables,
                                         inp.context_lens, inp.query_indptr(), ks, vs)
        ids = [1, 4, 5] if cfg.num_seqs > 5 else [0, 3]
        sub = subset_inputs(inp, ids)
        assert sub.key_cache.shape[0] < inp.key_cache.shape[0]
        ks, vs = sub.flat_scales()
        part = pa_oracle.paged_attention(sub.query_tokens, sub.key_cache, sub.value_cache, sub.block_tables,
                                         sub.context_lens, sub.query_indptr(), ks, vs)
        L = cfg.query_len
        rows = [s * L + t for s in ids for t in range(L)]
        assert torch.equal(part, full[rows])
        assert torch.equal(sub.query, inp.query[ids])
