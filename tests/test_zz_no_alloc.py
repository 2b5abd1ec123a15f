"""The entry point that allocates nothing (pa_decode_noalloc_sm100), through the C ABI.

Some users of this library cannot call cudaMalloc at all: a serving runtime that has already
given every byte of GPU memory to its own pool, or code that may be running while a stream is
being captured.  For them the split-KV workspaces live in a fixed array inside the library.
This checks that the variant returns what the normal entry point returns, on two calls in a
row with different inputs (the array keeps the previous call's contents, which must not
matter), and that a problem larger than the array is refused.

The file name sorts last on purpose: a run that stops at the first failure has then already
gone through every other test.
"""
import ctypes as C

import pytest
import torch

from _util import assert_close, golden_inputs, load_golden

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _params(inp, out):
    from triton_op_b200.pa_decode import build_params
    c = inp.cfg
    return build_params(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                        inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None,
                        inp.key_scale, inp.value_scale, None, c.partition_size, None, None, None, None, None)


def test_noalloc_entry_point_matches_the_normal_one_twice_in_a_row():
    from triton_op_b200 import _lib
    from triton_op_b200.inputs import unpack_mtp
    lib = _lib.lib()
    stream = torch.cuda.current_stream(DEV).cuda_stream
    with torch.cuda.device(DEV):
        for name in ("gqa4_ragged", "mtp4_g2_pertoken"):      # two calls in a row, different shapes
            inp = golden_inputs(name).to(DEV)
            c = inp.cfg
            want = torch.full_like(inp.query, float("nan"))
            p, keep = _params(inp, want)
            assert lib.pa_decode_sm100(C.byref(p), stream) == 0

            got = torch.full_like(inp.query, float("nan"))
            q, keep2 = _params(inp, got)
            q.exp_sums = None            # ignored by the variant: it brings its own workspaces
            q.max_logits = None
            q.tmp_out = None
            torch.cuda.synchronize()
            mem_before = torch.cuda.memory_allocated(DEV)
            free_before = torch.cuda.mem_get_info(DEV)[0]      # the driver's view: sees a cudaMalloc torch would not
            rc = lib.pa_decode_noalloc_sm100(C.byref(q), stream)
            assert rc == 0, lib.pa_strerror(rc)
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated(DEV) == mem_before
            assert torch.cuda.mem_get_info(DEV)[0] >= free_before
            assert not torch.isnan(got).any()
            # same kernels on the same inputs: equal well inside the tolerance of the other tests
            assert_close(got, want, what=f"{name}: noalloc vs normal entry point")
            ref = load_golden(name)["out"]
            assert_close(unpack_mtp(got, c.num_seqs, c.query_len, c.kv_heads), ref, what=f"{name}: noalloc vs golden")


def test_noalloc_entry_point_refuses_what_does_not_fit():
    from triton_op_b200 import _lib
    lib = _lib.lib()
    inp = golden_inputs("cfg1_small").to(DEV)
    out = torch.empty_like(inp.query)
    p, keep = _params(inp, out)
    rows_that_fit = _lib.PA_NOALLOC_SCRATCH_BYTES // 264
    p.max_partitions = rows_that_fit // (p.num_seqs * p.num_kv_heads * p.query_group_size * p.query_len) + 2
    with torch.cuda.device(DEV):
        rc = lib.pa_decode_noalloc_sm100(C.byref(p), torch.cuda.current_stream().cuda_stream)
    assert rc == -7 and b"limit" in lib.pa_strerror(rc)
    assert lib.pa_decode_noalloc_sm100(None, None) == -1
    # sizes whose product wraps around 64 bits must not slip under the limit
    p, keep = _params(inp, out)
    p.num_kv_heads = 2 ** 31 - 1
    p.max_partitions = 2 ** 31 - 1
    p.num_seqs = 2 ** 31 - 1
    with torch.cuda.device(DEV):
        assert lib.pa_decode_noalloc_sm100(C.byref(p), torch.cuda.current_stream().cuda_stream) == -7
