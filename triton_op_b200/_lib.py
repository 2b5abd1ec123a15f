"""ctypes binding of ``include/pa_decode_sm100.h``.

The library is the only compute path of this package: if it cannot be loaded the import of
the operator fails with an explicit error -- there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

PA_ABI_VERSION = 3

PA_OK = 0
PA_DT_BF16, PA_DT_E4M3FN = 0, 1
PA_QUANT_NONE, PA_QUANT_PER_TENSOR, PA_QUANT_PER_TOKEN = -1, 0, 1
PA_V_NORMAL, PA_V_TRANSPOSED = 0, 1
PA_DEV_WAIT_TIMEOUT, PA_DEV_BAD_PAGE_ID, PA_DEV_CTX_TOO_LONG = 1, 2, 4
PA_TRACE_WORDS = 8 * 64 * 4
PA_NOALLOC_SCRATCH_BYTES = 16 << 20
PA_IPC_HANDLE_BYTES = 64

EXPORTS = (
    "pa_decode_sm100", "pa_decode_noalloc_sm100", "pa_partition_sm100", "pa_reduce_sm100", "pa_merge_triples_sm100",
    "pa_merge_packed_triples_sm100", "pa_packed_triple_floats", "pa_exchange_alloc", "pa_exchange_open", "pa_exchange_close", "pa_exchange_free",
    "pa_exchange_bytes", "pa_reduce_push_sm100", "pa_merge_wait_sm100",
    "pa_cache_write_sm100", "pa_stream_probe_sm100", "pa_query_launch_sm100", "pa_strerror", "pa_last_cuda_error", "pa_abi_version",
)


class PaDecodeParams(C.Structure):
    """Field-for-field mirror of ``struct PaDecodeParams``."""
    _fields_ = (
        [("struct_size", C.c_uint32), ("abi_version", C.c_uint32)]
        + [(n, C.c_void_p) for n in (
            "out", "query", "key_cache", "value_cache", "block_tables", "context_lens",
            "query_scale", "key_scale", "value_scale", "alibi_slopes", "sink_tokens",
            "exp_sums", "max_logits", "tmp_out", "status", "trace", "merge_counters")]
        + [(n, C.c_int32) for n in (
            "num_seqs", "num_kv_heads", "query_group_size", "query_len", "head_size",
            "block_size", "num_blocks", "max_blocks_per_seq", "partition_size", "max_partitions")]
        + [(n, C.c_int64) for n in (
            "out_stride_seq", "out_stride_head", "q_stride_seq", "q_stride_head",
            "k_stride_block", "k_stride_head", "v_stride_block", "v_stride_head",
            "bt_stride_seq", "q_scale_stride_seq", "kv_scale_stride_block", "kv_scale_stride_head",
            "ws_stride_seq", "ws_stride_head", "ws_stride_part",
            "tmp_stride_seq", "tmp_stride_head", "tmp_stride_part", "tmp_stride_row")]
        + [(n, C.c_int32) for n in (
            "q_dtype", "kv_dtype", "out_dtype", "q_quant_mode", "kv_quant_mode", "v_layout")]
        + [("softmax_scale", C.c_float)]
        + [(n, C.c_int32) for n in ("tune_warps", "tune_stages", "tune_ctas", "tune_vstages", "tune_fuse", "tune_early")]
    )


class PaCacheWriteParams(C.Structure):
    """Field-for-field mirror of ``struct PaCacheWriteParams``."""
    _fields_ = (
        [("struct_size", C.c_uint32), ("abi_version", C.c_uint32)]
        + [(n, C.c_void_p) for n in ("key", "value", "slot_mapping", "key_cache", "value_cache",
                                     "key_scale", "value_scale", "status")]
        + [(n, C.c_int32) for n in ("num_tokens", "num_kv_heads", "head_size", "block_size", "num_blocks",
                                    "kv_dtype", "kv_quant_mode", "v_layout")]
        + [(n, C.c_int64) for n in ("key_stride_token", "key_stride_head", "value_stride_token", "value_stride_head",
                                    "k_stride_block", "k_stride_head", "v_stride_block", "v_stride_head",
                                    "kv_scale_stride_block", "kv_scale_stride_head")]
    )


class PaError(RuntimeError):
    """A non-zero PaStatus from the library."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().pa_strerror(status).decode()
        if status == -5:
            msg += f" [cudaError {lib().pa_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (status {status})")


_LIB = None


def lib() -> C.CDLL:
    """The loaded library; raises if it has not been built (``python -m triton_op_b200.build``)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.environ.get("PA_DECODE_LIB", LIB_PATH)      # a tuning build (e.g. with clock stamps) may be named here
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: the sm_100a CUDA library has not been built "
            "(run `python -m triton_op_b200.build`). There is no fallback path.")
    L = C.CDLL(path)
    P = C.POINTER(PaDecodeParams)
    L.pa_decode_sm100.argtypes = [P, C.c_void_p]
    L.pa_partition_sm100.argtypes = [P, C.c_void_p]
    L.pa_decode_noalloc_sm100.argtypes = [P, C.c_void_p]
    L.pa_reduce_sm100.argtypes = [P, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.pa_merge_triples_sm100.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    L.pa_merge_packed_triples_sm100.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                                C.c_void_p]
    L.pa_merge_packed_triples_sm100.restype = C.c_int
    L.pa_packed_triple_floats.argtypes = [C.c_int32, C.c_int32]
    L.pa_packed_triple_floats.restype = C.c_int64
    L.pa_query_launch_sm100.argtypes = [P] + [C.POINTER(C.c_int32)] * 4
    L.pa_exchange_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    L.pa_exchange_bytes.restype = C.c_int64
    L.pa_reduce_push_sm100.argtypes = [P, C.POINTER(C.c_void_p), C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]
    L.pa_reduce_push_sm100.restype = C.c_int
    L.pa_merge_wait_sm100.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_void_p]
    L.pa_merge_wait_sm100.restype = C.c_int
    L.pa_exchange_alloc.argtypes = [C.c_int64, C.POINTER(C.c_void_p), C.c_char_p]
    L.pa_exchange_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.pa_exchange_close.argtypes = [C.c_void_p]
    L.pa_exchange_free.argtypes = [C.c_void_p]
    for name in ("pa_exchange_alloc", "pa_exchange_open", "pa_exchange_close", "pa_exchange_free"):
        getattr(L, name).restype = C.c_int
    L.pa_cache_write_sm100.argtypes = [C.POINTER(PaCacheWriteParams), C.c_void_p]
    L.pa_cache_write_sm100.restype = C.c_int
    L.pa_stream_probe_sm100.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    L.pa_stream_probe_sm100.restype = C.c_int
    for name in ("pa_decode_sm100", "pa_decode_noalloc_sm100", "pa_partition_sm100", "pa_reduce_sm100",
                 "pa_merge_triples_sm100", "pa_query_launch_sm100", "pa_last_cuda_error",
                 "pa_abi_version"):
        getattr(L, name).restype = C.c_int
    L.pa_strerror.argtypes = [C.c_int]
    L.pa_strerror.restype = C.c_char_p
    if L.pa_abi_version() != PA_ABI_VERSION:
        raise ImportError("libpa_decode_sm100.so was built from a different ABI version; rebuild it")
    _LIB = L
    return L


def check(status: int, where: str) -> None:
    if status != PA_OK:
        raise PaError(status, where)
