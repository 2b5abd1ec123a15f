"""``paged_attention_decode`` -- the reference operator's Python surface over the sm_100a library.

Drop-in for ``paged_attention_decode`` of yanguahe/triton_op
(pa_decode_triton_gluon_fp8.py:1659-1897; the bf16-KV variant pa_decode_gluon.py:655-756 maps
onto the same call with ``query_sequence_length=1`` and ``query_scale=None``): same positional
arguments in the same order, same meaning, same returned dictionary keys.  Everything past
``alibi_slopes`` is keyword-only and new: the partition size (a module constant, 256, in the
reference) and the three workspaces, which the reference allocates and zero-fills on every call
(:1729-1733) and which a caller that cares about launch overhead passes in instead.

All tensors are torch CUDA tensors; the work is done by ``libpa_decode_sm100.so`` through its C
ABI (``include/pa_decode_sm100.h``) on torch's current stream.  No synchronisation, no copy and
(once the workspaces exist) no allocation happens in a call.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import PaDecodeParams

SEQUENCE_PARTITION_SIZE = 256  # pa_decode_triton_gluon_fp8.py:24
SUPPORTED_BLOCK_SIZES = (16, 64, 1024)  # pa_decode_triton_gluon_fp8.py:1747
FP8_DTYPE = torch.float8_e4m3fn  # OCP e4m3fn; the reference's AMD build uses e4m3fnuz


class PaArgumentError(AssertionError, ValueError):
    """Bad argument.  The reference signals these with ``assert`` (pa_decode_triton_gluon_fp8.py:
    1742-1790); deriving from both lets either style of caller catch it."""


def _fail(msg: str) -> None:
    raise PaArgumentError(msg)


def _inner_contiguous(t: torch.Tensor, first_dim: int) -> bool:
    """True when dims ``first_dim..`` of ``t`` are laid out densely (what ``t[0, 0].is_contiguous()``
    says for ``first_dim = 2``, without creating views)."""
    expect = 1
    shape, stride = t.shape, t.stride()
    for d in range(t.dim() - 1, first_dim - 1, -1):
        if shape[d] != 1 and stride[d] != expect:
            return False
        expect *= shape[d]
    return True


def _next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


_WORKSPACES: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
_SCALARS: Dict[Tuple, torch.Tensor] = {}


def get_workspaces(num_seqs: int, num_kv_heads: int, max_partitions: int, eq_group: int,
                   head_size: int, dtype: torch.dtype, device: torch.device
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(exp_sums, max_logits, tmp_output) of the reference's shapes, cached per shape and device.

    The reference makes these with ``torch.zeros`` on every call; the kernels here write every
    element the reduce reads, so the cached buffers are reused without clearing.
    """
    key = (num_seqs, num_kv_heads, max_partitions, eq_group, head_size, dtype, str(device))
    ws = _WORKSPACES.get(key)
    if ws is None:
        shape = (num_seqs, num_kv_heads, max_partitions, eq_group)
        ws = (torch.zeros(shape, dtype=torch.float32, device=device),
              torch.zeros(shape, dtype=torch.float32, device=device),
              torch.zeros(*shape, head_size, dtype=dtype, device=device))
        if len(_WORKSPACES) > 16:
            _WORKSPACES.clear()
        _WORKSPACES[key] = ws
    return ws


_COUNTERS: Dict[Tuple, torch.Tensor] = {}


def get_merge_counters(tmp_output: torch.Tensor, num_seqs: int, num_kv_heads: int) -> torch.Tensor:
    """The ``[num_seqs * num_kv_heads]`` int32 zeros that let a decode call run as one launch
    (``PaDecodeParams.merge_counters``), one array per workspace set: calls that share workspaces
    must not overlap anyway, and calls on different workspaces get different counters.  The kernel
    leaves them zero, so they are cleared only here, when they are made."""
    key = (str(tmp_output.device), tmp_output.data_ptr(), num_seqs * num_kv_heads)
    t = _COUNTERS.get(key)
    if t is None:
        if len(_COUNTERS) > 64:
            _COUNTERS.clear()       # blocks built earlier keep their own arrays alive
        t = torch.zeros(max(1, num_seqs * num_kv_heads), dtype=torch.int32, device=tmp_output.device)
        _COUNTERS[key] = t
    return t


def _scalar_on_device(value: float, device: torch.device) -> torch.Tensor:
    key = (float(value), str(device))
    t = _SCALARS.get(key)
    if t is None:
        if len(_SCALARS) > 256:
            _SCALARS.clear()
        t = torch.tensor(float(value), dtype=torch.float32, device=device)
        _SCALARS[key] = t
    return t


def _dtype_code(dt: torch.dtype, what: str) -> int:
    if dt == torch.bfloat16:
        return _lib.PA_DT_BF16
    if dt == FP8_DTYPE:
        return _lib.PA_DT_E4M3FN
    raise PaArgumentError(f"{what} tensor only support dtype in (torch.bfloat16, {FP8_DTYPE}), but got {dt}")


def _compute_type_matches(compute_type, out_dtype: torch.dtype) -> bool:
    """``compute_type`` is a Triton dtype in the reference (tl.bfloat16); torch dtypes and None are
    accepted too.  It must agree with the output dtype, which is what the kernels store."""
    if compute_type is None:
        return True
    if isinstance(compute_type, torch.dtype):
        return compute_type == out_dtype
    name = getattr(compute_type, "name", None) or str(compute_type)
    return {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "tl.bfloat16": torch.bfloat16,
            "fp16": torch.float16, "float16": torch.float16}.get(name, None) == out_dtype


def _kv_scale(scale, other, name: str, device) -> Tuple[Optional[torch.Tensor], int]:
    """Normalises a K or V scale argument to (tensor or None, PaQuantMode)."""
    if scale is None:
        return None, _lib.PA_QUANT_NONE
    if isinstance(scale, (int, float)):
        return _scalar_on_device(float(scale), device), _lib.PA_QUANT_PER_TENSOR
    if not (isinstance(scale, torch.Tensor) and scale.dtype == torch.float32):
        _fail(f"{name} tensor only support dtype == torch.float32, but got {name}.dtype == {getattr(scale, 'dtype', type(scale))}")
    if scale.dim() == 0 or scale.numel() == 1:
        return scale.reshape(()), _lib.PA_QUANT_PER_TENSOR
    if not (scale.dim() == 4):
        _fail(f"Expected 4D {name} tensor, but got shape {tuple(scale.shape)}")
    if not (scale.shape[-1] == 1):
        _fail(f"Expected {name}.shape[-1] == 1, but got {name}.shape[-1]={scale.shape[-1]}")
    return scale, _lib.PA_QUANT_PER_TOKEN


_PARAM_CACHE: Dict[tuple, PaDecodeParams] = {}


def _tensor_key(t) -> tuple:
    if t is None or not isinstance(t, torch.Tensor):
        return (t,)
    return (t.data_ptr(), t.shape, t.stride(), t.dtype)


def _params_key(output, query, key_cache, value_cache, sequence_lengths, block_tables, softmax_scale,
                query_sequence_length, max_sequence_length, compute_type, query_scale, key_scale, value_scale,
                alibi_slopes, partition_size, exp_sums, max_logits, tmp_output, status,
                sink_tokens=None) -> Optional[tuple]:
    """Everything the parameter block depends on: addresses, shapes, strides, dtypes, scalars.
    A decode loop calls with the same tensors every step, and validating them and filling the
    60-field block costs more host time than a small batch takes on the GPU."""
    try:
        return (str(output.device), float(softmax_scale), int(query_sequence_length), int(max_sequence_length),
                str(compute_type), int(partition_size)) + tuple(
            _tensor_key(t) for t in (output, query, key_cache, value_cache, sequence_lengths, block_tables,
                                     query_scale, key_scale, value_scale, alibi_slopes, exp_sums, max_logits,
                                     tmp_output, status, sink_tokens))
    except Exception:     # unexpected argument types: take the validating path, which reports them
        return None


def build_params(output, query, key_cache, value_cache, sequence_lengths, block_tables,
                 softmax_scale: float, query_sequence_length: int, max_sequence_length: int,
                 compute_type, query_scale, key_scale, value_scale, alibi_slopes,
                 partition_size: int, exp_sums, max_logits, tmp_output, status, tune, sink_tokens=None
                 ) -> Tuple[PaDecodeParams, tuple]:
    """Validated C parameter block for the arguments, from a small cache when the same tensors
    (addresses, shapes, strides, dtypes) and scalars were validated before."""
    key = None
    if tune is None:
        key = _params_key(output, query, key_cache, value_cache, sequence_lengths, block_tables, softmax_scale,
                          query_sequence_length, max_sequence_length, compute_type, query_scale, key_scale,
                          value_scale, alibi_slopes, partition_size, exp_sums, max_logits, tmp_output, status,
                          sink_tokens)
        hit = _PARAM_CACHE.get(key) if key is not None else None
        if hit is not None:
            p, ws = hit
            # a private copy: callers keep and edit their block (tuning sweeps, the no-allocation
            # entry point's tests), and the cached one must stay as validated
            return PaDecodeParams.from_buffer_copy(p), (output, query, key_cache, value_cache, sequence_lengths, block_tables, query_scale,
                       key_scale, value_scale, alibi_slopes) + ws[:3] + (status,) + ws[3:]
    p, keep, cacheable = _build_params(output, query, key_cache, value_cache, sequence_lengths, block_tables,
                                       softmax_scale, query_sequence_length, max_sequence_length, compute_type,
                                       query_scale, key_scale, value_scale, alibi_slopes, partition_size,
                                       exp_sums, max_logits, tmp_output, status, tune, sink_tokens)
    if key is not None and cacheable:
        if len(_PARAM_CACHE) >= 16:
            _PARAM_CACHE.clear()
        _PARAM_CACHE[key] = (PaDecodeParams.from_buffer_copy(p), keep[10:13] + keep[14:])    # the block, the workspaces and counters it points into
    return p, keep


def _build_params(output, query, key_cache, value_cache, sequence_lengths, block_tables,
                 softmax_scale: float, query_sequence_length: int, max_sequence_length: int,
                 compute_type, query_scale, key_scale, value_scale, alibi_slopes,
                 partition_size: int, exp_sums, max_logits, tmp_output, status, tune, sink_tokens=None
                 ) -> Tuple[PaDecodeParams, tuple, bool]:
    """Validates the arguments as the reference does and fills the C parameter block.

    Returns the block, a tuple of the tensors it points into (keep it alive across the call) and
    whether the block points only at the caller's tensors and the cached workspaces (then it
    may be reused for the same arguments).
    """
    given = (query, sequence_lengths, block_tables, query_scale, key_scale, value_scale)
    if not (isinstance(output, torch.Tensor)):
        _fail("output must be a torch.Tensor")
    dev = output.device
    if not (len(output.shape) == 3):
        _fail(f"Expected 3D output tensor, but got shape {tuple(output.shape)}")
    if not (len(query.shape) == 3):
        _fail(f"Expected 3D query tensor, but got shape {tuple(query.shape)}")
    if not (len(key_cache.shape) == 5):
        _fail(f"Expected 5D key_cache tensor, but got shape {tuple(key_cache.shape)}")
    if len(value_cache.shape) == 5:
        v_layout = _lib.PA_V_TRANSPOSED
    elif len(value_cache.shape) == 4:
        v_layout = _lib.PA_V_NORMAL
    else:
        raise RuntimeError(f"Unsupported value cache shape: {tuple(value_cache.shape)}")
    if not (output.dtype == torch.bfloat16):
        _fail(f"output tensor only support dtype == torch.bfloat16, but got output.dtype == {output.dtype}")
    if not (_compute_type_matches(compute_type, output.dtype)):
        _fail(f"compute_type {compute_type} disagrees with output.dtype {output.dtype}")
    q_dtype = _dtype_code(query.dtype, "query")
    kv_dtype = _dtype_code(key_cache.dtype, "key_cache")
    if not (value_cache.dtype == key_cache.dtype):
        _fail(f"value_cache.dtype {value_cache.dtype} != key_cache.dtype {key_cache.dtype}")
    for name, t in (("query", query), ("key_cache", key_cache), ("value_cache", value_cache),
                    ("sequence_lengths", sequence_lengths), ("block_tables", block_tables)):
        if not (t.device == dev):
            _fail(f"{name} must live on {dev}, the output's device")
    if not (sequence_lengths.dtype == torch.int32 and block_tables.dtype == torch.int32):
        _fail("sequence_lengths and block_tables must be int32")
    if not (query_sequence_length >= 1):
        _fail("query_sequence_length must be >= 1")
    if not (query_sequence_length <= 4):
        _fail(f"QUERY_SEQ_LEN={query_sequence_length}, Only support QUERY_SEQ_LEN <= 4")

    num_seqs, q_heads_total, head_size = query.shape
    if not (tuple(output.shape) == tuple(query.shape)):
        _fail("output and query must have the same shape")
    num_blocks, num_kv_heads = key_cache.shape[0], key_cache.shape[1]
    kv_block_size = key_cache.shape[-2]
    x = 16 // key_cache.element_size()
    if not (key_cache.shape[2] * key_cache.shape[4] == head_size and key_cache.shape[4] == x):
        _fail(f"key_cache must be [num_blocks, num_kv_heads, head_size/{x}, block_size, {x}]")
    if not (kv_block_size in SUPPORTED_BLOCK_SIZES):
        _fail(f"kv_block_size == {kv_block_size} not in {list(SUPPORTED_BLOCK_SIZES)}")
    heads_per_token = q_heads_total // query_sequence_length
    if not (heads_per_token * query_sequence_length == q_heads_total and heads_per_token % num_kv_heads == 0):
        _fail("query heads must be num_kv_heads * query_sequence_length * group_size")
    group = heads_per_token // num_kv_heads
    eq_group = group * query_sequence_length
    eq_group_pow2 = 16 if eq_group <= 16 else _next_pow2(eq_group)
    if not (eq_group_pow2 <= 64):
        _fail(f"equivalent_query_group_size_pow2={eq_group_pow2} exceeds maximum of 64")
    if v_layout == _lib.PA_V_NORMAL:
        if not (tuple(value_cache.shape) == (num_blocks, num_kv_heads, head_size, kv_block_size)):
            _fail("value_cache must be [num_blocks, num_kv_heads, head_size, block_size]")
    else:   # transposed: [num_blocks, num_kv_heads, block_size/x, head_size, x] (test_pa_mtp.py:472-497)
        if not (tuple(value_cache.shape) == (num_blocks, num_kv_heads, kv_block_size // x, head_size, x)):
            _fail(f"transposed value_cache must be [num_blocks, num_kv_heads, block_size/{x}, head_size, {x}]")
    if not (block_tables.dim() == 2 and block_tables.shape[0] == num_seqs and sequence_lengths.numel() == num_seqs):
        _fail("block_tables must be [num_seqs, max_blocks] and sequence_lengths [num_seqs]")
    if not (partition_size > 0 and (partition_size % kv_block_size == 0 or kv_block_size % partition_size == 0)):
        _fail("partition_size and block_size must divide one another")

    if query.stride(-1) != 1 or query.stride(1) != head_size:
        query = query.contiguous()
    if not (output.stride(-1) == 1):
        _fail("output's last dim must be contiguous")
    if not (_inner_contiguous(key_cache, 2) and _inner_contiguous(value_cache, 2)):
        _fail("the per-(block, head) slabs of the KV caches must be contiguous")
    if sequence_lengths.stride(0) != 1:
        sequence_lengths = sequence_lengths.contiguous()
    if block_tables.stride(1) != 1:
        block_tables = block_tables.contiguous()

    # ---- quantisation modes (pa_decode_triton_gluon_fp8.py:1752-1790)
    q_scale_t, q_mode, q_scale_stride = None, _lib.PA_QUANT_NONE, 0
    if query_scale is not None:
        if isinstance(query_scale, (int, float)):
            q_scale_t, q_mode = _scalar_on_device(float(query_scale), dev), _lib.PA_QUANT_PER_TENSOR
        else:
            if not (isinstance(query_scale, torch.Tensor) and query_scale.dtype == torch.float32):
                _fail(f"query_scale tensor only support dtype == torch.float32, but got query_scale.dtype == {getattr(query_scale, 'dtype', None)}")
            if query_scale.dim() == 0:
                q_scale_t, q_mode = query_scale, _lib.PA_QUANT_PER_TENSOR
            else:
                if not (query_scale.dim() == 3):
                    _fail(f"Expected 3D query_scale tensor, but got shape {tuple(query_scale.shape)}")
                if not (query_scale.shape[-1] == 1):
                    _fail(f"Expected query_scale.shape[-1] == 1, but got query_scale.shape[-1]={query_scale.shape[-1]}")
                q_scale_t = query_scale if query_scale.stride(1) == 1 else query_scale.contiguous()
                q_mode, q_scale_stride = _lib.PA_QUANT_PER_TOKEN, q_scale_t.stride(0)
    k_scale_t, kv_mode = None, _lib.PA_QUANT_NONE
    v_scale_t = None
    if key_scale is not None and value_scale is not None:
        k_scale_t, kv_mode = _kv_scale(key_scale, value_scale, "key_scale", dev)
        v_scale_t, v_mode = _kv_scale(value_scale, key_scale, "value_scale", dev)
        if not (kv_mode == v_mode and tuple(k_scale_t.shape) == tuple(v_scale_t.shape)):
            _fail(f"Key and value scales must have same shape, but got key: {tuple(k_scale_t.shape)}, value: {tuple(v_scale_t.shape)}")
        if kv_mode == _lib.PA_QUANT_PER_TOKEN:
            if not (tuple(k_scale_t.shape[:3]) == (num_blocks, num_kv_heads, kv_block_size)):
                _fail("per-token kv scales must be [num_blocks, num_kv_heads, block_size, 1]")
            if not (k_scale_t.stride(2) == 1 and v_scale_t.stride(2) == 1 and k_scale_t.stride() == v_scale_t.stride()):
                _fail("per-token kv scales must be contiguous along block_size and share strides")

    # ---- workspaces
    # The tcgen05 kernel works on 256-token partitions.  A larger partition size that is a multiple
    # of 256 is run as 256-token sub-partitions when the workspaces are the operator's own (their
    # layout is then nobody else's business; the output is the same attention, split finer).
    # Workspaces passed by the caller keep the layout the caller asked for.
    own_workspaces = exp_sums is None and max_logits is None and tmp_output is None
    if (own_workspaces and partition_size > SEQUENCE_PARTITION_SIZE and partition_size % SEQUENCE_PARTITION_SIZE == 0
            and kv_dtype == _lib.PA_DT_E4M3FN and not (tune and tune.get("warps"))):
        partition_size = SEQUENCE_PARTITION_SIZE
    max_partitions = max(1, (int(max_sequence_length) + partition_size - 1) // partition_size)
    if exp_sums is None or max_logits is None or tmp_output is None:
        ws = get_workspaces(num_seqs, num_kv_heads, max_partitions, eq_group, head_size, output.dtype, dev)
        exp_sums = ws[0] if exp_sums is None else exp_sums
        max_logits = ws[1] if max_logits is None else max_logits
        tmp_output = ws[2] if tmp_output is None else tmp_output
    ws_shape = (num_seqs, num_kv_heads, max_partitions, eq_group)
    for name, t, dt in (("exp_sums", exp_sums, torch.float32), ("max_logits", max_logits, torch.float32)):
        if not (t.dtype == dt and t.dim() == 4 and t.shape[0] == num_seqs and t.shape[1] == num_kv_heads and t.shape[2] >= max_partitions and t.shape[3] == eq_group and t.stride(3) == 1 and t.device == dev):
            _fail(f"{name} must be fp32 [num_seqs, num_kv_heads, >=max_partitions, eq_group] = {ws_shape}")
    if not (exp_sums.stride() == max_logits.stride()):
        _fail("exp_sums and max_logits must share strides")
    if not (tmp_output.dtype == output.dtype and tmp_output.dim() == 5 and tuple(tmp_output.shape[:2]) == ws_shape[:2] and tmp_output.shape[2] >= max_partitions and tuple(tmp_output.shape[3:]) == (eq_group, head_size) and tmp_output.stride(4) == 1 and tmp_output.device == dev):
        _fail(f"tmp_output must be {output.dtype} {ws_shape + (head_size,)}")

    p = PaDecodeParams()
    p.struct_size = C.sizeof(PaDecodeParams)
    p.abi_version = _lib.PA_ABI_VERSION
    p.out, p.query = output.data_ptr(), query.data_ptr()
    p.key_cache, p.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    p.block_tables, p.context_lens = block_tables.data_ptr(), sequence_lengths.data_ptr()
    p.query_scale = q_scale_t.data_ptr() if q_scale_t is not None else None
    p.key_scale = k_scale_t.data_ptr() if k_scale_t is not None else None
    p.value_scale = v_scale_t.data_ptr() if v_scale_t is not None else None
    if alibi_slopes is not None:
        if not (isinstance(alibi_slopes, torch.Tensor) and alibi_slopes.dtype == torch.float32 and alibi_slopes.device == dev
                and alibi_slopes.numel() == num_kv_heads * group and alibi_slopes.is_contiguous()):
            _fail("alibi_slopes must be a contiguous fp32 tensor with one slope per query head on the output's device")
    p.alibi_slopes = alibi_slopes.data_ptr() if alibi_slopes is not None else None
    if sink_tokens is not None:
        if not (isinstance(sink_tokens, torch.Tensor) and sink_tokens.dtype == torch.float32 and sink_tokens.device == dev
                and sink_tokens.numel() == num_kv_heads * group and sink_tokens.is_contiguous()):
            _fail("sink_tokens must be a contiguous fp32 tensor with one logit per query head on the output's device")
        p.sink_tokens = sink_tokens.data_ptr()
    p.exp_sums, p.max_logits, p.tmp_out = exp_sums.data_ptr(), max_logits.data_ptr(), tmp_output.data_ptr()
    p.status = status.data_ptr() if status is not None else None
    counters = None
    if tune and tune.get("fuse", 0) > 0 and num_seqs > 0:
        counters = get_merge_counters(tmp_output, num_seqs, num_kv_heads)
        p.merge_counters = counters.data_ptr()
    p.trace = tune["trace"].data_ptr() if tune and tune.get("trace") is not None else None
    p.num_seqs, p.num_kv_heads, p.query_group_size = num_seqs, num_kv_heads, group
    p.query_len, p.head_size, p.block_size = query_sequence_length, head_size, kv_block_size
    p.num_blocks, p.max_blocks_per_seq = num_blocks, block_tables.shape[1]
    p.partition_size, p.max_partitions = partition_size, max_partitions
    p.out_stride_seq, p.out_stride_head = output.stride(0), output.stride(1)
    p.q_stride_seq, p.q_stride_head = query.stride(0), query.stride(1)
    p.k_stride_block, p.k_stride_head = key_cache.stride(0), key_cache.stride(1)
    p.v_stride_block, p.v_stride_head = value_cache.stride(0), value_cache.stride(1)
    p.bt_stride_seq = block_tables.stride(0)
    p.q_scale_stride_seq = q_scale_stride
    if kv_mode == _lib.PA_QUANT_PER_TOKEN:
        p.kv_scale_stride_block, p.kv_scale_stride_head = k_scale_t.stride(0), k_scale_t.stride(1)
    p.ws_stride_seq, p.ws_stride_head, p.ws_stride_part = exp_sums.stride(0), exp_sums.stride(1), exp_sums.stride(2)
    p.tmp_stride_seq, p.tmp_stride_head = tmp_output.stride(0), tmp_output.stride(1)
    p.tmp_stride_part, p.tmp_stride_row = tmp_output.stride(2), tmp_output.stride(3)
    p.q_dtype, p.kv_dtype, p.out_dtype = q_dtype, kv_dtype, _lib.PA_DT_BF16
    p.q_quant_mode, p.kv_quant_mode, p.v_layout = q_mode, kv_mode, v_layout
    p.softmax_scale = float(softmax_scale)
    if tune:
        p.tune_warps = int(tune.get("warps", 0))
        p.tune_stages = int(tune.get("stages", 0))
        p.tune_ctas = int(tune.get("ctas", 0))
        p.tune_vstages = int(tune.get("vstages", 0))
        p.tune_fuse = int(tune.get("fuse", 0))
        p.tune_early = int(tune.get("early", 0))
    keep = (output, query, key_cache, value_cache, sequence_lengths, block_tables, q_scale_t, k_scale_t,
            v_scale_t, alibi_slopes, exp_sums, max_logits, tmp_output, status, counters)
    # copies made above (contiguous query, device scalars for Python-float scales) belong to this call
    used = (query, sequence_lengths, block_tables, q_scale_t, k_scale_t, v_scale_t)
    cacheable = all(u is g or (isinstance(u, torch.Tensor) and isinstance(g, torch.Tensor)
                               and u.data_ptr() == g.data_ptr()) for u, g in zip(used, given))
    return p, keep, cacheable


def paged_attention_decode(
    output: torch.Tensor,            # [num_seqs, num_kv_heads * query_len * group, head_size] bf16
    query: torch.Tensor,             # same shape; bf16 (or e4m3fn with query_scale)
    key_cache: torch.Tensor,         # [num_blocks, num_kv_heads, head_size/x, block_size, x]
    value_cache: torch.Tensor,       # [num_blocks, num_kv_heads, head_size, block_size]
    sequence_lengths: torch.Tensor,  # [num_seqs] int32
    block_tables: torch.Tensor,      # [num_seqs, max_blocks_per_seq] int32
    softmax_scale: float,
    query_sequence_length: int,
    max_sequence_length: int,
    compute_type,
    query_scale: Optional[torch.Tensor],
    key_scale: Optional[torch.Tensor],
    value_scale: Optional[torch.Tensor],
    num_sequence_partitions: int = 0,
    alibi_slopes: Optional[torch.Tensor] = None,
    *,
    partition_size: int = SEQUENCE_PARTITION_SIZE,
    exp_sums: Optional[torch.Tensor] = None,
    max_logits: Optional[torch.Tensor] = None,
    tmp_output: Optional[torch.Tensor] = None,
    status: Optional[torch.Tensor] = None,
    time_kernels: bool = False,
    sink_tokens: Optional[torch.Tensor] = None,
    tune: Optional[dict] = None,
) -> Dict:
    """Paged-attention decode with a split-KV partition pass and a log-sum-exp reduce.

    Arguments up to ``alibi_slopes`` are the reference's (pa_decode_triton_gluon_fp8.py:1659-1675).
    ``max_sequence_length`` only sizes the partition axis of the workspaces, as there.
    ``num_sequence_partitions`` is accepted and unused, as there.  Scales: ``None``, a 0-dim fp32
    CUDA tensor (per tensor) or ``[num_blocks, num_kv_heads, block_size, 1]`` fp32 (per token and
    head); a Python float is accepted for per-tensor scales like the bf16 reference entry does.

    Keyword-only additions: ``partition_size`` (reference constant 256); ``exp_sums`` /
    ``max_logits`` ``[num_seqs, num_kv_heads, P, eq_group]`` fp32 and ``tmp_output``
    ``[..., eq_group, head_size]`` in the output dtype, with ``P >= ceil(max_sequence_length /
    partition_size)`` -- when omitted they come from a per-shape cache, so the tensors in the
    returned dictionary are overwritten by the next call of the same shape; ``status``: optional
    int32 CUDA scalar the kernels OR ``PA_DEV_*`` bits into; ``time_kernels``: measure the two
    kernels with CUDA events (synchronises; off by default so the call stays asynchronous);
    ``sink_tokens``: fp32 ``[query heads]`` sink logits whose weight ``exp(sink - max)`` joins every
    row's softmax denominator in the reduce (the reference's unused Gluon reduce,
    pa_decode_triton_gluon_fp8.py:1117-1123).

    Returns the reference's dictionary (:1889-1897): ``triton_decode_time``,
    ``triton_reduce_time``, ``total_triton_time`` (microseconds; 0.0 unless ``time_kernels``),
    ``temporary_output``, ``final_output``, ``exponential_sums``, ``maximum_logits``; plus
    ``partition_size``, the split the returned workspaces hold: a requested multiple of 256 runs
    as 256-token sub-partitions unless the caller passed workspaces of its own.

    ``tune={"fuse": 1}`` runs the call as ONE launch where the shape allows it (e4m3fn KV, 256-token
    partitions, at most 8 query rows per kv head, at most 32 partitions, no ALiBi): work items are
    numbered so that a CTA computes all partitions of most (sequence, kv head) sets and merges
    them itself, instead of the reference's second launch (pa_decode_triton_gluon_fp8.py:
    1862-1887); ``1 + T`` asks for teams of T CTAs per (sequence, partition) row.  Bit-identical
    to the default two-launch form, and measured slower than it (that numbering reads the cache
    slower than the round-robin one, by more than the second launch costs), so it is opt-in.
    """
    p, keep = build_params(output, query, key_cache, value_cache, sequence_lengths, block_tables,
                           softmax_scale, query_sequence_length, max_sequence_length, compute_type,
                           query_scale, key_scale, value_scale, alibi_slopes, partition_size,
                           exp_sums, max_logits, tmp_output, status, tune, sink_tokens)
    if not output.is_cuda:
        raise RuntimeError("paged_attention_decode runs on CUDA tensors only; there is no CPU fallback")
    L = _lib.lib()
    decode_us = reduce_us = 0.0
    with torch.cuda.device(output.device):
        stream = torch.cuda.current_stream().cuda_stream
        if not time_kernels:
            _lib.check(L.pa_decode_sm100(C.byref(p), stream), "pa_decode_sm100")
        else:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record()
            _lib.check(L.pa_partition_sm100(C.byref(p), stream), "pa_partition_sm100")
            ev[1].record()
            _lib.check(L.pa_reduce_sm100(C.byref(p), None, None, None, stream), "pa_reduce_sm100")
            ev[2].record()
            ev[2].synchronize()
            decode_us = ev[0].elapsed_time(ev[1]) * 1e3
            reduce_us = ev[1].elapsed_time(ev[2]) * 1e3
    return {
        "triton_decode_time": decode_us,
        "triton_reduce_time": reduce_us,
        "temporary_output": keep[12],
        "final_output": output,
        "exponential_sums": keep[10],
        "maximum_logits": keep[11],
        "total_triton_time": decode_us + reduce_us,
        "partition_size": int(p.partition_size),   # the split the workspaces hold (256 for multiples of 256)
    }


def query_launch(*args, **kwargs) -> Dict[str, int]:
    """Grid, CTA size, dynamic shared memory and ring depth the partition kernel would use for the
    given ``paged_attention_decode`` arguments (nothing is launched)."""
    kwargs.pop("time_kernels", None)
    names = ("output", "query", "key_cache", "value_cache", "sequence_lengths", "block_tables",
             "softmax_scale", "query_sequence_length", "max_sequence_length", "compute_type",
             "query_scale", "key_scale", "value_scale", "num_sequence_partitions", "alibi_slopes")
    a = dict(zip(names, args))
    a.update(kwargs)
    p, _keep = build_params(a["output"], a["query"], a["key_cache"], a["value_cache"], a["sequence_lengths"],
                            a["block_tables"], a["softmax_scale"], a["query_sequence_length"],
                            a["max_sequence_length"], a.get("compute_type"), a.get("query_scale"),
                            a.get("key_scale"), a.get("value_scale"), a.get("alibi_slopes"),
                            a.get("partition_size", SEQUENCE_PARTITION_SIZE), a.get("exp_sums"),
                            a.get("max_logits"), a.get("tmp_output"), a.get("status"), a.get("tune"))
    vals = [C.c_int32(0) for _ in range(4)]
    with torch.cuda.device(a["output"].device):
        _lib.check(_lib.lib().pa_query_launch_sm100(C.byref(p), *[C.byref(v) for v in vals]),
                   "pa_query_launch_sm100")
    return {"grid_ctas": vals[0].value, "cta_threads": vals[1].value,
            "smem_bytes": vals[2].value, "ring_stages": vals[3].value}
