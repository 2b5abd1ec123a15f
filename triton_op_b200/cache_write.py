"""KV-cache write side: new key / value tokens into the paged caches the decode operator reads.

The reference prepares its caches offline (layouts: test_pa_mtp.py:109-172; per-token e4m3
quantisation ``quantize_kv_cache_symmetric``: :294-369).  A serving loop does the same for the
tokens of every step; :func:`write_kv_cache` is that step as one CUDA kernel
(``pa_cache_write_sm100``): quantise and scatter, no intermediate tensors.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .pa_decode import FP8_DTYPE, PaArgumentError

__all__ = ["write_kv_cache", "slots_for"]


def slots_for(block_tables: torch.Tensor, positions: torch.Tensor, seq_ids: torch.Tensor, block_size: int) -> torch.Tensor:
    """Slot (``block * block_size + offset``) of token ``positions[i]`` of sequence ``seq_ids[i]``."""
    blocks = block_tables[seq_ids.long(), (positions // block_size).long()].long()
    return blocks * block_size + (positions % block_size).long()


def write_kv_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                   slot_mapping: torch.Tensor, key_scale: Optional[torch.Tensor] = None,
                   value_scale: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """Writes ``key`` / ``value`` ``[T, Hkv, D]`` bf16 into the paged caches at ``slot_mapping [T]`` (int64).

    Caches: keys ``[NB, Hkv, D/x, bs, x]``, values ``[NB, Hkv, D, bs]`` or transposed
    ``[NB, Hkv, bs/16, D, 16]``; bf16 (bits copied, no scales) or e4m3fn.  For e4m3fn caches the
    scales select the mode: 0-dim fp32 tensors are per-tensor scales that are READ
    (``q = x / scale``); ``[NB, Hkv, bs, 1]`` fp32 tensors receive the per-token scales
    ``max(amax / 448, 1e-12)`` of the written tokens; ``None`` stores ``x`` unscaled.
    Negative slots are skipped.  Runs on the current stream; there is no CPU fallback.
    """
    if not (key.is_cuda and value.is_cuda and key_cache.is_cuda and value_cache.is_cuda):
        raise RuntimeError("write_kv_cache runs on CUDA tensors only; there is no CPU fallback")
    if key.dtype != torch.bfloat16 or value.dtype != torch.bfloat16 or key.shape != value.shape or key.dim() != 3:
        raise PaArgumentError("key and value must be bf16 [num_tokens, num_kv_heads, head_size] of one shape")
    if key_cache.dim() != 5 or value_cache.dim() not in (4, 5) or value_cache.dtype != key_cache.dtype:
        raise PaArgumentError("key_cache must be 5-D, value_cache 4-D or 5-D, of one dtype")
    T, hkv, d = key.shape
    nb, bs = key_cache.shape[0], key_cache.shape[3]
    x = 16 // key_cache.element_size()
    if tuple(key_cache.shape) != (nb, hkv, d // x, bs, x):
        raise PaArgumentError(f"key_cache must be [num_blocks, {hkv}, {d // x}, block_size, {x}]")
    trans = value_cache.dim() == 5
    want_v = (nb, hkv, bs // x, d, x) if trans else (nb, hkv, d, bs)
    if tuple(value_cache.shape) != want_v:
        raise PaArgumentError(f"value_cache must be {want_v}")
    if key_cache.dtype == torch.bfloat16:
        kv_dtype, mode = _lib.PA_DT_BF16, _lib.PA_QUANT_NONE
        if key_scale is not None or value_scale is not None:
            raise PaArgumentError("bf16 caches take no scales")
    elif key_cache.dtype == FP8_DTYPE:
        kv_dtype = _lib.PA_DT_E4M3FN
        if (key_scale is None) != (value_scale is None):
            raise PaArgumentError("key_scale and value_scale go together")
        if key_scale is None:
            mode = _lib.PA_QUANT_NONE
        elif key_scale.dim() == 0 and value_scale.dim() == 0:
            mode = _lib.PA_QUANT_PER_TENSOR
        elif tuple(key_scale.shape) == (nb, hkv, bs, 1) and tuple(value_scale.shape) == (nb, hkv, bs, 1):
            mode = _lib.PA_QUANT_PER_TOKEN
            if key_scale.stride(2) != 1 or value_scale.stride() != key_scale.stride():
                raise PaArgumentError("per-token scales must be contiguous along block_size and share strides")
        else:
            raise PaArgumentError("scales must be 0-dim (per tensor) or [num_blocks, num_kv_heads, block_size, 1]")
        for s in (key_scale, value_scale):
            if s is not None and (s.dtype != torch.float32 or not s.is_cuda):
                raise PaArgumentError("scales must be fp32 CUDA tensors")
    else:
        raise PaArgumentError(f"unsupported cache dtype {key_cache.dtype}")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != T or not slot_mapping.is_cuda:
        raise PaArgumentError("slot_mapping must be an int64 CUDA tensor with one entry per token")
    if key.stride(2) != 1:
        key = key.contiguous()
    if value.stride(2) != 1:
        value = value.contiguous()
    slot_mapping = slot_mapping.contiguous()

    p = _lib.PaCacheWriteParams()
    p.struct_size = C.sizeof(_lib.PaCacheWriteParams)
    p.abi_version = _lib.PA_ABI_VERSION
    p.key, p.value, p.slot_mapping = key.data_ptr(), value.data_ptr(), slot_mapping.data_ptr()
    p.key_cache, p.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    p.key_scale = key_scale.data_ptr() if key_scale is not None else None
    p.value_scale = value_scale.data_ptr() if value_scale is not None else None
    p.status = status.data_ptr() if status is not None else None
    p.num_tokens, p.num_kv_heads, p.head_size, p.block_size, p.num_blocks = T, hkv, d, bs, nb
    p.kv_dtype, p.kv_quant_mode = kv_dtype, mode
    p.v_layout = _lib.PA_V_TRANSPOSED if trans else _lib.PA_V_NORMAL
    p.key_stride_token, p.key_stride_head = key.stride(0), key.stride(1)
    p.value_stride_token, p.value_stride_head = value.stride(0), value.stride(1)
    p.k_stride_block, p.k_stride_head = key_cache.stride(0), key_cache.stride(1)
    p.v_stride_block, p.v_stride_head = value_cache.stride(0), value_cache.stride(1)
    if mode == _lib.PA_QUANT_PER_TOKEN:
        p.kv_scale_stride_block, p.kv_scale_stride_head = key_scale.stride(0), key_scale.stride(1)
    with torch.cuda.device(key.device):
        _lib.check(_lib.lib().pa_cache_write_sm100(C.byref(p), torch.cuda.current_stream().cuda_stream),
                   "pa_cache_write_sm100")
