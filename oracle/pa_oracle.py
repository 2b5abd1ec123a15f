"""CPU oracle for paged-attention decode.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py`` (its CPU-baseline legs, where this
module is what gets timed on host cores, and its parity checks of sampled sequences, where it is
the checker, outside every timed region) may import this module; the shipped operator
(``triton_op_b200``) never does.

It restates, in plain torch ops that run on CPU tensors (fp32 arithmetic), the pure-PyTorch
paged-attention path of yanguahe/triton_op, which is that repository's own correctness
reference:

* ``masked_attention``          <- test_pa_mtp.py:175-220  (reference_masked_attention)
* ``paged_attention``           <- test_pa_mtp.py:223-291  (torch_mha_extend)
* ``split_kv_partials`` /
  ``merge_partials``            <- the split-KV semantics of
                                   pa_decode_triton_gluon_fp8.py:514-1002 (partition kernel: m, l,
                                   normalised partial output per 256-token partition) and
                                   :1187-1333 (reduce kernel), in exact fp32 instead of fp8 MFMA.
* ``compare_arrays``            <- utils.py:5-106 (the reference's error metrics)

Parity pin: ``tests/golden/*.npz`` hold outputs of the reference's own two functions, loaded
from the reference checkout by ``tests/golden/make_golden.py`` and run on CPU; the CPU test
suite checks this module against them bit for bit (same torch ops in the same order), so the
oracle is pinned to the reference, not merely to itself.  The ALiBi bias and the split-KV
intermediates, which that PyTorch path does not have, are pinned by ``tests/golden/triton_*.npz``:
outputs of the reference's plain-Triton decode (pa_decode_triton.py:523-685) run on CPU under the
Triton interpreter by ``tests/golden/make_golden_triton.py`` (fp16 arithmetic there, so the
comparison has an fp16-level tolerance, stated in the test).  Sink tokens exist only in a Gluon
reduce kernel the reference never launches: parity of ``sink_tokens`` is unpinned by the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


def masked_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                     softmax_scale: float, output_dtype: torch.dtype,
                     is_causal: bool = True, alibi_slopes: Optional[torch.Tensor] = None,
                     sink_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of ``query [q, Hq, D]`` over ``key/value [k, Hkv, D]`` (test_pa_mtp.py:175-220).

    KV heads are repeated to the query heads, scores are fp32, the causal rule lets query row i
    (of q) see keys ``j <= i + (k - q)``: the cache already holds the q new tokens at its end.
    """
    hq, hkv = query.shape[1], key.shape[1]
    key = key.repeat_interleave(hq // hkv, dim=1)
    value = value.repeat_interleave(hq // hkv, dim=1)
    scores = torch.einsum("qhd,khd->hqk", query.float(), key.float()) * softmax_scale
    if alibi_slopes is not None:
        # the kernels' bias, pa_decode_triton_gluon_fp8.py:905-908: slope[head] * (key position - (context - 1)),
        # added to the scaled scores.  (The reference's PyTorch path has no ALiBi and its tests never pass
        # slopes; the Gluon kernel loads slopes for the first G rows of a kv head only, which leaves the later
        # MTP tokens without bias -- here every row of a head gets its head's slope.)
        kl = key.shape[0]
        rel = torch.arange(kl, dtype=torch.float32, device=query.device) - (kl - 1)
        scores = scores + alibi_slopes.float().view(-1, 1, 1) * rel.view(1, 1, -1)
    if is_causal:
        ql, kl = query.shape[0], key.shape[0]
        bias = torch.zeros(ql, kl, dtype=query.dtype, device=query.device)
        keep = torch.ones(ql, kl, dtype=torch.bool, device=query.device).tril(diagonal=kl - ql)
        bias.masked_fill_(keep.logical_not(), float("-inf"))
        scores += bias
    if sink_tokens is None:
        weights = torch.softmax(scores, dim=-1)
    else:
        # sink token per head: a weight exp(sink - max) in the denominator that carries no value
        # (pa_decode_triton_gluon_fp8.py:1117-1123; the maximum is that of the real keys)
        mx = scores.amax(dim=-1, keepdim=True)
        e = torch.exp(scores - mx)
        denom = e.sum(dim=-1, keepdim=True) + torch.exp(sink_tokens.float().view(-1, 1, 1) - mx)
        weights = e / denom
    out = torch.einsum("hqk,khd->qhd", weights.float(), value.float())
    return out.to(output_dtype)


def flatten_caches(key_cache: torch.Tensor, value_cache: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """[NB,Hkv,D/x,bs,x] / [NB,Hkv,D,bs] -> token-major [NB*bs, Hkv, D] (test_pa_mtp.py:259-260)."""
    nb, hkv, d, bs = value_cache.shape
    k_flat = key_cache.permute(0, 3, 1, 2, 4).contiguous().view(-1, hkv, d)
    v_flat = value_cache.permute(0, 3, 1, 2).contiguous().view(-1, hkv, d)
    return k_flat, v_flat


def gather_sequence(k_flat: torch.Tensor, v_flat: torch.Tensor, block_table: torch.Tensor,
                    context_len: int, block_size: int,
                    key_scale: Optional[torch.Tensor], value_scale: Optional[torch.Tensor]
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dequantised fp32 keys / values ``[ctx, Hkv, D]`` of one sequence (test_pa_mtp.py:270-283).

    ``key_scale`` / ``value_scale`` are the flat per-token form ``[Hkv, NB*bs]`` fp32 or None.
    """
    kv_dtype = k_flat.dtype
    token_idx = (block_table.repeat_interleave(block_size)[:context_len] * block_size
                 + torch.arange(context_len, device=block_table.device) % block_size)
    keys = k_flat.view(torch.int8)[token_idx].view(kv_dtype).to(torch.float)
    if key_scale is not None:
        keys *= key_scale[:, token_idx].t().unsqueeze(-1)
    values = v_flat.view(torch.int8)[token_idx].view(kv_dtype).to(torch.float)
    if value_scale is not None:
        values *= value_scale[:, token_idx].t().unsqueeze(-1)
    return keys, values


def paged_attention(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                    block_tables: torch.Tensor, context_lens: torch.Tensor,
                    query_indptr: torch.Tensor,
                    key_scale: Optional[torch.Tensor] = None,
                    value_scale: Optional[torch.Tensor] = None,
                    alibi_slopes: Optional[torch.Tensor] = None,
                    sink_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The reference's paged multi-head attention (test_pa_mtp.py:223-291).

    query ``[total_q, Hq, D]`` split per sequence by ``query_indptr [S+1]``; caches in the paged
    layouts; scales flat ``[Hkv, NB*bs]`` or None.  softmax_scale is fixed at ``1/sqrt(D)`` as in
    the reference (:250).  Returns ``[total_q, Hq, D]`` in the query dtype.
    """
    nb, hkv, d, bs = value_cache.shape
    softmax_scale = 1.0 / (d ** 0.5)
    out_dtype = query.dtype
    q_split = torch.tensor_split(query, query_indptr.tolist()[1:])
    k_flat, v_flat = flatten_caches(key_cache, value_cache)
    outs = []
    for s in range(query_indptr.shape[0] - 1):
        ctx = int(context_lens[s].item())
        keys, values = gather_sequence(k_flat, v_flat, block_tables[s], ctx, bs, key_scale, value_scale)
        outs.append(masked_attention(q_split[s], keys, values, softmax_scale, out_dtype, is_causal=True,
                                     alibi_slopes=alibi_slopes, sink_tokens=sink_tokens))
    return torch.cat(outs)


def split_kv_partials(query: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                      block_tables: torch.Tensor, context_lens: torch.Tensor, query_len: int,
                      softmax_scale: float, partition_size: int,
                      key_scale: Optional[torch.Tensor] = None,
                      value_scale: Optional[torch.Tensor] = None,
                      alibi_slopes: Optional[torch.Tensor] = None
                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Exact-fp32 statement of the partition kernel's outputs.

    query ``[S, Hkv*L*G, D]`` in the operator's row order (row ``r = t*G + g`` inside a kv head,
    test_pa_mtp.py:793-804).  Returns ``(max_logits, exp_sums, tmp_out)`` shaped
    ``[S,Hkv,P,eqG]``, ``[S,Hkv,P,eqG]``, ``[S,Hkv,P,eqG,D]`` (fp32), where for partition p
    m = max_j s_j, l = sum_j exp(s_j - m), o = sum_j exp(s_j - m) v_j / l over the partition's
    visible keys (pa_decode_triton_gluon_fp8.py:929-937,979-1002).  Row (t, g) sees key j iff
    ``(L-1-t) + j < ctx`` (:915-920).  Partitions with no visible key hold m=-inf, l=0, o=0;
    partitions beyond the context are left at m=-inf, l=0, o=0 as well.  ``alibi_slopes``
    ``[Hkv*G]``: the bias ``slope[head] * (j - (ctx - 1))`` on the scaled scores
    (pa_decode_triton.py:148-151, pa_decode_triton_gluon_fp8.py:905-908).
    """
    nb, hkv, d, bs = value_cache.shape
    S = query.shape[0]
    eqg = query.shape[1] // hkv
    G = eqg // query_len
    max_ctx = int(context_lens.max().item()) if S else 0
    P = max(1, (max_ctx + partition_size - 1) // partition_size)
    m_out = torch.full((S, hkv, P, eqg), float("-inf"))
    l_out = torch.zeros((S, hkv, P, eqg))
    o_out = torch.zeros((S, hkv, P, eqg, d))
    k_flat, v_flat = flatten_caches(key_cache, value_cache)
    for s in range(S):
        ctx = int(context_lens[s].item())
        if ctx <= 0:
            continue
        keys, values = gather_sequence(k_flat, v_flat, block_tables[s], ctx, bs, key_scale, value_scale)
        q = query[s].float().view(hkv, eqg, d)                       # [Hkv, eqG, D]
        scores = torch.einsum("hrd,khd->hrk", q, keys) * softmax_scale   # [Hkv, eqG, ctx]
        if alibi_slopes is not None:
            rel = torch.arange(ctx, dtype=torch.float32) - (ctx - 1)
            slope_of_row = alibi_slopes.float().view(hkv, G)[:, torch.arange(eqg) % G]      # [Hkv, eqG]
            scores = scores + slope_of_row[..., None] * rel
        t_of_row = torch.arange(eqg) // G
        limit = ctx - (query_len - 1 - t_of_row)                      # [eqG]
        visible = torch.arange(ctx)[None, :] < limit[:, None]        # [eqG, ctx]
        scores = scores.masked_fill(~visible[None], float("-inf"))
        for p in range((ctx + partition_size - 1) // partition_size):
            lo, hi = p * partition_size, min(ctx, (p + 1) * partition_size)
            sc = scores[:, :, lo:hi]
            m = sc.max(dim=-1).values                                  # [Hkv, eqG]
            m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
            e = torch.exp(sc - m_safe[..., None])
            e = torch.where(torch.isinf(sc), torch.zeros_like(e), e)
            l = e.sum(dim=-1)
            o = torch.einsum("hrk,khd->hrd", e, values[lo:hi])
            o = torch.where(l[..., None] > 0, o / l[..., None].clamp_min(1e-38), torch.zeros_like(o))
            m_out[s, :, p] = m
            l_out[s, :, p] = l
            o_out[s, :, p] = o
    return m_out, l_out, o_out


def merge_partials(max_logits: torch.Tensor, exp_sums: torch.Tensor, tmp_out: torch.Tensor) -> torch.Tensor:
    """Reduce over the partition axis (pa_decode_triton_gluon_fp8.py:1266-1313), fp32.

    Inputs ``[..., P, eqG]``, ``[..., P, eqG]``, ``[..., P, eqG, D]``; returns ``[..., eqG, D]``.
    Partitions with l == 0 weigh nothing.
    """
    m = max_logits.float()
    l = exp_sums.float()
    M = m.max(dim=-2, keepdim=True).values
    M_safe = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    w = torch.where(l > 0, l * torch.exp(m - M_safe), torch.zeros_like(l))
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    W = w.sum(dim=-2, keepdim=True)
    frac = torch.where(W > 0, w / W.clamp_min(1e-38), torch.zeros_like(w))
    o = torch.where(frac[..., None] > 0, tmp_out.float(), torch.zeros_like(tmp_out.float()))
    return (o * frac[..., None]).sum(dim=-3)


def merge_triples(m: torch.Tensor, l: torch.Tensor, o: torch.Tensor) -> torch.Tensor:
    """Cross-shard merge of (m, l, o) triples, shard axis first: ``[n, R]``, ``[n, R]``,
    ``[n, R, D]`` -> ``[R, D]``.  The same formula as ``merge_partials`` with shards as partitions."""
    return merge_partials(m, l, o)


def compare_arrays(arr1: np.ndarray, arr2: np.ndarray, k: int = 5,
                   thresholds=(0, 1e-6, 1e-5, 1e-4, 1e-3, 1e-2, 1e-1, 1e0, 1e1)) -> Dict:
    """The reference's numeric report (utils.py:5-106) without the printing.

    Returns max abs difference, ``max(|a-b| / (1 + |b|))``, the top-k differences, the histogram
    of differences over ``thresholds`` and the NaN counts of both inputs.
    """
    if arr1.shape != arr2.shape:
        raise ValueError("Input arrays must have the same shape")
    a = arr1.astype(np.float32)
    b = arr2.astype(np.float32)
    diff = np.abs(a - b)
    flat = diff.ravel()
    k = min(k, flat.size)
    top = np.argpartition(flat, -k)[-k:] if k else np.array([], dtype=np.int64)
    top = top[np.argsort(-flat[top])]
    pos = np.unravel_index(top, diff.shape) if k else ()
    top_k: List[Dict] = []
    for i in range(k):
        idx = tuple(int(dim[i]) for dim in pos)
        top_k.append({"value": float(diff[idx]), "position": idx,
                      "arr1_value": float(a[idx]), "arr2_value": float(b[idx])})
    stats = []
    for lo, hi in zip(thresholds[:-1], thresholds[1:]):
        cnt = int(np.sum((diff >= lo) & (diff < hi)))
        stats.append({"range": f"[{lo:.1e}, {hi:.1e})", "count": cnt, "percentage": 100 * cnt / max(1, a.size)})
    cnt = int(np.sum(diff >= thresholds[-1]))
    stats.append({"range": f">={thresholds[-1]:.1e}", "count": cnt, "percentage": 100 * cnt / max(1, a.size)})
    return {
        "max_abs_diff": float(diff.max()) if diff.size else 0.0,
        "max_diff_thr": float((diff / (1.0 + np.abs(b))).max()) if diff.size else 0.0,
        "top_k_diff": top_k,
        "threshold_stats": stats,
        "nan_info": {"arr1_nan_count": int(np.isnan(a).sum()), "arr2_nan_count": int(np.isnan(b).sum())},
    }


def write_kv_cache(key: torch.Tensor, value: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                   slot_mapping: torch.Tensor, key_scale: Optional[torch.Tensor] = None,
                   value_scale: Optional[torch.Tensor] = None) -> None:
    """CPU statement of the cache write side, in place on the cache (and per-token scale) tensors.

    Layouts as the reference builds them: keys ``[NB, Hkv, D/x, bs, x]`` (test_pa_mtp.py:150-151),
    values ``[NB, Hkv, D, bs]`` (:162) or shuffled ``[NB, Hkv, bs/x, D, x]`` (:472-497).  Per-token
    quantisation follows quantize_kv_cache_symmetric (:294-369) with the build's quantiser
    ``scale = max(amax / 448, 1e-12)``, ``q = (x / scale) -> e4m3fn``; 0-dim scales are read.
    ``key`` / ``value`` ``[T, Hkv, D]``; ``slot_mapping [T]`` (block * bs + offset, negative = skip).
    """
    T, hkv, d = key.shape
    nb, bs = key_cache.shape[0], key_cache.shape[3]
    x = key_cache.shape[4]
    fp8 = key_cache.dtype != torch.bfloat16
    trans = value_cache.dim() == 5
    for t in range(T):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        blk, off = slot // bs, slot % bs
        for which, src, cache, scale in (("k", key, key_cache, key_scale), ("v", value, value_cache, value_scale)):
            vec = src[t].float()                                  # [Hkv, D]
            if fp8:
                # values beyond the e4m3fn range saturate to +-448 (a plain torch cast would store NaN)
                if scale is None:
                    q = vec.clamp(-448.0, 448.0).to(cache.dtype)
                elif scale.dim() == 0:
                    q = (vec / scale.float()).clamp(-448.0, 448.0).to(cache.dtype)
                else:
                    s = (vec.abs().amax(dim=-1, keepdim=True) / 448.0).clamp_min(1e-12)    # [Hkv, 1]
                    scale[blk, :, off, 0] = s[:, 0]
                    q = (vec / s).to(cache.dtype)
            else:
                q = src[t]
            if which == "k":
                cache[blk, :, :, off, :] = q.view(hkv, d // x, x)
            elif trans:
                cache[blk, :, off // x, :, off % x] = q
            else:
                cache[blk, :, :, off] = q
