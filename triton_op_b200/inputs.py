"""KV-cache layouts, quantisers and seeded synthetic workloads for the decode operator.

Host-side mirror of the reference harness' input builders (yanguahe/triton_op):

* paged layouts -- key ``[NB, Hkv, D/x, bs, x]`` with ``x = 16 // itemsize`` and value
  ``[NB, Hkv, D, bs]`` (test_pa_mtp.py:149-162);
* per-token-per-head symmetric quantisation with scales ``[NB, Hkv, bs, 1]`` and their flat
  ``[Hkv, NB*bs]`` form for the PyTorch path (test_pa_mtp.py:294-369); the quantiser here is
  ``scale = amax / 448`` to OCP e4m3fn, per tensor or per (block, head, token) vector, and the
  same bytes are handed to every implementation;
* the MTP row permutation ``[S*L, Hq, D] <-> [S, Hkv*L*G, D]`` (test_pa_mtp.py:793-822, 903-909);
* the five seeded workloads the benchmark and the parity tests run (``CONFIGS``).

There is no dataset behind any of this: the reference measures on random tensors too.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
HEAD_SIZE = 128


# ----------------------------------------------------------------------------- layouts
def to_paged_key(k_tok: torch.Tensor) -> torch.Tensor:
    """Token-major ``[NB, Hkv, bs, D]`` -> paged key layout ``[NB, Hkv, D/x, bs, x]``."""
    nb, hkv, bs, d = k_tok.shape
    x = 16 // k_tok.element_size()
    return k_tok.view(nb, hkv, bs, d // x, x).permute(0, 1, 3, 2, 4).contiguous()


def to_paged_value(v_tok: torch.Tensor) -> torch.Tensor:
    """Token-major ``[NB, Hkv, bs, D]`` -> paged value layout ``[NB, Hkv, D, bs]``."""
    return v_tok.permute(0, 1, 3, 2).contiguous()


def from_paged_key(key_cache: torch.Tensor) -> torch.Tensor:
    nb, hkv, dx, bs, x = key_cache.shape
    return key_cache.permute(0, 1, 3, 2, 4).reshape(nb, hkv, bs, dx * x)


def from_paged_value(value_cache: torch.Tensor) -> torch.Tensor:
    return value_cache.permute(0, 1, 3, 2)


def shuffle_value_cache_layout(value_cache: torch.Tensor) -> torch.Tensor:
    """``[NB, Hkv, D, bs]`` -> transposed ``[NB, Hkv, bs/x, D, x]`` (test_pa_mtp.py:472-497)."""
    x = 16 // value_cache.element_size()
    nb, hkv, d, bs = value_cache.shape
    return value_cache.view(nb, hkv, d, bs // x, x).permute(0, 1, 3, 2, 4).contiguous()


# ----------------------------------------------------------------------------- quantisers
def quantize_per_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``scale = amax/448`` (0-dim fp32), ``q = (x/scale) -> e4m3fn``."""
    scale = (x.abs().amax().float() / FP8_MAX).clamp_min(1e-12)
    return (x.float() / scale).to(FP8), scale


def quantize_per_token(x_tok: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per (block, head, token) vector of ``[NB, Hkv, bs, D]``: scales ``[NB, Hkv, bs, 1]`` fp32."""
    scale = (x_tok.abs().amax(dim=-1, keepdim=True).float() / FP8_MAX).clamp_min(1e-12)
    return (x_tok.float() / scale).to(FP8), scale


def flat_scale(scale: Optional[torch.Tensor], num_blocks: int, num_kv_heads: int, block_size: int
               ) -> Optional[torch.Tensor]:
    """A scale argument in the flat ``[Hkv, NB*bs]`` form the PyTorch path takes
    (test_pa_mtp.py:351,360)."""
    if scale is None:
        return None
    if scale.dim() == 0:
        return scale.expand(num_kv_heads, num_blocks * block_size).contiguous()
    return scale.permute(1, 0, 2, 3).contiguous().view(num_kv_heads, num_blocks * block_size)


# ----------------------------------------------------------------------------- MTP row order
def pack_mtp(x: torch.Tensor, num_seqs: int, query_len: int, num_kv_heads: int) -> torch.Tensor:
    """``[S*L, Hq, D]`` (token-major, the PyTorch path's order) -> ``[S, Hkv*L*G, D]`` (the
    operator's order: inside a kv head, row ``t*G + g``)."""
    sl, hq, d = x.shape
    g = hq // num_kv_heads
    return (x.reshape(num_seqs, query_len, num_kv_heads, g, d).transpose(1, 2)
            .reshape(num_seqs, num_kv_heads * query_len * g, d))


def unpack_mtp(x: torch.Tensor, num_seqs: int, query_len: int, num_kv_heads: int) -> torch.Tensor:
    """Inverse of ``pack_mtp``."""
    s, rows, d = x.shape
    g = rows // (num_kv_heads * query_len)
    return (x.reshape(num_seqs, num_kv_heads, query_len, g, d).transpose(1, 2)
            .reshape(num_seqs * query_len, num_kv_heads * g, d))


# ----------------------------------------------------------------------------- workloads
@dataclass
class DecodeConfig:
    """One synthetic decode workload.  ``context`` is ``("fixed", n)``, ``("uniform", lo, hi)``
    (inclusive), ``("cycle", [..])`` or ``("lognormal", median, sigma, lo, hi)``."""
    name: str
    num_seqs: int
    q_heads: int
    kv_heads: int
    block_size: int
    query_len: int
    context: tuple
    kv_dtype: str = "fp8"           # "fp8" | "bf16"
    quant: str = "per_tensor"       # "per_tensor" | "per_token" | "none"
    partition_size: int = 256
    pool_blocks: Optional[int] = None  # physical blocks; default: exactly what the tables use
    head_size: int = HEAD_SIZE


CONFIGS: Dict[str, DecodeConfig] = {
    # CPU-runnable case of the reference's own PyTorch path
    "cfg1_small": DecodeConfig("cfg1_small", 4, 8, 1, 16, 1, ("uniform", 1, 512), pool_blocks=128),
    # Llama-3-8B-shaped decode, the configuration the headline metric is quoted on
    "cfg2_llama8b": DecodeConfig("cfg2_llama8b", 64, 32, 8, 16, 1, ("fixed", 4096), pool_blocks=20000),
    # Llama-3-70B-shaped MTP decode, 1024-token pages, per-token scales
    "cfg3_llama70b_mtp": DecodeConfig("cfg3_llama70b_mtp", 128, 64, 8, 1024, 2, ("uniform", 1024, 8192),
                                      quant="per_token"),
    # long-context single-kv-head shard, partition 512
    "cfg4_longctx": DecodeConfig("cfg4_longctx", 8, 8, 1, 16, 1, ("cycle", [32768, 65536, 131072]),
                                 partition_size=512),
    # large-batch serving mix, fp8 and bf16 KV
    "cfg5_serving_fp8": DecodeConfig("cfg5_serving_fp8", 1024, 32, 8, 16, 1,
                                     ("lognormal", 2048, 1.0, 16, 32768)),
    "cfg5_serving_bf16": DecodeConfig("cfg5_serving_bf16", 1024, 32, 8, 16, 1,
                                      ("lognormal", 2048, 1.0, 16, 32768), kv_dtype="bf16", quant="none"),
}


def draw_context_lens(cfg: DecodeConfig, gen: torch.Generator) -> torch.Tensor:
    kind = cfg.context[0]
    s = cfg.num_seqs
    if kind == "fixed":
        return torch.full((s,), int(cfg.context[1]), dtype=torch.int32)
    if kind == "uniform":
        return torch.randint(int(cfg.context[1]), int(cfg.context[2]) + 1, (s,), generator=gen, dtype=torch.int32)
    if kind == "cycle":
        vals = list(cfg.context[1])
        return torch.tensor([vals[i % len(vals)] for i in range(s)], dtype=torch.int32)
    if kind == "lognormal":
        _, median, sigma, lo, hi = cfg.context
        z = torch.randn(s, generator=gen)
        return torch.exp(math.log(median) + sigma * z).round().clamp(lo, hi).to(torch.int32)
    raise ValueError(f"unknown context spec {cfg.context}")


@dataclass
class DecodeInputs:
    """Everything one decode call needs, plus what the PyTorch path wants for the same data."""
    cfg: DecodeConfig
    query: torch.Tensor            # [S, Hkv*L*G, D] bf16, operator row order
    query_tokens: torch.Tensor     # [S*L, Hq, D] bf16, token-major (the PyTorch path's order)
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    key_scale: Optional[torch.Tensor]    # None | 0-dim | [NB, Hkv, bs, 1]
    value_scale: Optional[torch.Tensor]
    block_tables: torch.Tensor     # [S, max_blocks] int32
    context_lens: torch.Tensor     # [S] int32
    softmax_scale: float
    max_context: int
    meta: dict = field(default_factory=dict)

    @property
    def kv_bytes(self) -> int:
        """Algorithmic KV bytes one call must read: sum_s ctx_s * Hkv * D * 2 * itemsize."""
        c = self.cfg
        item = self.key_cache.element_size()
        return int(self.context_lens.to(torch.int64).sum().item()) * c.kv_heads * c.head_size * 2 * item

    def to(self, device) -> "DecodeInputs":
        mv = lambda t: None if t is None else t.to(device)
        return DecodeInputs(self.cfg, mv(self.query), mv(self.query_tokens), mv(self.key_cache),
                            mv(self.value_cache), mv(self.key_scale), mv(self.value_scale),
                            mv(self.block_tables), mv(self.context_lens), self.softmax_scale,
                            self.max_context, dict(self.meta))

    def flat_scales(self) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        nb, hkv = self.key_cache.shape[0], self.key_cache.shape[1]
        bs = self.cfg.block_size
        return flat_scale(self.key_scale, nb, hkv, bs), flat_scale(self.value_scale, nb, hkv, bs)

    def query_indptr(self) -> torch.Tensor:
        return torch.arange(self.cfg.num_seqs + 1, dtype=torch.int32, device=self.query.device) * self.cfg.query_len


def _gen_tokens(num_blocks: int, hkv: int, bs: int, d: int, seed: int, device, chunk_blocks: int,
                dist: str):
    """Yields ``(b0, b1, fp32 [b1-b0, Hkv, bs, D])`` chunks; chunk i is drawn from its own seed so
    a two-pass quantiser sees the same numbers twice."""
    for ci, b0 in enumerate(range(0, num_blocks, chunk_blocks)):
        b1 = min(num_blocks, b0 + chunk_blocks)
        g = torch.Generator(device=device)
        g.manual_seed(seed * 1000003 + ci)
        shape = (b1 - b0, hkv, bs, d)
        if dist == "uniform":
            x = torch.rand(shape, generator=g, device=device, dtype=torch.float32) * 2 - 1
        else:
            x = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        yield b0, b1, x


def make_cache(num_blocks: int, hkv: int, bs: int, d: int, seed: int, device, kv_dtype: str, quant: str,
               is_key: bool, dist: str = "normal", chunk_bytes: int = 1 << 28):
    """One paged cache (key or value) of seeded random tokens and its scale (or None)."""
    chunk_blocks = max(1, chunk_bytes // (hkv * bs * d * 4))
    layout = to_paged_key if is_key else to_paged_value
    if kv_dtype == "bf16":
        parts = [layout(x.to(torch.bfloat16)) for _, _, x in _gen_tokens(num_blocks, hkv, bs, d, seed, device, chunk_blocks, dist)]
        return torch.cat(parts), None
    if quant == "per_token":
        caches, scales = [], []
        for _, _, x in _gen_tokens(num_blocks, hkv, bs, d, seed, device, chunk_blocks, dist):
            q, s = quantize_per_token(x)
            caches.append(layout(q))
            scales.append(s)
        return torch.cat(caches), torch.cat(scales)
    # per tensor: pass 1 finds amax, pass 2 quantises the same numbers
    amax = torch.zeros((), device=device)
    for _, _, x in _gen_tokens(num_blocks, hkv, bs, d, seed, device, chunk_blocks, dist):
        amax = torch.maximum(amax, x.abs().amax())
    scale = (amax / FP8_MAX).clamp_min(1e-12).float()
    parts = [layout((x / scale).to(FP8)) for _, _, x in _gen_tokens(num_blocks, hkv, bs, d, seed, device, chunk_blocks, dist)]
    return torch.cat(parts), (scale if quant == "per_tensor" else None)


def make_inputs(cfg: DecodeConfig, seed: int = 0, device="cpu", num_seqs: Optional[int] = None,
                context_lens: Optional[torch.Tensor] = None, dist: str = "normal") -> DecodeInputs:
    """Builds the workload ``cfg`` from ``seed``.

    q/K/V are N(0,1) (``dist="uniform"`` gives the reference harness' U(-1,1)), q is cast to
    bf16, block tables are slices of one random permutation of the pool (unique pages), the
    softmax scale is ``1/sqrt(D)``.  ``num_seqs`` / ``context_lens`` override the config for
    reduced-size variants.  Small index tensors are drawn on CPU so they do not depend on the
    device; the bulk tensors are drawn on ``device``.
    """
    if num_seqs is not None:
        cfg = DecodeConfig(**{**cfg.__dict__, "num_seqs": num_seqs})
    gen = torch.Generator()
    gen.manual_seed(seed)
    ctx = draw_context_lens(cfg, gen) if context_lens is None else context_lens.to(torch.int32).cpu()
    assert ctx.numel() == cfg.num_seqs
    bs, d, hkv = cfg.block_size, cfg.head_size, cfg.kv_heads
    blocks_per_seq = ((ctx.to(torch.int64) + bs - 1) // bs)
    used = int(blocks_per_seq.sum().item())
    max_blocks = int(blocks_per_seq.max().item()) if cfg.num_seqs else 1
    pool = cfg.pool_blocks if cfg.pool_blocks is not None else used
    pool = max(pool, used, 1)
    perm = torch.randperm(pool, generator=gen)[:used].to(torch.int32)
    block_tables = torch.zeros((cfg.num_seqs, max(1, max_blocks)), dtype=torch.int32)
    off = 0
    for s in range(cfg.num_seqs):
        n = int(blocks_per_seq[s])
        block_tables[s, :n] = perm[off:off + n]
        off += n

    gq = torch.Generator(device=device)
    gq.manual_seed(seed + 17)
    L, hq = cfg.query_len, cfg.q_heads
    if dist == "uniform":
        q_tok = torch.rand((cfg.num_seqs * L, hq, d), generator=gq, device=device) * 2 - 1
    else:
        q_tok = torch.randn((cfg.num_seqs * L, hq, d), generator=gq, device=device)
    q_tok = q_tok.to(torch.bfloat16)
    query = pack_mtp(q_tok, cfg.num_seqs, L, hkv).contiguous()

    key_cache, key_scale = make_cache(pool, hkv, bs, d, seed * 2 + 101, device, cfg.kv_dtype, cfg.quant, True, dist)
    value_cache, value_scale = make_cache(pool, hkv, bs, d, seed * 2 + 202, device, cfg.kv_dtype, cfg.quant, False, dist)
    return DecodeInputs(cfg, query, q_tok, key_cache, value_cache, key_scale, value_scale,
                        block_tables.to(device), ctx.to(device), 1.0 / math.sqrt(d),
                        int(ctx.max().item()) if cfg.num_seqs else 0,
                        {"pool_blocks": pool, "used_blocks": used, "seed": seed, "dist": dist})


def subset_inputs(inp: DecodeInputs, seq_ids) -> DecodeInputs:
    """``inp`` restricted to the sequences ``seq_ids``, with only their pages kept and renumbered
    (page ``i`` of the result is the ``i``-th page the kept sequences use).  The bytes every kept
    sequence sees are unchanged, so a result computed on the subset equals the rows of the full
    batch; the pool shrinks from gigabytes to what a few sequences need, which is what a parity
    check of a sampled handful of sequences wants to move to the host."""
    ids = [int(i) for i in seq_ids]
    cfg = inp.cfg
    bs, L = cfg.block_size, cfg.query_len
    ctx = inp.context_lens[ids].cpu()
    nblk = ((ctx.to(torch.int64) + bs - 1) // bs).tolist()
    rows = inp.block_tables[ids].cpu()
    pages = torch.cat([rows[i, :n] for i, n in enumerate(nblk)] + [rows.new_zeros(0)]).long()
    if pages.numel() == 0:
        pages = torch.zeros(1, dtype=torch.long)
    tables = torch.zeros((len(ids), max(1, max(nblk, default=1))), dtype=torch.int32)
    off = 0
    for i, n in enumerate(nblk):
        tables[i, :n] = torch.arange(off, off + n, dtype=torch.int32)
        off += n
    dev = inp.key_cache.device
    pg = pages.to(dev)
    pick = lambda t: t if (t is None or t.dim() == 0) else t[pg]
    tok_rows = [s * L + t for s in ids for t in range(L)]
    sub_cfg = DecodeConfig(**{**cfg.__dict__, "num_seqs": len(ids), "pool_blocks": None})
    return DecodeInputs(sub_cfg, inp.query[ids], inp.query_tokens[tok_rows], inp.key_cache[pg], inp.value_cache[pg],
                        pick(inp.key_scale), pick(inp.value_scale), tables.to(dev), ctx.to(dev), inp.softmax_scale,
                        int(ctx.max().item()) if len(ids) else 0, dict(inp.meta, subset_of=ids))
