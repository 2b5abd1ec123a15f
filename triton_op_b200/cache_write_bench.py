"""Throughput of the KV-cache write kernel on synthetic token streams.

    python -m triton_op_b200.cache_write_bench [--tokens 65536] [--heads 8] [--block-size 16] [--steps 50]

Prints one JSON line per slot pattern:
  scattered   every token in a random slot (a decode step's writes, one token per sequence)
  prefill     512-token chunks of consecutive positions starting 5 slots into a page, pages shuffled
Algorithmic bytes per (token, head): 512 read (bf16 key and value) + 256 written (e4m3) + 8 (two
fp32 scales).  Timed with CUDA events after warm-up; inputs are larger than L2 from 32 768 tokens on.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .cache_write import write_kv_cache
from .inputs import FP8


def _peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"])
    except Exception:
        return 6650.0   # an earlier measurement of this pool's B200s


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=65536)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--steps", type=int, default=50)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("cache_write_bench: no CUDA device; the kernel has no CPU path")
    dev = torch.device("cuda:0")
    T, hkv, bs, d = args.tokens, args.heads, args.block_size, 128
    nb = max(T // bs * 2, 64)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    key = torch.randn(T, hkv, d, device=dev, generator=gen).to(torch.bfloat16)
    value = torch.randn(T, hkv, d, device=dev, generator=gen).to(torch.bfloat16)
    kc = torch.zeros(nb, hkv, d // 16, bs, 16, device=dev).to(FP8)
    vc = torch.zeros(nb, hkv, d, bs, device=dev).to(FP8)
    ks = torch.zeros(nb, hkv, bs, 1, device=dev)
    vs = torch.zeros(nb, hkv, bs, 1, device=dev)
    pos = torch.arange(T, device=dev)
    pages = torch.randperm(nb, device=dev, generator=gen)
    inner = pos % 512 + 5
    patterns = {
        "scattered": torch.randperm(nb * bs, device=dev, generator=gen)[:T],
        "prefill": pages[((pos // 512) * ((512 + 5 + bs - 1) // bs) + inner // bs) % nb] * bs + inner % bs,
    }
    peak = _peak_gbs()
    for name, slots in patterns.items():
        for _ in range(3):
            write_kv_cache(key, value, kc, vc, slots, ks, vs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            write_kv_cache(key, value, kc, vc, slots, ks, vs)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        nbytes = T * hkv * (2 * 2 * d + 2 * d + 8)
        gbs = nbytes / us / 1e3
        print(json.dumps({"metric": "kv_cache_write_bandwidth", "pattern": name, "tokens": T, "kv_heads": hkv,
                          "block_size": bs, "quant": "e4m3fn per-token", "us_per_call": us, "value": gbs, "unit": "GB/s",
                          "algorithmic_bytes": nbytes,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "frac": gbs / peak}}), flush=True)


if __name__ == "__main__":
    main()
