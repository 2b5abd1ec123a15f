#!/usr/bin/env python
"""Benchmark of the paged-attention decode operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

A step is one decode call (partition kernel + reduce kernel) over one batch of synthetic input.
The headline workload at every N is the Llama-3-8B-shaped configuration the metric is quoted on
(64 sequences x 4096 tokens, 32 query / 8 kv heads, fp8 KV, 16-token pages) per GPU: sequences
are independent, so ranks shard the batch with no collective and the scaling is weak.

One JSON line is printed by rank 0:
  value      KV bytes all ranks read per step / device time of the step (max over ranks), inputs
             resident in HBM;
  e2e        the same metric through the public entry point with the step's inputs (query, block
             tables, context lengths) coming from pinned host memory and the output copied back,
             the host reading every result before it issues the next step; `e2e.pipelined` is the
             same loop two steps deep (two independent batches interleaved);
  roofline   the partition kernel alone against the measured HBM copy bandwidth (read+write) and
             against a read-only streaming probe run in the same process;
  cpu_baseline  the oracle (a CPU port of the reference's own PyTorch path) on a bounded sample;
  workloads  after the headline, in the same process: the other configurations (one GPU), or the
             multi-GPU splits of the long-context, serving-mix and MTP configurations (N > 1),
             each with its step time, KV GB/s and the largest error of a sampled handful of
             sequences against the oracle.
`--impl reference` times the CPU path as the reference arm (rank 0 only).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from triton_op_b200.inputs import CONFIGS, draw_context_lens, make_inputs, subset_inputs, unpack_mtp  # noqa: E402

METRIC = "kv_read_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 << 20     # B200
ATOL, RTOL = 2e-2, 1e-2  # bf16 outputs against the PyTorch path

# dram__bytes_read.sum + dram__bytes_write.sum of one partition-kernel launch divided by the
# algorithmic KV bytes of that launch, per workload, from the ncu captures summarised under
# profiles/ (captured on the workload itself or on fewer of its sequences; traffic grows in
# proportion to the sequences).  Workloads without a capture report no traffic.
NCU_TRAFFIC_PER_KV_BYTE = {"cfg2_llama8b": 1.033, "cfg3_llama70b_mtp": 1.07, "cfg4_longctx": 1.036}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs.

    Every sample is kept; a sample counts as taken under load when the SM clock is above half of
    its maximum (an idle B200 parks far below that).  The median of the loaded samples is the
    clock the timed kernels ran at; the reasons are those seen in any sample."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        loaded, every, mx, reasons = [], [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                clk = float(parts[0])
                mx = float(parts[1])
            except ValueError:
                continue
            every.append(clk)
            if clk > 0.5 * mx:
                loaded.append(clk)
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        loaded.sort()
        use = loaded if loaded else sorted(every)
        return {"sm_mhz": use[len(use) // 2] if use else None, "sm_max_mhz": mx, "samples": len(every),
                "samples_under_load": len(loaded), "reasons": sorted(reasons)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo",
                                rank=rank, world_size=world,
                                device_id=torch.device(f"cuda:{local}") if torch.cuda.is_available() else None)
    return rank, world, local


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()


def _all_reduce(x: float, world: int, device, op) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=op)
    return float(t.item())


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    return _all_reduce(x, world, device, dist.ReduceOp.MAX)


def sum_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    return _all_reduce(x, world, device, dist.ReduceOp.SUM)


# ----------------------------------------------------------------------------- CPU arm
def cpu_reference_time(inp_cpu, sample_seqs: int, repeats: int = 1):
    """Times the oracle (CPU port of the reference's PyTorch path) on the first `sample_seqs`
    sequences of the workload.  Returns (seconds per pass, KV bytes of the sample, threads)."""
    from oracle import pa_oracle  # checker / CPU baseline only; never on the product path
    c = inp_cpu.cfg
    n = min(sample_seqs, c.num_seqs)
    L = c.query_len
    ks, vs = inp_cpu.flat_scales()
    q = inp_cpu.query_tokens[: n * L]
    bt = inp_cpu.block_tables[:n]
    ctx = inp_cpu.context_lens[:n]
    indptr = torch.arange(n + 1, dtype=torch.int32) * L
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        pa_oracle.paged_attention(q, inp_cpu.key_cache, inp_cpu.value_cache, bt, ctx, indptr, ks, vs)
        best = min(best, time.perf_counter() - t0)
    item = inp_cpu.key_cache.element_size()
    kv_bytes = int(ctx.to(torch.int64).sum().item()) * c.kv_heads * c.head_size * 2 * item
    return best, kv_bytes, torch.get_num_threads()


def oracle_error(sub, got_rows: torch.Tensor) -> dict:
    """Largest error of `got_rows` (operator row order, the sequences of `sub`) against the oracle
    run on the host.  The oracle is the checker here, outside every timed region."""
    from oracle import pa_oracle  # checker only
    cpu = sub.to("cpu")
    c = cpu.cfg
    ks, vs = cpu.flat_scales()
    ref = pa_oracle.paged_attention(cpu.query_tokens, cpu.key_cache, cpu.value_cache, cpu.block_tables,
                                    cpu.context_lens, cpu.query_indptr(), ks, vs).float()
    got = unpack_mtp(got_rows.cpu(), c.num_seqs, c.query_len, c.kv_heads).float()
    err = (got - ref).abs()
    ok = bool((err <= ATOL + RTOL * ref.abs()).all()) and not bool(torch.isnan(got).any())
    return {"max_abs_err": float(err.max()) if err.numel() else 0.0, "within_tolerance": ok,
            "checked_sequences": cpu.meta.get("subset_of"), "atol": ATOL, "rtol": RTOL}


def run_reference_arm(args, rank: int, world: int):
    """The reference's own CPU implementation of the path, on this box's host cores."""
    if rank != 0:
        return
    cfg = CONFIGS[args.workload]
    sample = 8
    # only the sample's pages are materialised: the pool is exactly what the sample uses
    small = type(cfg)(**{**cfg.__dict__, "num_seqs": sample, "pool_blocks": None})
    inp = make_inputs(small, seed=0, device="cpu")
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_time(inp, sample)
    times = []
    kvb = 0
    for _ in range(args.steps):
        t, kvb, thr = cpu_reference_time(inp, sample)
        times.append(t)
    t_step = sum(times) / len(times)
    value = kvb / t_step / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": f"first {sample} of {cfg.num_seqs} sequences per step",
                   "kv": "fp8 e4m3fn per-tensor scales", "context_len": cfg.context[1] if cfg.context[0] == "fixed" else str(cfg.context)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample} sequences ({kvb} KV bytes) per step, oracle/pa_oracle.py on host cores "
                                   "(the reference is Python source that does not travel to the GPU machine; the port is "
                                   "pinned bit for bit to fixtures its own functions generated)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
class Workload:
    """One workload on this rank under one sharding mode: inputs, the call, what it reads."""

    def __init__(self, name: str, mode: str, exchange: str, rank: int, world: int, dev, num_seqs: int = 0,
                 graph: bool = True):
        from triton_op_b200 import paged_attention_decode
        self.name, self.mode, self.exchange, self.rank, self.world, self.dev = name, mode, exchange, rank, world, dev
        cfg = CONFIGS[name]
        if num_seqs > 0:   # reduced batch: for profiler captures, never for a reported number
            cfg = type(cfg)(**{**cfg.__dict__, "num_seqs": num_seqs, "pool_blocks": None})
        self.status = torch.zeros((), dtype=torch.int32, device=dev)
        self.decoder = None
        self.global_ids = None      # sequences-strong: indices of this rank's sequences in the global batch
        if mode == "sequences-weak":
            self.inp = make_inputs(cfg, seed=rank, device=dev)      # every rank its own batch of the full size
        elif mode == "sequences-strong":
            # one global batch; every rank computes the same plan and builds only its own sequences
            from triton_op_b200.sharding import shard_sequences
            gen = torch.Generator()
            gen.manual_seed(0)
            lens = draw_context_lens(cfg, gen)
            mine = shard_sequences(lens.tolist(), world, "balanced")[rank]     # by token count
            self.global_ids = mine
            sub = type(cfg)(**{**cfg.__dict__, "num_seqs": len(mine), "pool_blocks": None})
            self.inp = make_inputs(sub, seed=rank, device=dev, context_lens=lens[mine])
        elif mode == "kv-partitions":
            # every rank builds the same pool (same seed) and reads only the pages of its ranges
            from triton_op_b200.sharding import KvShardedDecoder, plan_kv_shards
            self.inp = make_inputs(cfg, seed=0, device=dev)
            plan = plan_kv_shards(self.inp.context_lens.tolist(), world, cfg.partition_size, cfg.query_len)[rank]
            self.decoder = KvShardedDecoder(self.inp.query, self.inp.key_cache, self.inp.value_cache, plan,
                                            self.inp.block_tables, self.inp.softmax_scale, self.inp.key_scale,
                                            self.inp.value_scale, partition_size=cfg.partition_size,
                                            status=self.status, exchange=exchange)
        else:
            raise ValueError(mode)
        inp = self.inp
        self.cfg = c = inp.cfg
        self.out = torch.empty_like(inp.query) if self.decoder is None else self.decoder.out
        self.kv_bytes = inp.kv_bytes if self.decoder is None else self.decoder.kv_bytes
        self.step_ctx = inp.context_lens if self.decoder is None else self.decoder.context_lens
        self.step_bt = inp.block_tables if self.decoder is None else self.decoder.tables
        self._decode = paged_attention_decode
        # The KV-partition-sharded step is three short launches; replayed as one CUDA graph, or the
        # host's launch rate is what gets timed.
        self.step_graph = None
        if self.decoder is not None and graph:
            try:
                self.step_graph = self.decoder.capture()
            except Exception as exc:  # noqa: BLE001 - eager launches are still a valid measurement
                sys.stderr.write(f"bench.py: CUDA graph capture of the sharded step failed ({exc}); using eager launches\n")
                self.step_graph = None
        # L2: a step that reads less than about twice the L2 would find its KV there on the next
        # iteration, so L2 is flushed before every timed step (a 256 MB write, then a read of the same
        # buffer so that the step does not also pay for writing the flush's dirty lines back) and the
        # steps are timed one by one.
        self.flush_l2 = self.kv_bytes < 2 * L2_BYTES
        self.flush_buf = torch.empty(64 << 20, dtype=torch.int32, device=dev) if self.flush_l2 else None
        self.align = torch.zeros(1, dtype=torch.float32, device=dev) if (self.flush_l2 and world > 1) else None

    # -- the step
    def call(self, query=None, ctx=None, bt=None, out=None, workspaces=None):
        inp, c, d = self.inp, self.cfg, self.decoder
        if d is not None:       # KV-partition sharding: partial attention, exchange, merge
            if query is not None and query is not d.query:
                d.query.copy_(query, non_blocking=True)
                d.context_lens.copy_(ctx, non_blocking=True)
                d.tables.copy_(bt, non_blocking=True)
                d.step()
            elif self.step_graph is not None:
                self.step_graph.replay()
            else:
                d.step()
            return
        ws = workspaces or (None, None, None)
        self._decode(self.out if out is None else out, inp.query if query is None else query, inp.key_cache,
                     inp.value_cache, self.step_ctx if ctx is None else ctx, self.step_bt if bt is None else bt,
                     inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None, inp.key_scale,
                     inp.value_scale, partition_size=c.partition_size, status=self.status,
                     exp_sums=ws[0], max_logits=ws[1], tmp_output=ws[2])

    def partition_params(self):
        from triton_op_b200.pa_decode import build_params
        if self.decoder is not None:
            return self.decoder.params
        inp, c = self.inp, self.cfg
        p, keep = build_params(self.out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                               inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None,
                               inp.key_scale, inp.value_scale, None, c.partition_size, None, None, None, self.status, None)
        self._keep = keep
        return p

    # -- timing
    def flush(self):
        self.flush_buf.zero_()
        self.flush_buf.sum()
        if self.align is not None:
            # the ranks' flushes do not end together; without this the first rank's step would be
            # timed waiting for the last rank's flush.  (One element: it leaves L2 as the flush did.)
            import torch.distributed as dist
            dist.all_reduce(self.align)

    def timed(self, fn, n: int, flush=None) -> float:
        """Milliseconds per call of fn over n calls, on the device (CUDA events on the launching stream)."""
        ev = lambda: torch.cuda.Event(enable_timing=True)
        flush = self.flush_l2 if flush is None else flush
        torch.cuda.synchronize()
        if not flush:
            a, b = ev(), ev()
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n
        pairs = [(ev(), ev()) for _ in range(n)]
        for a, b in pairs:
            self.flush()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / n

    def check(self, n_sample: int = 3) -> dict:
        """A sampled handful of this rank's sequences against the oracle (rank 0 reports)."""
        c = self.cfg
        g = torch.Generator().manual_seed(12345)
        ids = sorted(torch.randperm(c.num_seqs, generator=g)[:min(n_sample, c.num_seqs)].tolist())
        self.call()
        torch.cuda.synchronize()
        return oracle_error(subset_inputs(self.inp, ids), self.out[ids])

    def close(self):
        if self.decoder is not None:
            self.decoder.close()


def isolated_kernel_us(fn, n: int, dev) -> float:
    """Microseconds per launch of fn with a plain (non-dependent) kernel between launches, so that no
    launch's set-up hides under its predecessor's drain."""
    spacer = torch.zeros(1 << 20, dtype=torch.float32, device=dev)
    ev = lambda: torch.cuda.Event(enable_timing=True)
    pairs = [(ev(), ev()) for _ in range(n)]
    torch.cuda.synchronize()
    for a, b in pairs:
        spacer.add_(1.0)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in pairs) / n * 1e3


def measure_extra(name: str, mode: str, exchange: str, args, rank: int, world: int, dev, steps: int) -> dict:
    """One non-headline workload: step time (device, max over ranks), KV GB/s over all ranks, the
    partition kernel's share of the copy bandwidth, parity of a sample, device status."""
    from triton_op_b200 import _lib
    t_build = time.perf_counter()
    w = Workload(name, mode, exchange, rank, world, dev, graph=not args.no_graph)
    torch.cuda.synchronize()
    t_build = time.perf_counter() - t_build
    for _ in range(3):
        w.call()
    torch.cuda.synchronize()
    barrier(world)
    ms_step = max_over_ranks(w.timed(w.call, steps), world, dev)
    barrier(world)
    p = w.partition_params()
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    ms_warm = None
    if w.flush_l2:
        # back to back: the sharded step as it is; a one-GPU call straight through the C ABI (the
        # Python operator's own time per call would be what is timed on these short workloads)
        warm_call = w.call if w.decoder is not None else (
            lambda: _lib.check(L.pa_decode_sm100(C.byref(p), stream), "pa_decode_sm100"))
        ms_warm = max_over_ranks(w.timed(warm_call, max(steps, 200) if w.decoder is None else steps, flush=False), world, dev)
        barrier(world)
    us_partition = w.timed(lambda: _lib.check(L.pa_partition_sm100(C.byref(p), stream), "pa_partition_sm100"),
                           max(5, min(steps, 50))) * 1e3
    us_partition = max_over_ranks(us_partition, world, dev)
    parity = w.check() if rank == 0 else None
    if rank != 0 and w.decoder is not None:
        w.call()                    # the sharded step is collective: every rank takes part in rank 0's check
        torch.cuda.synchronize()
    barrier(world)
    total_kv = sum_over_ranks(float(w.kv_bytes), world, dev)
    max_kv = max_over_ranks(float(w.kv_bytes), world, dev)
    dev_status = int(max_over_ranks(float(int(w.status.item())), world, dev))
    peak, _ = measured_peak()
    c = w.cfg
    res = {
        "sharding": mode if world > 1 or mode == "kv-partitions" else "one GPU",
        "us_per_call": ms_step * 1e3, "kv_gbs": total_kv / (ms_step * 1e-3) / 1e9,
        "pct_of_nominal_hbm": 100.0 * total_kv / (ms_step * 1e-3) / 1e9 / (NOMINAL_HBM_GBS * world),
        "kv_bytes_all_gpus": total_kv,
        "partition_kernel_us": us_partition,
        "partition_kernel_frac_of_copy_peak": (max_kv / (us_partition * 1e-6) / 1e9) / peak,
        "l2": "flushed before every timed step" if w.flush_l2 else "inputs larger than L2",
        "parity": parity, "device_status": dev_status, "steps": steps,
        "launch": ("CUDA graph replay" if w.step_graph is not None else "eager launches"),
        "kv": ("bf16" if c.kv_dtype == "bf16" else "fp8 e4m3fn") + ", " + c.quant.replace("_", "-") + " scales",
        "build_s": round(t_build, 1),
    }
    if ms_warm is not None:
        res["us_per_call_back_to_back"] = ms_warm * 1e3
    if mode == "kv-partitions":
        res["exchange"] = exchange if world > 1 else "none (one GPU)"
    if world > 1:
        res["token_imbalance_max_over_mean"] = max_kv / (total_kv / world)
    w.close()
    del w
    torch.cuda.empty_cache()
    return res


def measure_cache_write(dev, steps: int) -> dict:
    """The write side (quantise + scatter of new tokens into the paged caches), two slot patterns."""
    from triton_op_b200.cache_write import write_kv_cache
    from triton_op_b200.inputs import FP8
    T, hkv, bs, d = 65536, 8, 16, 128
    nb = T // bs * 2
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
        "prefill_chunks": pages[((pos // 512) * ((512 + 5 + bs - 1) // bs) + inner // bs) % nb] * bs + inner % bs,
    }
    peak, _ = measured_peak()
    nbytes = T * hkv * (2 * 2 * d + 2 * d + 8)
    out = {"tokens": T, "kv_heads": hkv, "block_size": bs, "quant": "e4m3fn per-token",
           "algorithmic_bytes": nbytes, "l2": "inputs larger than L2 (151 MB moved per call)"}
    for name, slots in patterns.items():
        for _ in range(3):
            write_kv_cache(key, value, kc, vc, slots, ks, vs)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            write_kv_cache(key, value, kc, vc, slots, ks, vs)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / steps
        out[name] = {"us_per_call": us, "gbs": nbytes / us / 1e3, "frac_of_copy_peak": nbytes / us / 1e3 / peak}
    return out


def run_ours(args, rank: int, world: int, local: int):
    from triton_op_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the operator has no CPU path")
    L = _lib.lib()  # raises when the CUDA library is missing
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    mode = args.sharding
    if mode == "auto":      # long single-head contexts split by KV partition, batches by sequence
        mode = "kv-partitions" if (args.workload == "cfg4_longctx" and world > 1) else "sequences-weak"
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()     # from before the warm-up to the end of the clock burst below
    w = Workload(args.workload, mode, args.exchange, rank, world, dev, num_seqs=args.num_seqs, graph=not args.no_graph)
    inp, c, cfg = w.inp, w.cfg, CONFIGS[args.workload]
    kv_bytes = w.kv_bytes

    # ---- device-resident inputs: K steps between two events on the launching stream
    for _ in range(args.warmup):
        w.call()
    torch.cuda.synchronize()
    barrier(world)
    ms_step = max_over_ranks(w.timed(w.call, args.steps), world, dev)
    barrier(world)
    ms_warm = None      # small workloads: also back to back, KV partly in L2 (reported beside the cold number)
    if w.flush_l2:
        ms_warm = max_over_ranks(w.timed(w.call, args.steps, flush=False), world, dev)
        barrier(world)

    # ---- the partition kernel alone (the dominant kernel) for the roofline: back to back (every
    # launch a programmatic dependent of the one before, as in a decode loop) and isolated
    p = w.partition_params()
    stream = torch.cuda.current_stream().cuda_stream
    launch_partition = lambda: _lib.check(L.pa_partition_sm100(C.byref(p), stream), "pa_partition_sm100")
    n_k = max(20, min(args.steps, 200))
    us_partition = w.timed(launch_partition, n_k) * 1e3
    us_partition_iso = isolated_kernel_us(launch_partition, n_k, dev) if not w.flush_l2 else us_partition

    # ---- read-only streaming ceiling: the same number of bytes through bulk copies, nothing computed
    read_ceiling = None
    kc, vc = inp.key_cache, inp.value_cache
    each = min(kc.numel() * kc.element_size(), vc.numel() * vc.element_size(), kv_bytes // 2) // 8192 * 8192
    if each >= L2_BYTES:
        probe = lambda: _lib.check(L.pa_stream_probe_sm100(kc.data_ptr(), vc.data_ptr(), each, w.status.data_ptr(), stream),
                                   "pa_stream_probe_sm100")
        for _ in range(3):
            probe()
        us_probe = w.timed(probe, n_k, flush=False) * 1e3
        read_ceiling = {"gbs": 2 * each / us_probe / 1e3, "us": us_probe, "bytes": 2 * each,
                        "how": "pa_stream_probe_sm100: 2 KB bulk copies into shared-memory rings, one CTA per SM, no compute"}

    # ---- clock burst: the same call back to back for long enough that the 20 ms sampler sees load
    burst_us = None
    if rank == 0 or world > 1:
        n_burst = int(min(20000, max(args.steps, args.burst_seconds / max(ms_step * 1e-3, 1e-6))))
        burst_us = w.timed(w.call, n_burst, flush=False) * 1e3
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: the step's inputs arrive from pinned host memory, the output goes back.
    # Query, context lengths and block tables travel as ONE staging buffer (one H2D copy per step).
    parts = [inp.query, w.step_ctx, w.step_bt]
    offs, total = [], 0
    for t in parts:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256

    def view(buf, t, off):
        n = t.numel() * t.element_size()
        return buf[off:off + n].view(t.dtype).view(t.shape)

    class Slot:     # one in-flight step: staging buffers, outputs and (for the pipelined loop) its own workspaces
        def __init__(self, own_workspaces: bool):
            self.hbuf = torch.empty(total, dtype=torch.uint8).pin_memory()
            self.dbuf = torch.empty(total, dtype=torch.uint8, device=dev)
            for t, off in zip(parts, offs):
                view(self.hbuf, t, off).copy_(t)
            self.dq, self.dctx, self.dbt = (view(self.dbuf, t, off) for t, off in zip(parts, offs))
            self.out = w.out if not own_workspaces else torch.empty_like(w.out)
            self.hout = torch.empty_like(w.out, device="cpu").pin_memory()
            self.ws = None
            if own_workspaces and w.decoder is None:
                eqg = c.q_heads // c.kv_heads * c.query_len
                P = (inp.max_context + c.partition_size - 1) // c.partition_size
                shape = (c.num_seqs, c.kv_heads, P, eqg)
                self.ws = (torch.zeros(shape, dtype=torch.float32, device=dev), torch.zeros(shape, dtype=torch.float32, device=dev),
                           torch.zeros(shape + (c.head_size,), dtype=torch.bfloat16, device=dev))
            self.graph = None
            self.stream = torch.cuda.current_stream()
            self.done = torch.cuda.Event()

        def body(self):
            self.dbuf.copy_(self.hbuf, non_blocking=True)
            if w.decoder is not None:
                w.call(self.dq, self.dctx, self.dbt)
            else:
                w.call(self.dq, self.dctx, self.dbt, out=self.out, workspaces=self.ws)
            self.hout.copy_(self.out, non_blocking=True)

        def capture(self):
            # The step (copy in, the operator's public call, copy out) is captured once in a CUDA graph and
            # replayed per step, as a serving loop would: the operator allocates nothing and does not
            # synchronise, so it is capturable.  Without NCCL in the step; falls back to eager launches.
            if w.decoder is not None or args.no_graph:
                return
            try:
                for _ in range(2):
                    self.body()          # warm the parameter and workspace caches outside the capture
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.body()
                self.graph = g
            except Exception as exc:      # capture refused: measure the eager path
                sys.stderr.write(f"bench.py: CUDA graph capture of the e2e step failed ({exc}); using eager launches\n")
                self.graph = None
                torch.cuda.synchronize()

        def launch(self):
            if self.graph is not None:
                self.graph.replay()
            else:
                self.body()

    serial = Slot(own_workspaces=False)
    serial.capture()

    def e2e_step():
        serial.launch()
        torch.cuda.current_stream().synchronize()   # the caller reads the result every step

    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    barrier(world)
    torch.cuda.synchronize()
    ev = lambda: torch.cuda.Event(enable_timing=True)
    if not w.flush_l2:
        t0 = time.perf_counter()
        g0, g1 = ev(), ev()
        g0.record()
        for _ in range(args.steps):
            e2e_step()
        g1.record()
        torch.cuda.synchronize()
        ms_e2e = max(g0.elapsed_time(g1), (time.perf_counter() - t0) * 1e3) / args.steps
    else:       # the flush stays outside the timed region: every step is clocked on its own
        spent = 0.0
        for _ in range(args.steps):
            w.flush()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e2e_step()
            spent += time.perf_counter() - t0
        ms_e2e = spent * 1e3 / args.steps
    ms_e2e = max_over_ranks(ms_e2e, world, dev)
    h2d = total
    d2h = serial.hout.numel() * serial.hout.element_size()

    # ---- the same loop two steps deep: two independent batches take turns, each with its own
    # staging buffers, output and workspaces and its own stream, so one batch's copies run under the
    # other's kernels; the host reads a result one step after it issued it.
    ms_e2e_pipe = None
    if w.decoder is None and not w.flush_l2 and not args.no_graph:
        slots = []
        streams = [torch.cuda.Stream(device=dev) for _ in range(2)]
        for s in streams:
            with torch.cuda.stream(s):
                sl = Slot(own_workspaces=True)
                sl.stream = s
                sl.capture()
                slots.append(sl)
        torch.cuda.synchronize()

        def pipe(n):
            for k in range(n + 1):
                if k < n:
                    sl = slots[k % 2]
                    with torch.cuda.stream(sl.stream):
                        sl.launch()
                        sl.done.record(sl.stream)
                if k >= 1:
                    slots[(k - 1) % 2].done.synchronize()   # the host reads step k-1's result

        pipe(4)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        pipe(args.steps)
        torch.cuda.synchronize()
        ms_e2e_pipe = max_over_ranks((time.perf_counter() - t0) * 1e3 / args.steps, world, dev)

    parity = w.check() if (rank == 0 and args.num_seqs == 0) else None
    if rank != 0 and w.decoder is not None and args.num_seqs == 0:
        w.call()
        torch.cuda.synchronize()
    barrier(world)
    total_kv = sum_over_ranks(float(kv_bytes), world, dev)
    dev_status = int(max_over_ranks(float(int(w.status.item())), world, dev))
    launches_per_step = 2 if w.decoder is None else w.decoder.launches_per_step
    value_launch = "CUDA graph replay of the sharded step" if w.step_graph is not None else "eager launches"
    e2e_launch = ("CUDA graph replay of (copy in, paged_attention_decode, copy out)" if serial.graph is not None
                  else "eager launches")
    flush_l2 = w.flush_l2
    w.close()
    del w, serial
    torch.cuda.empty_cache()

    # ---- the other workloads, in the same process
    workloads = None
    if not args.no_workloads and args.num_seqs == 0:
        workloads = {}
        steps_x = max(5, min(args.steps, 50))
        if world == 1:
            specs = [(n, "sequences-weak", "p2p") for n in CONFIGS if n != args.workload]
        else:
            specs = [("cfg4_longctx", "kv-partitions", "p2p"), ("cfg4_longctx", "kv-partitions", "nccl"),
                     ("cfg5_serving_fp8", "sequences-strong", "p2p"), ("cfg5_serving_bf16", "sequences-strong", "p2p"),
                     ("cfg3_llama70b_mtp", "sequences-strong", "p2p")]
        for name, m, ex in specs:
            key = name if m != "kv-partitions" or world == 1 else f"{name}/{ex}"
            try:
                workloads[key] = measure_extra(name, m, ex, args, rank, world, dev, steps_x)
            except Exception as exc:  # noqa: BLE001 - the headline line must still be printed
                workloads[key] = {"error": f"{type(exc).__name__}: {exc}"}
                torch.cuda.empty_cache()
        if world == 1:
            try:
                workloads["cache_write"] = measure_cache_write(dev, steps_x)
            except Exception as exc:  # noqa: BLE001
                workloads["cache_write"] = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        return
    peak, peak_kind = measured_peak()
    achieved = kv_bytes / (us_partition * 1e-6) / 1e9
    value = total_kv / (ms_step * 1e-3) / 1e9

    # ---- CPU baseline on a bounded sample of the same workload (rank 0, N = 1 only)
    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        sample = 8
        sub = type(cfg)(**{**cfg.__dict__, "num_seqs": sample, "pool_blocks": None})
        cpu_inp = make_inputs(sub, seed=0, device="cpu")
        torch.set_num_threads(max(1, os.cpu_count() or 1))
        cpu_reference_time(cpu_inp, sample)
        t_cpu, kvb_cpu, threads = cpu_reference_time(cpu_inp, sample, repeats=3)
        cpu_baseline = {"value": kvb_cpu / t_cpu / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"first {sample} of {cfg.num_seqs} sequences ({kvb_cpu} KV bytes), best of 3, "
                                  f"oracle/pa_oracle.py with torch CPU threads"}

    roofline = {"bound": "hbm", "kernel": "partition kernel (pa_partition_sm100)", "achieved": achieved, "peak": peak,
                "peak_kind": peak_kind + " (torch copy_, read+write)", "unit": "GB/s", "frac": achieved / peak,
                "us_per_launch": us_partition, "algorithmic_bytes": kv_bytes,
                "traffic": (NCU_TRAFFIC_PER_KV_BYTE[args.workload] * kv_bytes)
                           if args.workload in NCU_TRAFFIC_PER_KV_BYTE else None,
                "us_per_launch_isolated": us_partition_iso, "frac_isolated": kv_bytes / (us_partition_iso * 1e-6) / 1e9 / peak,
                "note": "us_per_launch: launches back to back, each a programmatic dependent of the one before (its set-up "
                        "overlaps the predecessor's drain, as in a decode loop); us_per_launch_isolated: a plain kernel "
                        "between launches, nothing overlaps"}
    if read_ceiling is not None:
        roofline["read_only_ceiling"] = read_ceiling
        roofline["frac_of_read_only_ceiling"] = achieved / read_ceiling["gbs"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "us_per_call": ms_step * 1e3,
        "higher_is_better": True, "scaling": "weak" if mode == "sequences-weak" else "strong", "vs_baseline": None,
        "dtype": "bf16 x bf16 -> f32" if c.kv_dtype == "bf16" else "e4m3 x e4m3 -> f32",
        "data": "synthetic",
        "pct_of_nominal_hbm": 100.0 * value / (NOMINAL_HBM_GBS * world),
        "call_frac_of_read_only_ceiling": (value / world / read_ceiling["gbs"]) if read_ceiling else None,
        "config": {"workload": args.workload, "num_seqs_per_gpu": c.num_seqs, "q_heads": c.q_heads,
                   "kv_heads": c.kv_heads, "head_size": c.head_size, "block_size": c.block_size,
                   "query_len": c.query_len, "context_len": inp.max_context if c.context[0] == "fixed" else str(c.context),
                   "kv": ("bf16" if c.kv_dtype == "bf16" else "fp8 e4m3fn") + ", " + c.quant.replace("_", "-") + " scales",
                   "partition_size": c.partition_size, "kv_bytes_per_gpu": kv_bytes,
                   "l2": ("L2 flushed (256 MB written, then read) before every timed step; KV read per step: %.1f MB per GPU"
                          if flush_l2 else "inputs larger than L2 (KV read per step: %.0f MB per GPU)") % (kv_bytes / 1e6),
                   "sharding": {"sequences-weak": "sequences, one full batch per GPU, no collective",
                                "sequences-strong": "one batch, sequences dealt out by token count, no collective",
                                "kv-partitions": "KV partition ranges per GPU; (max, sum, out) triples exchanged ("
                                                 + args.exchange + ") and merged"}[mode]},
        "roofline": roofline,
        "cpu_baseline": cpu_baseline,
        "l2_warm": None if ms_warm is None else {"us_per_call": ms_warm * 1e3, "value": total_kv / (ms_warm * 1e-3) / 1e9,
                                                 "unit": UNIT, "note": "the same steps back to back without the L2 flush"},
        "value_launch": value_launch,
        "e2e": {"value": total_kv / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "us_per_call": ms_e2e * 1e3,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "launch": e2e_launch,
                "note": "query, block tables and context lengths from pinned host memory (one staging copy), output copied back, "
                        "the host waits for every result before the next step; the KV cache is resident state, as in serving",
                "pipelined": None if ms_e2e_pipe is None else {
                    "value": total_kv / (ms_e2e_pipe * 1e-3) / 1e9, "unit": UNIT, "us_per_call": ms_e2e_pipe * 1e3,
                    "note": "two independent batches take turns on two streams (own staging buffers, outputs and workspaces): "
                            "one's copies run under the other's kernels; every result is read by the host one step later"}},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": dict(clocks or {}, burst_us_per_call=burst_us,
                       note="sampled every 20 ms from before the warm-up to the end of a burst of the same call back to back"),
        "parity": parity,
        "device_status": dev_status,
        "workloads": workloads,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2_llama8b", choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="headline only: skip the other workloads")
    ap.add_argument("--sharding", default="auto",
                    choices=["auto", "sequences-weak", "sequences-strong", "kv-partitions"],
                    help="multi-GPU split; auto = KV partitions for the long-context workload, else one batch per GPU")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="KV-partition sharding: triples exchanged by NVLink peer stores or by an NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true", help="run the e2e step with eager launches instead of a CUDA graph")
    ap.add_argument("--burst-seconds", type=float, default=0.6,
                    help="length of the back-to-back burst the clock sampler watches (0 for profiler captures)")
    ap.add_argument("--num-seqs", type=int, default=0,
                    help="override the workload's batch size (profiler captures of the large workloads)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        run_reference_arm(args, rank, int(os.environ.get("WORLD_SIZE", "1")))
        return
    rank, world, local = dist_setup(args.gpus)
    try:
        run_ours(args, rank, world, local)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
