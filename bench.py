#!/usr/bin/env python
"""Benchmark of the paged-attention decode operator.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

A step is one decode call (partition kernel + reduce kernel) over one batch of synthetic input.
The workload at every N is the Llama-3-8B-shaped configuration the headline metric is quoted on
(64 sequences x 4096 tokens, 32 query / 8 kv heads, fp8 KV, 16-token pages) per GPU: sequences
are independent, so ranks shard the batch with no collective and the scaling is weak.

One JSON line is printed by rank 0:
  value      KV bytes all ranks read per step / device time of the step (max over ranks), inputs
             resident in HBM;
  e2e        the same metric through the public entry point with the step's inputs (query, block
             tables, context lengths) coming from pinned host memory and the output copied back;
  roofline   the partition kernel alone against the measured HBM copy bandwidth;
  cpu_baseline  the oracle (a CPU port of the reference's own PyTorch path) on a bounded sample.
`--impl reference` times that CPU path as the reference arm (rank 0 only).
"""
from __future__ import annotations

import argparse
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

from triton_op_b200.inputs import CONFIGS, make_inputs  # noqa: E402

METRIC = "kv_read_hbm_bandwidth"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one partition-kernel launch divided by the
# algorithmic KV bytes of that launch, per workload, from the ncu captures summarised under
# profiles/ (captured on the workload itself or on fewer of its sequences; traffic grows in
# proportion to the sequences).  Workloads without a capture report no traffic.
L2_BYTES = 126 << 20     # B200

NCU_TRAFFIC_PER_KV_BYTE = {"cfg2_llama8b": 1.024, "cfg3_llama70b_mtp": 1.07, "cfg4_longctx": 1.036}


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

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
        mhz, mx, reasons = [], None, set()
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
            if clk > 0.5 * mx:  # samples taken while the GPU was under load
                mhz.append(clk)
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx,
                "samples_under_load": len(mhz), "reasons": sorted(reasons)}


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


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


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
                         "sample": f"{sample} sequences ({kvb} KV bytes) per step, oracle/pa_oracle.py on host cores"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm
def run_ours(args, rank: int, world: int, local: int):
    import ctypes as C
    from triton_op_b200 import _lib, paged_attention_decode
    from triton_op_b200.pa_decode import build_params

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the operator has no CPU path")
    _lib.lib()  # raises when the CUDA library is missing
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    cfg = CONFIGS[args.workload]
    if args.num_seqs > 0:   # reduced batch: for profiler captures, never for a reported number
        cfg = type(cfg)(**{**cfg.__dict__, "num_seqs": args.num_seqs, "pool_blocks": None})
    mode = args.sharding
    if mode == "auto":      # long single-head contexts split by KV partition, batches by sequence
        mode = "kv-partitions" if (args.workload == "cfg4_longctx" and world > 1) else "sequences-weak"
    status = torch.zeros((), dtype=torch.int32, device=dev)
    decoder = None
    if mode == "sequences-weak":
        inp = make_inputs(cfg, seed=rank, device=dev)      # every rank its own batch of the full size
    elif mode == "sequences-strong":
        # one global batch; every rank computes the same plan and builds only its own sequences
        from triton_op_b200.inputs import draw_context_lens
        from triton_op_b200.sharding import shard_sequences
        gen = torch.Generator()
        gen.manual_seed(0)
        lens = draw_context_lens(cfg, gen)
        policy = "balanced" if cfg.context[0] == "lognormal" else "contiguous"
        mine = shard_sequences(lens.tolist(), world, policy)[rank]
        sub = type(cfg)(**{**cfg.__dict__, "num_seqs": len(mine), "pool_blocks": None})
        inp = make_inputs(sub, seed=rank, device=dev, context_lens=lens[mine])
    else:
        # every rank builds the same pool (same seed) and reads only the pages of its ranges
        from triton_op_b200.sharding import KvShardedDecoder, plan_kv_shards
        inp = make_inputs(cfg, seed=0, device=dev)
        plan = plan_kv_shards(inp.context_lens.tolist(), world, cfg.partition_size, cfg.query_len)[rank]
        decoder = KvShardedDecoder(inp.query, inp.key_cache, inp.value_cache, plan, inp.block_tables,
                                   inp.softmax_scale, inp.key_scale, inp.value_scale,
                                   partition_size=cfg.partition_size, status=status, exchange=args.exchange)
    c = inp.cfg
    out = torch.empty_like(inp.query) if decoder is None else decoder.out

    def call(query, ctx, bt):
        if decoder is not None:       # KV-partition sharding: partial attention, all-gather, merge
            if query is not decoder.query:
                decoder.query.copy_(query, non_blocking=True)
                decoder.context_lens.copy_(ctx, non_blocking=True)
                decoder.tables.copy_(bt, non_blocking=True)
                decoder.step()
            elif step_graph is not None:
                step_graph.replay()
            else:
                decoder.step()
            return
        paged_attention_decode(out, query, inp.key_cache, inp.value_cache, ctx, bt, inp.softmax_scale,
                               c.query_len, inp.max_context, torch.bfloat16, None, inp.key_scale,
                               inp.value_scale, partition_size=c.partition_size, status=status)

    kv_bytes = inp.kv_bytes if decoder is None else decoder.kv_bytes
    step_ctx = inp.context_lens if decoder is None else decoder.context_lens
    step_bt = inp.block_tables if decoder is None else decoder.tables
    ev = lambda: torch.cuda.Event(enable_timing=True)

    # ---- device-resident inputs: K steps between two events on the launching stream.
    # The KV-partition-sharded step is three short launches; replayed as one CUDA graph, or the
    # host's launch rate is what gets timed.
    step_graph = None
    if decoder is not None and not args.no_graph:
        try:
            step_graph = decoder.capture()
        except Exception as exc:  # noqa: BLE001 - eager launches are still a valid measurement
            sys.stderr.write(f"bench.py: CUDA graph capture of the sharded step failed ({exc}); using eager launches\n")
            step_graph = None
    for _ in range(args.warmup):
        call(inp.query, step_ctx, step_bt)
    torch.cuda.synchronize()
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # A step that reads less than about twice the L2 would find its KV there on the next iteration:
    # then L2 is flushed before every timed step (a 256 MB write, then a read of the same buffer so
    # that the step does not also pay for writing 126 MB of the flush's dirty lines back) and the
    # steps are timed one by one.
    flush_l2 = kv_bytes < 2 * L2_BYTES
    flush_buf = torch.empty(64 << 20, dtype=torch.int32, device=dev) if flush_l2 else None

    align = torch.zeros(1, dtype=torch.float32, device=dev) if (flush_l2 and world > 1) else None

    def flush():
        flush_buf.zero_()
        flush_buf.sum()
        if align is not None:
            # the ranks' flushes do not end together; without this the first rank's step would be
            # timed waiting for the last rank's flush.  (One element: it leaves L2 as the flush did.)
            import torch.distributed as dist
            dist.all_reduce(align)

    def timed_steps(fn, n):
        """Milliseconds per call of fn over n calls, on the device."""
        torch.cuda.synchronize()
        if not flush_l2:
            a, b = ev(), ev()
            a.record()
            for _ in range(n):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / n
        pairs = [(ev(), ev()) for _ in range(n)]
        for a, b in pairs:
            flush()
            a.record()
            fn()
            b.record()
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in pairs) / n

    ms_step = max_over_ranks(timed_steps(lambda: call(inp.query, step_ctx, step_bt), args.steps), world, dev)
    barrier(world)
    ms_warm = None      # small workloads: also back to back, KV partly in L2 (reported beside the cold number)
    if flush_l2:
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        for _ in range(args.steps):
            call(inp.query, step_ctx, step_bt)
        b.record()
        torch.cuda.synchronize()
        ms_warm = max_over_ranks(a.elapsed_time(b) / args.steps, world, dev)
        barrier(world)

    # ---- the partition kernel alone (the dominant kernel) for the roofline
    if decoder is None:
        p, keep = build_params(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                               inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None,
                               inp.key_scale, inp.value_scale, None, c.partition_size, None, None, None, status, None)
    else:
        p = decoder.params
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    n_k = max(20, min(args.steps, 200))
    us_partition = timed_steps(lambda: _lib.check(L.pa_partition_sm100(C.byref(p), stream), "pa_partition_sm100"),
                               n_k) * 1e3
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: the step's inputs arrive from pinned host memory, the output goes back.
    # Query, context lengths and block tables travel as ONE staging buffer (one H2D copy per step).
    parts = [inp.query, step_ctx, step_bt]
    offs, total = [], 0
    for t in parts:
        offs.append(total)
        total += (t.numel() * t.element_size() + 255) // 256 * 256
    hbuf = torch.empty(total, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(total, dtype=torch.uint8, device=dev)

    def view(buf, t, off):
        n = t.numel() * t.element_size()
        return buf[off:off + n].view(t.dtype).view(t.shape)

    for t, off in zip(parts, offs):
        view(hbuf, t, off).copy_(t)
    dq, dctx, dbt = (view(dbuf, t, off) for t, off in zip(parts, offs))
    hout = torch.empty_like(out, device="cpu").pin_memory()

    def e2e_body():
        dbuf.copy_(hbuf, non_blocking=True)
        call(dq, dctx, dbt)
        hout.copy_(out, non_blocking=True)

    # The step (copy in, the operator's public call, copy out) is captured once in a CUDA graph and
    # replayed per step, as a serving loop would: the operator allocates nothing and does not
    # synchronise, so it is capturable.  Without NCCL in the step; falls back to eager launches.
    e2e_graph = None
    if decoder is None and not args.no_graph:
        try:
            for _ in range(2):
                e2e_body()          # warm the parameter and workspace caches outside the capture
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                e2e_body()
            e2e_graph = g
        except Exception as exc:      # capture refused: measure the eager path
            sys.stderr.write(f"bench.py: CUDA graph capture of the e2e step failed ({exc}); using eager launches\n")
            e2e_graph = None
            torch.cuda.synchronize()

    def e2e_step():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            e2e_body()
        torch.cuda.current_stream().synchronize()   # the caller reads the result every step

    for _ in range(max(3, args.warmup // 2)):
        e2e_step()
    barrier(world)
    torch.cuda.synchronize()
    if not flush_l2:
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
            flush()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            e2e_step()
            spent += time.perf_counter() - t0
        ms_e2e = spent * 1e3 / args.steps
    ms_e2e = max_over_ranks(ms_e2e, world, dev)
    h2d = total
    d2h = hout.numel() * hout.element_size()

    total_kv = sum_over_ranks(float(kv_bytes), world, dev)
    dev_status = int(status.item())
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

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "us_per_call": ms_step * 1e3,
        "higher_is_better": True, "scaling": "weak" if mode == "sequences-weak" else "strong", "vs_baseline": None,
        "dtype": "bf16 x bf16 -> f32" if c.kv_dtype == "bf16" else "e4m3 x e4m3 -> f32",
        "data": "synthetic",
        "pct_of_nominal_hbm": 100.0 * value / (NOMINAL_HBM_GBS * world),
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
        "roofline": {"bound": "hbm", "kernel": "partition kernel (pa_partition_sm100)", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind + " (torch copy_, read+write)", "unit": "GB/s", "frac": achieved / peak,
                     "us_per_launch": us_partition, "algorithmic_bytes": kv_bytes,
                     "traffic": (NCU_TRAFFIC_PER_KV_BYTE[args.workload] * kv_bytes)
                                if args.workload in NCU_TRAFFIC_PER_KV_BYTE else None},
        "cpu_baseline": cpu_baseline,
        "l2_warm": None if ms_warm is None else {"us_per_call": ms_warm * 1e3, "value": total_kv / (ms_warm * 1e-3) / 1e9,
                                                 "unit": UNIT, "note": "the same steps back to back without the L2 flush"},
        "value_launch": "CUDA graph replay of the sharded step" if step_graph is not None else "eager launches",
        "e2e": {"value": total_kv / (ms_e2e * 1e-3) / 1e9, "unit": UNIT, "us_per_call": ms_e2e * 1e3,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "launch": "CUDA graph replay of (copy in, paged_attention_decode, copy out)" if e2e_graph is not None
                          else "eager launches",
                "note": "query, block tables and context lengths from pinned host memory (one staging copy), output copied back; "
                        "the KV cache is resident state, as in serving"},
        "gpu_launches": (2 if decoder is None else decoder.launches_per_step) * args.steps,
        "clocks": clocks,
        "device_status": dev_status,
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
    ap.add_argument("--sharding", default="auto",
                    choices=["auto", "sequences-weak", "sequences-strong", "kv-partitions"],
                    help="multi-GPU split; auto = KV partitions for the long-context workload, else one batch per GPU")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="KV-partition sharding: triples exchanged by NVLink peer stores or by an NCCL all-gather")
    ap.add_argument("--no-graph", action="store_true", help="run the e2e step with eager launches instead of a CUDA graph")
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
