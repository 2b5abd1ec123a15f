"""The NVLink peer-store exchange of KV-partition-sharded decode, on two GPUs of one node (skipped
with fewer).  Every rank decodes its ranges, its reduce stores the triples into both ranks' buffers, and
both merge; both must end up with the single-GPU result.  A second case leaves one rank's push out
and checks that the other's bounded wait gives up with PA_DEV_WAIT_TIMEOUT instead of hanging."""
from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, ret):
    import torch.distributed as dist
    from triton_op_b200 import _lib
    from triton_op_b200.inputs import DecodeConfig, make_inputs, pack_mtp
    from triton_op_b200.sharding import KvShardedDecoder, PeerExchange, plan_kv_shards
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from _util import oracle_output

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device(f"cuda:{rank}")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        cfg = DecodeConfig("p2p", 3, 8, 1, 16, 1, ("fixed", 1))
        lens = [9000, 513, 2300]
        inp = make_inputs(cfg, seed=3, device=dev, context_lens=torch.tensor(lens))     # same seed: same pool on both
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        plan = plan_kv_shards(lens, world, 256, 1)[rank]
        dec = KvShardedDecoder(inp.query, inp.key_cache, inp.value_cache, plan, inp.block_tables, inp.softmax_scale,
                               inp.key_scale, inp.value_scale, partition_size=256, status=status, exchange="p2p")
        want = pack_mtp(oracle_output(inp), 3, 1, 1).float()
        worst = 0.0
        for _ in range(3):                      # several steps: both buffer parities, growing epochs
            out = dec.step()
            torch.cuda.synchronize()
            worst = max(worst, float((out.float() - want).abs().max()))
        graph = dec.capture()                   # the step number is counted on the device: replays stay in step
        for _ in range(3):
            dec.out.zero_()
            graph.replay()
            torch.cuda.synchronize()
            worst = max(worst, float((dec.out.float() - want).abs().max()))
        ret[f"err{rank}"] = worst
        ret[f"status{rank}"] = int(status.item())
        dist.barrier()
        # bounded wait: rank 1 does not push this step; rank 0's merge must give up, not hang
        ex = PeerExchange(dec._rows, 128, dev)
        st2 = torch.zeros(1, dtype=torch.int32, device=dev)
        if rank == 0:
            ex.reduce_push(dec.params)
            ex.merge(dec.out, st2)
            torch.cuda.synchronize()
            ret["timeout_status"] = int(st2.item())
        dist.barrier()
        ex.close()
        dec.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_peer_store_exchange_on_two_gpus():
    import torch.multiprocessing as mp
    from triton_op_b200 import _lib
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert ret["err0"] < 2e-2 and ret["err1"] < 2e-2, dict(ret)
    assert ret["status0"] == 0 and ret["status1"] == 0
    assert ret["timeout_status"] == _lib.PA_DEV_WAIT_TIMEOUT
