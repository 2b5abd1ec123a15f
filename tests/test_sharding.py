"""Multi-GPU host logic on CPU: sequence sharding, KV-partition sharding, and the triple exchange
over a two-process ``gloo`` group.  The attention arithmetic on this path is the oracle's; the
CUDA kernels that produce and merge triples on a GPU are covered by the GPU tests."""
from __future__ import annotations

import os
import socket

import pytest
import torch

from triton_op_b200.inputs import CONFIGS, DecodeConfig, draw_context_lens, make_inputs
from triton_op_b200.sharding import (KvShard, gather_and_merge, local_block_table, plan_kv_shards,
                                     shard_sequences, shard_token_counts)


# ----------------------------------------------------------------------------- sequences
def test_contiguous_sharding_covers_every_sequence_once():
    lens = list(range(1, 38))
    for world in (1, 2, 3, 4, 8):
        shards = shard_sequences(lens, world, "contiguous")
        assert sorted(i for s in shards for i in s) == list(range(len(lens)))
        sizes = [len(s) for s in shards]
        assert max(sizes) - min(sizes) <= 1
        assert all(s == list(range(s[0], s[-1] + 1)) for s in shards if s)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_balanced_sharding_of_the_serving_mix(world):
    cfg = CONFIGS["cfg5_serving_fp8"]
    gen = torch.Generator()
    gen.manual_seed(0)
    lens = draw_context_lens(cfg, gen).tolist()
    shards = shard_sequences(lens, world, "balanced")
    assert sorted(i for s in shards for i in s) == list(range(cfg.num_seqs))
    tokens = shard_token_counts(lens, shards)
    assert sum(tokens) == sum(lens)
    mean = sum(tokens) / world
    assert max(tokens) <= 1.01 * mean, (tokens, mean)        # 1024 lognormal sequences balance to < 1 %
    contiguous = shard_token_counts(lens, shard_sequences(lens, world, "contiguous"))
    assert max(tokens) <= max(contiguous)
    assert shards == shard_sequences(lens, world, "balanced")  # deterministic: every rank computes the same plan


def test_balanced_sharding_edge_cases():
    assert shard_sequences([], 4) == [[], [], [], []]
    assert shard_sequences([5], 3) == [[0], [], []]
    assert shard_sequences([7, 7, 7, 7], 2) == [[0, 2], [1, 3]]
    with pytest.raises(ValueError):
        shard_sequences([1], 0)
    with pytest.raises(ValueError):
        shard_sequences([1], 2, "random")


# ----------------------------------------------------------------------------- KV partitions
@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("psize", [256, 512])
def test_kv_plan_covers_each_context_in_partition_multiples(world, psize):
    lens = [0, 1, 255, 256, 257, 511, 513, 4096, 32768, 65536, 131072, 100000]
    plan = plan_kv_shards(lens, world, psize, query_len=1)
    assert len(plan) == world and all(len(p) == len(lens) for p in plan)
    for s, ctx in enumerate(lens):
        pos = 0
        sizes = []
        for r in range(world):
            sh = plan[r][s]
            assert sh.begin == pos or sh.tokens == 0
            if sh.tokens:
                assert sh.begin % psize == 0
                pos = sh.end
            sizes.append((sh.tokens + psize - 1) // psize)
        assert pos == ctx
        assert max(sizes) - min(sizes) <= 1        # partitions dealt out evenly


def test_kv_plan_keeps_the_causal_tail_in_one_range():
    # 513 tokens, partition 256, three ranks: the last partition holds one token, fewer than the
    # query_len - 1 = 3 keys the causal rule can hide, so it joins the previous range
    plan = plan_kv_shards([513], 3, 256, query_len=4)
    got = [(p[0].begin, p[0].end) for p in plan]
    assert got == [(0, 256), (256, 513), (513, 513)]
    assert [p[0].local_query_len for p in plan] == [1, 4, 4]
    assert plan[0][0].holds_tail is False and plan[1][0].holds_tail is True
    # with query_len = 1 nothing moves
    plan = plan_kv_shards([513], 3, 256, query_len=1)
    assert [(p[0].begin, p[0].end) for p in plan] == [(0, 256), (256, 512), (512, 513)]


def test_local_block_table_slices_the_range():
    bt = torch.arange(80, dtype=torch.int32).view(2, 40) + 100
    shards = [KvShard(256, 512, 600, 1), KvShard(0, 40, 40, 1)]
    loc = local_block_table(bt, shards, 16)
    assert loc.shape == (2, 16)
    assert loc[0].tolist() == list(range(116, 132))
    assert loc[1, :3].tolist() == [140, 141, 142] and loc[1, 3:].abs().sum() == 0
    with pytest.raises(ValueError):
        local_block_table(bt, [KvShard(8, 24, 600, 1), KvShard(0, 0, 0, 1)], 16)


# ----------------------------------------------------------------------------- the merge, oracle arithmetic
def _rank_triples(inp, shards, partition_size):
    """(m, l, o) of one rank's ranges, by the oracle: partition outputs, then merged over partitions."""
    from oracle import pa_oracle
    c = inp.cfg
    tables = local_block_table(inp.block_tables, shards, c.block_size)
    ks, vs = inp.flat_scales()
    S, rows, D = inp.query.shape
    m_out = torch.full((S, rows), float("-inf"))
    l_out = torch.zeros((S, rows))
    o_out = torch.zeros((S, rows, D))
    for kind in sorted({sh.local_query_len for sh in shards}):
        lens = torch.tensor([sh.local_context_len if sh.local_query_len == kind else 0 for sh in shards],
                            dtype=torch.int32)
        if int(lens.sum()) == 0:
            continue
        m, l, o = pa_oracle.split_kv_partials(inp.query, inp.key_cache, inp.value_cache, tables, lens, kind,
                                              inp.softmax_scale, partition_size, ks, vs)
        M = m.max(dim=2).values                                              # [S, Hkv, eqG]
        M_safe = torch.where(torch.isinf(M), torch.zeros_like(M), M)
        W = (l * torch.exp(m - M_safe[:, :, None])).nan_to_num(0.0).sum(dim=2)
        O = pa_oracle.merge_partials(m, l, o)                                # [S, Hkv, eqG, D]
        for s, sh in enumerate(shards):
            if sh.local_query_len == kind and sh.tokens > 0:
                m_out[s], l_out[s], o_out[s] = M[s].reshape(-1), W[s].reshape(-1), O[s].reshape(rows, D)
    return m_out.reshape(-1), l_out.reshape(-1), o_out.reshape(-1, D)


def _full_output(inp):
    from oracle import pa_oracle
    from triton_op_b200.inputs import pack_mtp
    ks, vs = inp.flat_scales()
    ref = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables,
                                    inp.context_lens, inp.query_indptr(), ks, vs)
    return pack_mtp(ref, inp.cfg.num_seqs, inp.cfg.query_len, inp.cfg.kv_heads).float()


_KV_CASES = {
    "decode": (DecodeConfig("kvshard", 3, 8, 2, 16, 1, ("fixed", 1)), [2300, 700, 256]),
    "mtp3": (DecodeConfig("kvshard_mtp", 4, 8, 2, 16, 3, ("fixed", 1), quant="per_token"), [1500, 513, 258, 40]),
}


@pytest.mark.parametrize("case", sorted(_KV_CASES))
@pytest.mark.parametrize("world", [2, 3])
def test_kv_sharded_attention_equals_full_attention(case, world):
    from oracle import pa_oracle
    cfg, lens = _KV_CASES[case]
    inp = make_inputs(cfg, seed=5, device="cpu", context_lens=torch.tensor(lens))
    plan = plan_kv_shards(lens, world, 256, cfg.query_len)
    triples = [_rank_triples(inp, plan[r], 256) for r in range(world)]
    merged = pa_oracle.merge_triples(torch.stack([t[0] for t in triples]), torch.stack([t[1] for t in triples]),
                                     torch.stack([t[2] for t in triples]))
    want = _full_output(inp).reshape(-1, cfg.head_size)
    assert torch.allclose(merged, want, atol=2e-2, rtol=1e-2)      # `want` went through a bf16 rounding
    assert (merged - want).abs().max() < 8e-3


# ----------------------------------------------------------------------------- two gloo ranks
def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_rank(rank: int, world: int, port: int, case: str, ret):
    import torch.distributed as dist
    from oracle import pa_oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg, lens = _KV_CASES[case]
        inp = make_inputs(cfg, seed=5, device="cpu", context_lens=torch.tensor(lens))   # same seed: same pool
        plan = plan_kv_shards(lens, world, 256, cfg.query_len)
        m, l, o = _rank_triples(inp, plan[rank], 256)
        merged = gather_and_merge(m, l, o, merge=pa_oracle.merge_triples)
        want = _full_output(inp).reshape(-1, cfg.head_size)
        ret[rank] = float((merged - want).abs().max())
        # sequence sharding on the same group: the ranks' token counts add up
        owned = shard_sequences(lens, world, "balanced")[rank]
        mine = torch.tensor([sum(lens[i] for i in owned)], dtype=torch.int64)
        dist.all_reduce(mine)
        ret[rank + world] = int(mine.item())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", sorted(_KV_CASES))
def test_two_gloo_ranks_exchange_and_merge_triples(case):
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_rank, args=(r, world, port, case, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert ret[0] < 8e-3 and ret[1] < 8e-3, dict(ret)
    assert ret[2] == ret[3] == sum(_KV_CASES[case][1])
