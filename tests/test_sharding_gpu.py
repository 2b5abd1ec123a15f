"""KV-partition sharding on one GPU: the ranks' launches run one after another on the same
device, their triples are stacked as an all-gather would and merged by the merge kernel."""
from __future__ import annotations

import pytest
import torch

from _util import assert_close, oracle_output, run_operator
from triton_op_b200.inputs import DecodeConfig, make_inputs, pack_mtp
from triton_op_b200.sharding import decode_kv_shard, local_block_table, merge_triples_cuda, plan_kv_shards

pytestmark = pytest.mark.gpu

_CASES = {
    "decode_p256": (DecodeConfig("kvs", 3, 8, 2, 16, 1, ("fixed", 1)), [2300, 700, 256], 256),
    "decode_p512": (DecodeConfig("kvs512", 4, 8, 1, 16, 1, ("fixed", 1), partition_size=512), [9000, 4096, 513, 100], 512),
    "mtp3_pertoken": (DecodeConfig("kvs_mtp", 4, 8, 2, 16, 3, ("fixed", 1), quant="per_token"), [1500, 513, 258, 40], 256),
    "mtp2_block1024": (DecodeConfig("kvs_1024", 3, 16, 2, 1024, 2, ("fixed", 1), quant="per_token"), [5000, 2049, 1024], 1024),
    "bf16_kv": (DecodeConfig("kvs_bf16", 3, 8, 2, 16, 1, ("fixed", 1), kv_dtype="bf16", quant="none"), [1300, 700, 256], 256),
}


@pytest.mark.parametrize("case", sorted(_CASES))
@pytest.mark.parametrize("world", [2, 4])
def test_kv_sharded_decode_matches_single_call_and_oracle(case, world):
    cfg, lens, cut = _CASES[case]
    inp = make_inputs(cfg, seed=11, device="cuda:0", context_lens=torch.tensor(lens))
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    plan = plan_kv_shards(lens, world, cut, cfg.query_len)       # ranges cut at multiples of `cut`
    triples = []
    for rank in range(world):
        tables = local_block_table(inp.block_tables, plan[rank], cfg.block_size)
        triples.append(decode_kv_shard(inp.query, inp.key_cache, inp.value_cache, plan[rank], tables,
                                       inp.softmax_scale, inp.key_scale, inp.value_scale,
                                       partition_size=cfg.partition_size, status=status))
    merged = merge_triples_cuda(torch.stack([t[0] for t in triples]), torch.stack([t[1] for t in triples]),
                                torch.stack([t[2] for t in triples]))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = pack_mtp(oracle_output(inp), cfg.num_seqs, cfg.query_len, cfg.kv_heads).reshape(-1, cfg.head_size)
    assert_close(merged, want, what=f"{case} over {world} ranks vs oracle")
    single, _ = run_operator(inp)
    single = pack_mtp(single, cfg.num_seqs, cfg.query_len, cfg.kv_heads).reshape(-1, cfg.head_size)
    assert (merged.float() - single.float()).abs().max().item() < 1.6e-2   # two bf16 roundings apart at most


def test_merge_kernel_ignores_empty_shards():
    R, D = 37, 128
    g = torch.Generator(device="cuda:0")
    g.manual_seed(3)
    m = torch.randn(3, R, device="cuda:0", generator=g)
    l = torch.rand(3, R, device="cuda:0", generator=g) + 0.5
    o = torch.randn(3, R, D, device="cuda:0", generator=g)
    m[1], l[1] = float("-inf"), 0.0              # a rank with nothing to do
    o[1] = float("nan")                            # whose output rows may hold anything
    m[2, :5], l[2, :5] = float("-inf"), 0.0
    out = merge_triples_cuda(m, l, o)
    from oracle import pa_oracle
    o_ref = o.clone()
    o_ref[1] = 0.0
    want = pa_oracle.merge_triples(m.cpu(), l.cpu(), o_ref.cpu())
    assert_close(out, want, what="merge kernel")
    # all shards empty -> zeros
    out0 = merge_triples_cuda(torch.full((2, R), float("-inf"), device="cuda:0"), torch.zeros(2, R, device="cuda:0"),
                              torch.zeros(2, R, D, device="cuda:0"))
    assert float(out0.float().abs().max()) == 0.0


def test_prepared_decoder_single_rank_equals_operator():
    from triton_op_b200.sharding import KvShardedDecoder
    cfg, lens, cut = _CASES["decode_p512"]
    inp = make_inputs(cfg, seed=11, device="cuda:0", context_lens=torch.tensor(lens))
    plan = plan_kv_shards(lens, 1, cut, cfg.query_len)
    dec = KvShardedDecoder(inp.query, inp.key_cache, inp.value_cache, plan[0], inp.block_tables, inp.softmax_scale,
                           inp.key_scale, inp.value_scale, partition_size=cfg.partition_size)
    assert dec.kv_bytes == inp.kv_bytes
    got = dec.step().clone()
    again = dec.step()
    torch.cuda.synchronize()
    assert torch.equal(got, again)
    single, _ = run_operator(inp)
    single = pack_mtp(single, cfg.num_seqs, cfg.query_len, cfg.kv_heads)
    assert (got.float() - single.float()).abs().max().item() < 8e-3     # fp32 triple, then one bf16 rounding


def test_packed_merge_equals_plain_merge():
    import ctypes as C
    from triton_op_b200 import _lib
    L = _lib.lib()
    W, R, D = 3, 21, 128                      # 2R = 42 floats: the o block starts after 2 floats of padding
    n = int(L.pa_packed_triple_floats(R, D))
    assert n == 44 + R * D
    g = torch.Generator(device="cuda:0")
    g.manual_seed(9)
    m = torch.randn(W, R, device="cuda:0", generator=g)
    l = torch.rand(W, R, device="cuda:0", generator=g) + 0.1
    o = torch.randn(W, R, D, device="cuda:0", generator=g)
    packed = torch.full((W, n), float("nan"), device="cuda:0")
    packed[:, :R], packed[:, R:2 * R], packed[:, 44:] = m, l, o.reshape(W, -1)
    out = torch.empty(R, D, dtype=torch.bfloat16, device="cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(L.pa_merge_packed_triples_sm100(out.data_ptr(), D, packed.data_ptr(), W, R, D, stream), "packed merge")
    want = merge_triples_cuda(m, l, o)
    torch.cuda.synchronize()
    assert torch.equal(out, want)
