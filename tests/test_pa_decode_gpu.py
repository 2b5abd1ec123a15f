"""GPU parity of the CUDA operator (through the C ABI) against the oracle and the fixtures."""
import ctypes as C

import pytest
import torch

from _util import (ATOL, GOLDEN_CASES, RTOL, assert_close, golden_inputs, load_golden, oracle_output,
                   run_operator)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _status():
    return torch.zeros((), dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("name", sorted(GOLDEN_CASES))
def test_operator_matches_reference_golden(name):
    """Same seeded inputs as the fixture (built on CPU, moved to the GPU); the expected output is
    what the reference's own PyTorch path produced."""
    gold = load_golden(name)
    inp = golden_inputs(name).to(DEV)
    st = _status()
    out, res = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    err = assert_close(out, gold["out"], what=name)
    # far inside the tolerance in practice: the arithmetic is exact up to fp32 accumulation,
    # bf16-precision probabilities and the bf16 rounding of the partial outputs
    assert err < 8e-3, f"{name}: max abs err {err}"


@pytest.mark.parametrize("name", ["cfg1_small", "gqa4_ragged", "mtp2_g8", "mtp4_g2_pertoken", "partition512"])
def test_partition_intermediates(name):
    """exp_sums / max_logits / tmp_output against the exact-fp32 split-KV statement."""
    from oracle import pa_oracle
    cpu = golden_inputs(name)
    c = cpu.cfg
    ks, vs = cpu.flat_scales()
    inp = cpu.to(DEV)
    _, res = run_operator(inp)
    torch.cuda.synchronize()
    psize = res["partition_size"]        # 512 runs as 256-token sub-partitions on the operator's own workspaces
    assert psize == 256
    m_ref, l_ref, o_ref = pa_oracle.split_kv_partials(cpu.query, cpu.key_cache, cpu.value_cache, cpu.block_tables,
                                                      cpu.context_lens, c.query_len, cpu.softmax_scale,
                                                      psize, ks, vs)
    m, l, o = res["maximum_logits"].cpu(), res["exponential_sums"].cpu(), res["temporary_output"].float().cpu()
    for s in range(c.num_seqs):
        np_s = (int(cpu.context_lens[s]) + psize - 1) // psize
        ms, ls, os_ = m[s, :, :np_s], l[s, :, :np_s], o[s, :, :np_s]
        mr, lr, orr = m_ref[s, :, :np_s], l_ref[s, :, :np_s], o_ref[s, :, :np_s]
        live = lr > 0
        assert torch.equal(torch.isinf(ms), ~live)
        assert torch.allclose(ms[live], mr[live], atol=1e-4, rtol=1e-5)
        assert torch.allclose(ls, lr, atol=1e-4, rtol=2e-4)
        assert torch.allclose(os_, orr, atol=6e-3, rtol=8e-3)


def _check_partials(cpu, res_ws, psize, what):
    """exp_sums / max_logits / tmp_output of a run against the exact-fp32 split-KV statement."""
    from oracle import pa_oracle
    c = cpu.cfg
    ks, vs = cpu.flat_scales()
    m_ref, l_ref, o_ref = pa_oracle.split_kv_partials(cpu.query, cpu.key_cache, cpu.value_cache, cpu.block_tables,
                                                      cpu.context_lens, c.query_len, cpu.softmax_scale, psize, ks, vs)
    es, ml, tmp = (t.cpu() for t in res_ws)
    for s in range(c.num_seqs):
        np_s = (int(cpu.context_lens[s]) + psize - 1) // psize
        live = l_ref[s, :, :np_s] > 0
        assert torch.equal(torch.isinf(ml[s, :, :np_s]), ~live), what
        assert torch.allclose(ml[s, :, :np_s][live], m_ref[s, :, :np_s][live], atol=1e-4, rtol=1e-5), what
        assert torch.allclose(es[s, :, :np_s], l_ref[s, :, :np_s], atol=1e-4, rtol=2e-4), what
        assert torch.allclose(tmp[s, :, :np_s].float(), o_ref[s, :, :np_s], atol=6e-3, rtol=8e-3), what


def _caller_workspaces(inp, psize, fill=float("nan")):
    c = inp.cfg
    P = (inp.max_context + psize - 1) // psize
    shape = (c.num_seqs, c.kv_heads, P, c.q_heads // c.kv_heads * c.query_len)
    es = torch.full(shape, fill, dtype=torch.float32, device=DEV)
    ml = torch.full(shape, fill, dtype=torch.float32, device=DEV)
    tmp = torch.full(shape + (c.head_size,), fill, dtype=torch.bfloat16, device=DEV)
    return es, ml, tmp


@pytest.mark.parametrize("kernel", ["tcgen05", "mma.sync"])
def test_partition512_on_caller_workspaces_keeps_their_layout(kernel):
    """Workspaces passed by the caller are filled at the partition size asked for: by the tcgen05
    kernel (two 256-token work items per partition, merged in the second one's epilogue), or by the
    mma.sync kernel when tune warps asks for it."""
    from triton_op_b200.pa_decode import query_launch
    cpu = golden_inputs("partition512")
    c = cpu.cfg
    inp = cpu.to(DEV)
    tune = None if kernel == "tcgen05" else {"warps": 8}
    es, ml, tmp = _caller_workspaces(inp, 512)
    launch = query_launch(torch.empty_like(inp.query), inp.query, inp.key_cache, inp.value_cache, inp.context_lens,
                          inp.block_tables, inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None,
                          inp.key_scale, inp.value_scale, partition_size=512, exp_sums=es, max_logits=ml,
                          tmp_output=tmp, tune=tune)
    assert launch["cta_threads"] == (512 if kernel == "tcgen05" else 256)
    st = _status()
    got, res = run_operator(inp, exp_sums=es, max_logits=ml, tmp_output=tmp, status=st, tune=tune)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert res["partition_size"] == 512
    assert_close(got, oracle_output(cpu), what="partition 512, caller workspaces")
    _check_partials(cpu, (es, ml, tmp), 512, f"partition 512 on the {kernel} kernel")


@pytest.mark.parametrize("shape", [
    # (seqs, q heads, kv heads, block, L, context spec, quant)
    (11, 32, 8, 16, 1, ("cycle", [1, 255, 256, 257, 511, 512, 513, 767, 768, 769, 1300]), "per_tensor"),
    (9, 16, 2, 16, 1, ("uniform", 1, 6000), "per_token"),
    (6, 8, 1, 64, 2, ("uniform", 200, 5000), "per_tensor"),
    (4, 8, 2, 1024, 4, ("uniform", 900, 7000), "per_token"),
    (3, 16, 1, 16, 1, ("uniform", 3000, 9000), "per_tensor"),       # 16 rows per item
    (200, 8, 2, 16, 1, ("uniform", 1, 1100), "per_tensor"),         # many sequences, most partitions single or short
    (2, 8, 1, 16, 1, ("fixed", 40000), "per_tensor"),               # long: a CTA holds many pairs
])
def test_partition512_pairs_on_the_tensor_cores(shape):
    """The PAIR form against the exact split-KV statement at partition 512: contexts that end in
    the first or the second half of a partition or exactly on a boundary, all page sizes, MTP,
    per-token scales, 4 / 8 / 16 rows per item; workspaces start as NaN and a second call gives the
    same bits; the mma.sync kernel's result (16-token pages only) agrees within the tolerance."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    S, hq, hkv, bs, L, ctx, quant = shape
    cfg = DecodeConfig("pair", S, hq, hkv, bs, L, ctx, quant=quant, partition_size=512)
    cpu = make_inputs(cfg, seed=S * 7 + bs, device="cpu")
    if S >= 9:
        cpu.context_lens[S // 2] = 0
    inp = cpu.to(DEV)
    es, ml, tmp = _caller_workspaces(inp, 512)
    st = _status()
    got, res = run_operator(inp, exp_sums=es, max_logits=ml, tmp_output=tmp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and res["partition_size"] == 512
    assert_close(got, oracle_output(cpu), what=f"pairs {shape}")
    if S * inp.max_context <= 120000:
        _check_partials(cpu, (es, ml, tmp), 512, f"pairs {shape}")
    first = (got.clone(), es.clone(), ml.clone(), tmp.clone())
    got2, _ = run_operator(inp, exp_sums=es, max_logits=ml, tmp_output=tmp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(got2.view(torch.int16), first[0].view(torch.int16))
    live = ~torch.isnan(first[1])      # entries past a sequence's last partition are never written
    assert torch.equal(es[live], first[1][live]) and torch.equal(ml[live], first[2][live])
    if bs == 16:
        es2, ml2, tmp2 = _caller_workspaces(inp, 512)
        ref, _ = run_operator(inp, exp_sums=es2, max_logits=ml2, tmp_output=tmp2, tune={"warps": 8})
        assert_close(got, ref, what=f"pairs {shape}: tcgen05 against mma.sync")


def test_workspaces_need_no_clearing_and_runs_are_bit_identical():
    inp = golden_inputs("gqa4_ragged").to(DEV)
    c = inp.cfg
    P = (inp.max_context + c.partition_size - 1) // c.partition_size
    eqg = c.q_heads // c.kv_heads * c.query_len
    shape = (c.num_seqs, c.kv_heads, P, eqg)
    outs = []
    for fill in (float("nan"), 1e30):
        es = torch.full(shape, fill, dtype=torch.float32, device=DEV)
        ml = torch.full(shape, fill, dtype=torch.float32, device=DEV)
        tmp = torch.full(shape + (c.head_size,), fill, dtype=torch.bfloat16, device=DEV)
        out, _ = run_operator(inp, exp_sums=es, max_logits=ml, tmp_output=tmp)
        outs.append(out.clone())
    torch.cuda.synchronize()
    assert not torch.isnan(outs[0]).any()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert_close(outs[0], load_golden("gqa4_ragged")["out"], what="poisoned workspaces")


def test_garbage_beyond_context_is_ignored():
    """Bytes of the last page past the context length (NaN patterns included) and block-table
    entries past the last valid page must not influence the result."""
    cpu = golden_inputs("cfg1_small")
    inp = cpu.to(DEV)
    base, _ = run_operator(inp)
    bs = cpu.cfg.block_size
    k = inp.key_cache.clone().view(torch.uint8)
    v = inp.value_cache.clone().view(torch.uint8)
    bt = inp.block_tables.clone()
    for s in range(cpu.cfg.num_seqs):
        ctx = int(cpu.context_lens[s])
        nblk = (ctx + bs - 1) // bs
        last = int(cpu.block_tables[s, nblk - 1])
        used = ctx - (nblk - 1) * bs
        if used < bs:
            k[last, :, :, used:, :] = 0x7F   # e4m3fn NaN
            v[last, :, :, used:] = 0xFF
        bt[s, nblk:] = 2 ** 30               # would fault if it were ever dereferenced
    inp.key_cache = k.view(torch.float8_e4m3fn)
    inp.value_cache = v.view(torch.float8_e4m3fn)
    inp.block_tables = bt
    st = _status()
    out, _ = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(out.view(torch.int16), base.view(torch.int16))


@pytest.mark.parametrize("name", ["gqa4_ragged", "mtp4_g2_pertoken", "bf16_kv"])
@pytest.mark.parametrize("case", ["peaked", "one-hot", "flat", "underflow", "zero query", "zero keys"])
def test_extreme_logit_distributions(name, case):
    """Queries scaled by powers of two from 2^-120 to 2^8 (attention from uniform to one-hot; the
    query rows' power-of-two pre-scale at both ends of its range), all-zero queries and all-zero
    keys, against the oracle on the same inputs."""
    import copy
    cpu = copy.copy(golden_inputs(name))
    factor = {"peaked": 2.0 ** 4, "one-hot": 2.0 ** 8, "flat": 2.0 ** -40, "underflow": 2.0 ** -120,
              "zero query": 0.0, "zero keys": 1.0}[case]
    cpu.query = (cpu.query.float() * factor).to(torch.bfloat16)
    cpu.query_tokens = (cpu.query_tokens.float() * factor).to(torch.bfloat16)
    if case == "zero keys":
        cpu.key_cache = torch.zeros_like(cpu.key_cache.view(torch.uint8 if cpu.key_cache.element_size() == 1 else torch.int16)).view(cpu.key_cache.dtype)
    ref = oracle_output(cpu)
    st = _status()
    out, _ = run_operator(cpu.to(DEV), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(out, ref, what=f"{name}, {case}")


def test_bad_page_id_and_long_context_are_clamped_and_reported():
    from triton_op_b200 import _lib
    inp = golden_inputs("cfg1_small").to(DEV)
    inp.block_tables = inp.block_tables.clone()
    inp.block_tables[0, 0] = 10 ** 6
    st = _status()
    run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) & _lib.PA_DEV_BAD_PAGE_ID
    inp2 = golden_inputs("cfg1_small").to(DEV)
    inp2.context_lens = inp2.context_lens.clone()
    inp2.context_lens[1] = inp2.block_tables.shape[1] * 16 + 5
    st2 = _status()
    run_operator(inp2, status=st2)
    torch.cuda.synchronize()
    assert int(st2.item()) & _lib.PA_DEV_CTX_TOO_LONG


def test_tuning_knobs_do_not_change_results():
    inp = golden_inputs("gqa4_ragged").to(DEV)
    base, _ = run_operator(inp)
    # ring depth and grid size only change scheduling: bit-identical results
    for tune in ({"ctas": 3}, {"stages": 3, "ctas": 1}, {"ctas": 148}):
        out, _ = run_operator(inp, tune=tune)
        assert torch.equal(out.view(torch.int16), base.view(torch.int16)), tune
    # warps = 4 / 8 selects the mma.sync kernel: same math, different rounding order
    ref = load_golden("gqa4_ragged")["out"]
    for tune in ({"warps": 4}, {"warps": 8, "stages": 2}, {"warps": 4, "ctas": 2}):
        out, _ = run_operator(inp, tune=tune)
        assert_close(out, ref, what=str(tune))


def test_ring_depths_never_drop_below_the_issue_lag():
    """The host plan keeps the K ring of the tcgen05 kernel at least as deep as the three softmax
    groups and the V ring at least two deep; a request for less, or a batch whose in-kernel index
    leaves no room for that, is refused instead of launching a shallower ring (nothing is launched
    here: the plan is queried)."""
    from triton_op_b200 import _lib
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    from triton_op_b200.pa_decode import query_launch
    inp = golden_inputs("gqa4_ragged").to(DEV)
    c = inp.cfg
    args = lambda i: (torch.empty_like(i.query), i.query, i.key_cache, i.value_cache, i.context_lens, i.block_tables,
                      i.softmax_scale, i.cfg.query_len, i.max_context, torch.bfloat16, None, i.key_scale, i.value_scale)
    assert query_launch(*args(inp))["ring_stages"] >= 3
    assert query_launch(*args(inp), tune={"stages": 3})["ring_stages"] == 3
    for tune in ({"stages": 2}, {"stages": 1}, {"vstages": 1}):
        with pytest.raises(_lib.PaError) as err:
            query_launch(*args(inp), tune=tune)
        assert err.value.status == -3, tune
    # thousands of sequences: the index eats into the rings, which shrink to (3, 2) and no further
    big = make_inputs(DecodeConfig("many", 4000, 4, 1, 16, 1, ("fixed", 16)), seed=5, device=DEV)
    assert query_launch(*args(big))["ring_stages"] >= 3
    huge = make_inputs(DecodeConfig("too_many", 12000, 4, 1, 16, 1, ("fixed", 16)), seed=5, device=DEV)
    with pytest.raises(_lib.PaError) as err:
        query_launch(*args(huge))
    assert err.value.status == -7


@pytest.mark.parametrize("name", ["cfg1_small", "gqa4_ragged", "mtp2_g8", "mtp4_g2_pertoken", "pertoken_g8", "bs64_g5"])
def test_single_launch_decode_matches_the_two_launch_form(name):
    """tune fuse = 1: the decode call is one launch (the softmax group that stores the last partition
    of a (sequence, kv head) in its CTA merges the set; sets cut by the end of a team's range are
    handed over through the counters).  Same arithmetic in the same order as the reduce kernel:
    bit-identical outputs, counters back at zero, twice in a row."""
    from triton_op_b200.pa_decode import get_merge_counters, query_launch
    inp = golden_inputs(name).to(DEV)
    c = inp.cfg
    two, res2 = run_operator(inp)
    launch = query_launch(torch.empty_like(inp.query), inp.query, inp.key_cache, inp.value_cache, inp.context_lens,
                          inp.block_tables, inp.softmax_scale, c.query_len, inp.max_context, torch.bfloat16, None,
                          inp.key_scale, inp.value_scale, tune={"fuse": 1})
    assert launch["cta_threads"] == 16 * 32
    for _ in range(2):
        st = _status()
        one, res1 = run_operator(inp, status=st, tune={"fuse": 1})
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        assert torch.equal(one.view(torch.int16), two.view(torch.int16))
        counters = get_merge_counters(res1["temporary_output"], c.num_seqs, c.kv_heads)
        assert int(counters.abs().sum().item()) == 0
    assert_close(one, load_golden(name)["out"], what=f"{name}: single launch")


@pytest.mark.parametrize("team", [0, 1, 2, 4])
def test_single_launch_decode_on_the_benchmark_shape(team):
    """Teams of 1, 2 or 4 CTAs per (sequence, partition) row (0: the library's choice): a set is
    merged inside one CTA or handed over once, whichever way the rows are cut."""
    from triton_op_b200.inputs import CONFIGS, make_inputs
    inp = make_inputs(CONFIGS["cfg2_llama8b"], seed=3, device=DEV, num_seqs=24)
    two, _ = run_operator(inp)
    st = _status()
    for _ in range(3):
        one, _ = run_operator(inp, status=st, tune={"fuse": 1 + team})
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))


@pytest.mark.parametrize("shape", [(2, 8000, 8, 4), (3, 8192, 2, 8), (40, 700, 8, 4), (7, 5000, 1, 8), (300, 3000, 4, 4)])
def test_single_launch_decode_with_sets_cut_in_many_places(shape):
    """Few long sequences: a (sequence, kv head) set of up to 32 partitions is spread over many
    teams (a team may hold one or two rows), so most sets are merged by an owner that waits for
    the counts of several other CTAs; many short ones: most sets lie inside one CTA; empty
    sequences in between.  Bit-identical to the two-launch form either way."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    from triton_op_b200.pa_decode import get_merge_counters
    S, ctx, hkv, g = shape
    cfg = DecodeConfig("cut", S, hkv * g, hkv, 16, 1, ("uniform", ctx // 3, ctx))
    inp = make_inputs(cfg, seed=S + ctx, device=DEV)
    if S >= 7:
        inp.context_lens[S // 2] = 0
        inp.context_lens[S - 1] = 0
    two, _ = run_operator(inp)
    st = _status()
    for _ in range(3):
        one, res = run_operator(inp, status=st, tune={"fuse": 1})
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))
    assert int(get_merge_counters(res["temporary_output"], S, hkv).abs().sum().item()) == 0


@pytest.mark.parametrize("bs,ql,quant", [(64, 1, "per_token"), (1024, 2, "per_token"), (1024, 1, "per_tensor"), (64, 2, "per_tensor")])
def test_single_launch_decode_with_long_pages(bs, ql, quant):
    """The single-launch form on pages of 64 and 1024 tokens, with the per-token scales staged in the
    query slots: bit-identical to the two-launch form, counters back at zero."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    from triton_op_b200.pa_decode import get_merge_counters
    cfg = DecodeConfig("fuse_pages", 30, 8, 4, bs, ql, ("uniform", 1, 3000), quant=quant)
    inp = make_inputs(cfg, seed=bs + ql, device=DEV)
    two, _ = run_operator(inp)
    st = _status()
    for _ in range(2):
        one, res = run_operator(inp, status=st, tune={"fuse": 1})
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(one.view(torch.int16), two.view(torch.int16))
    assert int(get_merge_counters(res["temporary_output"], 30, 4).abs().sum().item()) == 0


@pytest.mark.parametrize("form", ["two launches", "single launch", "partition 512"])
def test_lengths_and_tables_written_by_the_kernel_just_before_the_call(form):
    """The tcgen05 kernel builds its partition index before its dependency wait and checks it after
    (in all its forms: the team ranges of the single-launch form and the item counts of the
    512-token form are derived from the index that passed the check).
    Here the kernel right before every call in the stream rewrites the context lengths and the block
    tables (what a serving loop's bookkeeping kernel does), alternating between two batches, with a
    long decode call before it so that the next call's CTAs are resident early: every result must be
    the one for the lengths and tables as written."""
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, unpack_mtp
    cfg = DecodeConfig("early", 48, 32, 8, 16, 1, ("uniform", 1, 3000))
    a = make_inputs(cfg, seed=51, device=DEV)
    b = make_inputs(cfg, seed=52, device=DEV)           # other lengths, other tables, same pool size or smaller
    nb = min(a.key_cache.shape[0], b.key_cache.shape[0])
    width = max(a.block_tables.shape[1], b.block_tables.shape[1])
    pad = lambda t: torch.nn.functional.pad(t, (0, width - t.shape[1]))
    tables = [pad(a.block_tables) % nb, pad(b.block_tables) % nb]
    lens = [a.context_lens, b.context_lens]
    kc, vc = a.key_cache[:nb], a.value_cache[:nb]
    cur_tables, cur_lens = tables[0].clone(), lens[0].clone()
    max_ctx = int(max(int(lens[0].max()), int(lens[1].max())))
    want = []
    for v in range(2):
        out = torch.empty_like(a.query)
        paged_attention_decode(out, a.query, kc, vc, lens[v].clone(), tables[v].clone(), a.softmax_scale, 1, max_ctx,
                               torch.bfloat16, None, a.key_scale, a.value_scale, tune={"early": -1})
        want.append(out.clone())
    torch.cuda.synchronize()
    st = _status()
    outs = []
    kw = {}
    if form == "single launch":
        kw = {"tune": {"fuse": 1}}
    if form == "partition 512":
        P = (max_ctx + 511) // 512
        kw = {"partition_size": 512,
              "exp_sums": torch.zeros((48, 8, P, 4), dtype=torch.float32, device=DEV),
              "max_logits": torch.zeros((48, 8, P, 4), dtype=torch.float32, device=DEV),
              "tmp_output": torch.zeros((48, 8, P, 4, 128), dtype=torch.bfloat16, device=DEV)}
    for it in range(40):
        v = (it * 7 + it // 3) % 2
        out = torch.empty_like(a.query)
        cur_lens.copy_(lens[v])            # kernels in the same stream, directly before the call
        cur_tables.copy_(tables[v])
        paged_attention_decode(out, a.query, kc, vc, cur_lens, cur_tables, a.softmax_scale, 1, max_ctx, torch.bfloat16, None,
                               a.key_scale, a.value_scale, status=st, **kw)
        outs.append((v, out))
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    for v, out in outs:
        if form == "partition 512":     # another split: the same attention within the tolerance
            assert_close(out, want[v], what="partition 512 after rewritten lengths")
        else:
            assert torch.equal(out.view(torch.int16), want[v].view(torch.int16))


def test_zero_length_sequences_and_empty_batch():
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    cfg = DecodeConfig("zeros", 5, 8, 2, 16, 1, ("fixed", 100))
    ctx = torch.tensor([0, 100, 1, 0, 257], dtype=torch.int32)
    cpu = make_inputs(cfg, seed=3, context_lens=ctx)
    ref = oracle_output(_nonempty(cpu))
    out, _ = run_operator(cpu.to(DEV))
    torch.cuda.synchronize()
    keep = [1, 2, 4]
    assert_close(out[keep], ref, what="non-empty sequences")
    assert torch.count_nonzero(out[[0, 3]].float()) == 0   # empty context -> zeros


def _nonempty(inp):
    """The same workload without its zero-length sequences (the PyTorch path cannot take them)."""
    import copy
    keep = [i for i in range(inp.cfg.num_seqs) if int(inp.context_lens[i]) > 0]
    out = copy.copy(inp)
    out.cfg = type(inp.cfg)(**{**inp.cfg.__dict__, "num_seqs": len(keep)})
    out.query_tokens = inp.query_tokens[keep]
    out.query = inp.query[keep]
    out.block_tables = inp.block_tables[keep]
    out.context_lens = inp.context_lens[keep]
    return out


def test_llama8b_shape_full_size_against_oracle_on_device():
    """The benchmark configuration at full size; the oracle runs on the GPU in fp32."""
    from triton_op_b200.inputs import CONFIGS, make_inputs
    inp = make_inputs(CONFIGS["cfg2_llama8b"], seed=0, device=DEV)
    st = _status()
    out, res = run_operator(inp, status=st)
    ref = oracle_output(inp)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(out, ref, what="cfg2_llama8b")
    # size-independent property: probabilities sum to one, so with V == const the output is const
    inp.value_cache = torch.full_like(inp.value_cache.float(), 1.5).to(torch.float8_e4m3fn)
    out1, _ = run_operator(inp)
    expect = 1.5 * float(inp.value_scale)
    assert torch.allclose(out1.float(), torch.full_like(out1.float(), expect), rtol=1e-2, atol=0)


# ----------------------------------------------------------------------------- reference test matrix
# test_pa_mtp.py:48-54 of the reference: block sizes {16, 64, 1024}, (Hq, Hkv) in {(5,1), (8,1),
# (10,1), (16,1), (64,4)}, query length 1-4, context {512, 4096, 4097}, batch {4, 80, 128}, and the
# whole sweep again with the shuffled value layout (--trans_v).  Here every shape runs at batch 3
# in both value layouts, uniform data as in that harness, per-token scales (what the harness feeds
# the Gluon kernel), with the oracle run on the GPU; batches 80 and 128 follow below.
_MATRIX = [(bs, hq, hkv, ql, ctx)
           for bs in (16, 64, 1024)
           for (hq, hkv) in ((5, 1), (8, 1), (10, 1), (16, 1), (64, 4))
           for ql in (1, 2, 3, 4)
           for ctx in (512, 4096, 4097)]


@pytest.mark.parametrize("bs,hq,hkv,ql,ctx", _MATRIX)
def test_reference_matrix(bs, hq, hkv, ql, ctx):
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, shuffle_value_cache_layout, unpack_mtp
    cfg = DecodeConfig(f"m{bs}_{hq}_{hkv}_{ql}_{ctx}", 3, hq, hkv, bs, ql, ("fixed", ctx), quant="per_token")
    inp = make_inputs(cfg, seed=bs + hq + ql, device=DEV, dist="uniform")
    st = _status()
    out, _ = run_operator(inp, status=st)
    ref = oracle_output(inp)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(out, ref, what=cfg.name)
    # the same call on the shuffled value layout [NB, Hkv, bs/16, D, 16]: same products in the same order
    out_t = torch.full_like(inp.query, float("nan"))
    paged_attention_decode(out_t, inp.query, inp.key_cache, shuffle_value_cache_layout(inp.value_cache), inp.context_lens,
                           inp.block_tables, inp.softmax_scale, ql, inp.max_context, torch.bfloat16, None, inp.key_scale,
                           inp.value_scale, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert torch.equal(unpack_mtp(out_t, 3, ql, hkv), out), f"{cfg.name}: transposed value layout differs"


@pytest.mark.parametrize("batch,bs,hq,hkv,ql,ctx", [(80, 16, 8, 1, 2, 4097), (128, 1024, 64, 4, 1, 4096),
                                                    (128, 64, 10, 1, 3, 512), (80, 1024, 16, 1, 4, 4097)])
def test_reference_matrix_large_batches(batch, bs, hq, hkv, ql, ctx):
    """Batches 80 and 128 of the reference's sweep (test_pa_mtp.py:52): the oracle checks a sample of
    the sequences, and every sequence must equal its own result in a batch of one sample."""
    import copy
    from triton_op_b200.inputs import DecodeConfig, make_inputs, subset_inputs
    cfg = DecodeConfig(f"b{batch}_{bs}_{hq}_{ql}", batch, hq, hkv, bs, ql, ("fixed", ctx), quant="per_token")
    inp = make_inputs(cfg, seed=batch + bs, device=DEV, dist="uniform")
    st = _status()
    out, _ = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and bool(torch.isfinite(out.float()).all())
    pick = sorted(torch.randperm(batch, generator=torch.Generator().manual_seed(batch))[:5].tolist())
    sub = subset_inputs(inp, pick)
    rows = [s * ql + t for s in pick for t in range(ql)]
    assert_close(out[rows], oracle_output(sub), what=f"{cfg.name}: sampled sequences vs oracle")
    out_sub, _ = run_operator(sub, status=st)
    assert torch.equal(out_sub, out[rows])


@pytest.mark.parametrize("batch,hq,hkv,ql,bs", [(1500, 16, 1, 1, 64), (1200, 8, 1, 2, 1024), (4500, 4, 1, 1, 64)])
def test_batches_too_large_for_staged_token_scales(batch, hq, hkv, ql, bs):
    """With per-token scales and pages of 64 tokens or more the kernel keeps an item's scales in its
    query slot -- while the in-kernel index of the batch (8 bytes per sequence) leaves room for the
    2 KB per slot.  These batches do not: the form whose softmax threads fetch the scales runs, and
    a sample agrees with the oracle and, bit for bit, with its own batch of five (which is staged)."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs, subset_inputs
    from triton_op_b200.pa_decode import query_launch
    cfg = DecodeConfig(f"big{batch}", batch, hq, hkv, bs, ql, ("uniform", 1, 300), quant="per_token")
    inp = make_inputs(cfg, seed=batch, device=DEV)
    st = _status()
    out, _ = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and bool(torch.isfinite(out.float()).all())
    pick = sorted(torch.randperm(batch, generator=torch.Generator().manual_seed(batch))[:5].tolist())
    sub = subset_inputs(inp, pick)
    rows = [s * ql + t for s in pick for t in range(ql)]
    assert_close(out[rows], oracle_output(sub), what=f"{cfg.name}: sampled sequences vs oracle")
    out_sub, _ = run_operator(sub, status=st)        # the small batch runs the staged form
    assert torch.equal(out_sub, out[rows])
    big = query_launch(torch.empty_like(inp.query), inp.query, inp.key_cache, inp.value_cache, inp.context_lens,
                       inp.block_tables, inp.softmax_scale, ql, inp.max_context, torch.bfloat16, None,
                       inp.key_scale, inp.value_scale)
    assert big["ring_stages"] >= 3 and big["smem_bytes"] <= 227 * 1024


@pytest.mark.parametrize("name,num_seqs", [("cfg3_llama70b_mtp", 12), ("cfg4_longctx", 3), ("cfg5_serving_fp8", 48),
                                           ("cfg5_serving_bf16", 48)])
def test_baseline_configs_reduced_batch(name, num_seqs):
    """The other benchmark configurations at their real shapes and length distributions, fewer sequences."""
    from triton_op_b200.inputs import CONFIGS, make_inputs
    inp = make_inputs(CONFIGS[name], seed=1, device=DEV, num_seqs=num_seqs)
    st = _status()
    out, _ = run_operator(inp, status=st)
    ref = oracle_output(inp)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(out, ref, what=name)


@pytest.mark.parametrize("lens,psize,ql", [([12000, 100, 4096], 256, 1),       # 47 partitions: 4 warps per row
                                            ([40000, 9000, 300], 256, 2),      # 157 partitions: 16 warps per row
                                            ([70000, 513], 512, 1)])           # 137 partitions of 512 tokens
def test_long_contexts_use_the_multi_warp_reduce(lens, psize, ql):
    """Rows with more than 32 partitions are merged by several warps; the result must not depend on
    how the partitions were dealt out, so it is compared with the oracle and with the triples path."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs
    cfg = DecodeConfig("long", len(lens), 4 * ql, 1, 16, ql, ("fixed", 1), partition_size=psize)
    inp = make_inputs(cfg, seed=21, device=DEV, context_lens=torch.tensor(lens))
    out, res = run_operator(inp)
    torch.cuda.synchronize()
    assert res["exponential_sums"].shape[2] > 32
    assert_close(out, oracle_output(inp), what=f"{lens} partition {psize}")


def test_mixed_lengths_up_to_128_partitions():
    """A serving-mix batch: rows of one chunk of partitions next to rows of two to four (the reduce
    kernel that deals the further chunks of a CTA's long rows over its sixteen warps).  Against the
    oracle, and every sequence bit-equal to itself in a smaller batch with other neighbours."""
    from triton_op_b200.inputs import DecodeConfig, make_inputs, subset_inputs
    lens = [20000, 300, 9000, 33, 32768, 8193, 5000, 16, 8192, 24577, 1, 12000, 700, 16385, 64, 31000, 2000, 10000]
    cfg = DecodeConfig("mix", len(lens), 32, 8, 16, 1, ("fixed", 1))
    inp = make_inputs(cfg, seed=61, device=DEV, context_lens=torch.tensor(lens))
    st = _status()
    out, res = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert 32 < res["exponential_sums"].shape[2] <= 128
    assert_close(out, oracle_output(inp), what="mixed lengths")
    for pick in ([0, 4, 5], [1, 2, 3, 9, 15, 17], [4]):
        sub = subset_inputs(inp, pick)
        if sub.max_context <= 8192:
            continue
        out_sub, _ = run_operator(sub, status=st)
        assert torch.equal(out_sub, out[pick]), pick
    assert int(st.item()) == 0


@pytest.mark.parametrize("heads,ql,bs,kvq", [((32, 8), 1, 16, "per_tensor"), ((16, 2), 1, 16, "per_token"),
                                             ((16, 2), 2, 1024, "per_token"), ((10, 1), 3, 64, "per_tensor")])
@pytest.mark.parametrize("qmode", ["per_tensor", "per_token"])
def test_fp8_query_with_query_scale(heads, ql, bs, kvq, qmode):
    """e4m3fn query rows with a per-tensor or per-row query scale (the reference's fp8 entry,
    pa_decode_triton_gluon_fp8.py:1752-1768): compared with the oracle on the dequantised rows."""
    from oracle import pa_oracle
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import FP8, FP8_MAX, DecodeConfig, make_inputs, pack_mtp, unpack_mtp
    hq, hkv = heads
    cfg = DecodeConfig("fp8q", 3, hq, hkv, bs, ql, ("fixed", 1), quant=kvq)
    inp = make_inputs(cfg, seed=17, device=DEV, context_lens=torch.tensor([700, 2049, 33]))
    q = inp.query_tokens.float()                                    # [S*L, Hq, D]
    if qmode == "per_tensor":
        scale = (q.abs().amax() / FP8_MAX).clamp_min(1e-12)
        scale_tok = scale
    else:
        scale_tok = (q.abs().amax(dim=-1, keepdim=True) / FP8_MAX).clamp_min(1e-12)   # [S*L, Hq, 1]
        scale = pack_mtp(scale_tok.expand(-1, -1, 1).contiguous(), cfg.num_seqs, ql, hkv).contiguous()  # operator row order
    q8_tok = (q / scale_tok).to(FP8)
    q_deq = q8_tok.float() * scale_tok
    q8 = pack_mtp(q8_tok.view(torch.uint8), cfg.num_seqs, ql, hkv).contiguous().view(FP8)
    out = torch.full(q8.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    paged_attention_decode(out, q8, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                           inp.softmax_scale, ql, inp.max_context, torch.bfloat16, scale, inp.key_scale,
                           inp.value_scale, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ks, vs = inp.flat_scales()
    ref = pa_oracle.paged_attention(q_deq, inp.key_cache, inp.value_cache, inp.block_tables, inp.context_lens,
                                    inp.query_indptr(), ks, vs)
    assert_close(unpack_mtp(out, cfg.num_seqs, ql, hkv), ref, what=f"fp8 query {qmode}")


@pytest.mark.parametrize("bs", [16, 64, 1024])
@pytest.mark.parametrize("heads,ql,quant", [((8, 1), 1, "per_tensor"), ((16, 2), 2, "per_token")])
def test_transposed_value_layout(bs, heads, ql, quant):
    """Value cache in the reference's shuffled layout [NB, Hkv, bs/16, D, 16] (test_pa_mtp.py:472-497):
    same results as the normal layout, ragged last pages included."""
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, shuffle_value_cache_layout, unpack_mtp
    hq, hkv = heads
    cfg = DecodeConfig("transv", 4, hq, hkv, bs, ql, ("fixed", 1), quant=quant)
    inp = make_inputs(cfg, seed=23, device=DEV, context_lens=torch.tensor([1300, 257, 4097, 15]))
    v_t = shuffle_value_cache_layout(inp.value_cache)
    assert v_t.dim() == 5 and v_t.shape[2] == bs // 16 and v_t.shape[4] == 16
    # garbage (NaN patterns) behind the end of every context must not leak through the other layout either
    out = torch.full_like(inp.query, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    paged_attention_decode(out, inp.query, inp.key_cache, v_t, inp.context_lens, inp.block_tables,
                           inp.softmax_scale, ql, inp.max_context, torch.bfloat16, None, inp.key_scale,
                           inp.value_scale, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_close(unpack_mtp(out, cfg.num_seqs, ql, hkv), oracle_output(inp), what=f"trans_v bs={bs}")
    normal, _ = run_operator(inp)
    assert torch.equal(unpack_mtp(out, cfg.num_seqs, ql, hkv), normal)     # same products, same order


@pytest.mark.parametrize("heads,ql,bs,quant,kv,tune", [
    ((32, 8), 1, 16, "per_tensor", "fp8", None), ((8, 1), 1, 64, "per_token", "fp8", None),
    ((16, 2), 2, 1024, "per_token", "fp8", None), ((16, 1), 1, 16, "per_tensor", "fp8", None),
    ((10, 1), 4, 16, "per_tensor", "fp8", None),
    # the mma.sync fp8 kernel (asked for explicitly) and the bf16-KV kernel
    ((32, 8), 1, 16, "per_tensor", "fp8", {"warps": 8}), ((16, 2), 2, 16, "per_token", "fp8", {"warps": 4}),
    ((32, 8), 1, 16, "none", "bf16", None), ((16, 2), 2, 16, "none", "bf16", None)])
def test_alibi_slopes(heads, ql, bs, quant, kv, tune):
    """ALiBi bias slope[head] * (key position - (context - 1)) (pa_decode_triton_gluon_fp8.py:905-908,
    pa_decode_triton.py:148-151) on all three partition kernels, against the oracle, whose statement of
    the bias is pinned to a run of the reference's Triton path (tests/golden/triton_*_alibi.npz)."""
    from oracle import pa_oracle
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, unpack_mtp
    hq, hkv = heads
    cfg = DecodeConfig("alibi", 3, hq, hkv, bs, ql, ("fixed", 1), quant=quant, kv_dtype=kv)
    inp = make_inputs(cfg, seed=29, device=DEV, context_lens=torch.tensor([900, 2050, 17]))
    slopes = (2.0 ** (-8.0 * torch.arange(1, hq + 1, dtype=torch.float32) / hq)).to(DEV)   # the usual geometric slopes
    out = torch.full_like(inp.query, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = paged_attention_decode(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                                 inp.softmax_scale, ql, inp.max_context, torch.bfloat16, None, inp.key_scale,
                                 inp.value_scale, 0, slopes, status=status, tune=tune)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ks, vs = inp.flat_scales()
    ref = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables, inp.context_lens,
                                    inp.query_indptr(), ks, vs, alibi_slopes=slopes)
    assert_close(unpack_mtp(out, cfg.num_seqs, ql, hkv), ref, what="alibi")
    no_bias, _ = run_operator(inp, tune=tune)
    assert (unpack_mtp(out, cfg.num_seqs, ql, hkv).float() - no_bias.float()).abs().max() > 1e-2   # the bias matters


def _triton_golden(name):
    import importlib.util, os
    import numpy as np
    here = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_golden_triton", os.path.join(here, "make_golden_triton.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    z = np.load(os.path.join(here, name + ".npz"))
    inp, slopes = mod.case_inputs(name)
    return inp, slopes, {k: torch.from_numpy(z[k].copy()) for k in ("out", "tmp_output", "exp_sums", "max_logits")}


@pytest.mark.parametrize("name", ["triton_g4", "triton_g4_alibi", "triton_g16", "triton_g16_alibi"])
@pytest.mark.parametrize("kv", ["bf16", "fp8"])
def test_operator_matches_the_reference_triton_run(name, kv):
    """Output and split-KV intermediates against fixtures the reference's own Triton decode produced
    (pa_decode_triton.py:523-685 under the Triton interpreter, fp16 arithmetic), with and without
    ALiBi: the bf16-KV kernel on the same values, and the fp8 kernels on the values quantised per
    tensor (then the fixture is only as close as the quantisation allows: looser bounds, stated)."""
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import from_paged_key, from_paged_value, quantize_per_tensor, to_paged_key, to_paged_value
    inp, slopes, gold = _triton_golden(name)
    inp = inp.to(DEV)
    c = inp.cfg
    kc, vc, ksc, vsc = inp.key_cache, inp.value_cache, None, None
    if kv == "fp8":
        k8, ksc = quantize_per_tensor(from_paged_key(kc).contiguous())
        v8, vsc = quantize_per_tensor(from_paged_value(vc).contiguous())
        kc, vc = to_paged_key(k8), to_paged_value(v8)
    out = torch.full_like(inp.query, float("nan"))
    st = _status()
    res = paged_attention_decode(out, inp.query, kc, vc, inp.context_lens, inp.block_tables, inp.softmax_scale, 1,
                                 inp.max_context, torch.bfloat16, None, ksc, vsc, 0,
                                 None if slopes is None else slopes.to(DEV), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    # bf16 KV: the same values as the reference saw; tolerance = this build's bar for bf16 outputs.
    # fp8 KV: e4m3 keeps 4 significant bits of each key / value element; the per-element noise
    # averages out over the head dimension and the context, one e4m3 element is off by up to 6 %, and ALiBi with a steep slope makes an output row nearly one value row.
    atol, rtol = (ATOL, RTOL) if kv == "bf16" else (6e-2, 7e-2)
    assert_close(out, gold["out"], atol=atol, rtol=rtol, what=f"{name} {kv}: output")
    m, l, o = res["maximum_logits"].cpu(), res["exponential_sums"].cpu(), res["temporary_output"].float().cpu()
    if kv == "bf16":
        for s in range(c.num_seqs):
            np_s = (int(inp.context_lens[s]) + 255) // 256
            assert torch.allclose(m[s, :, :np_s], gold["max_logits"][s, :, :np_s], atol=1e-2, rtol=2e-3)
            assert torch.allclose(l[s, :, :np_s], gold["exp_sums"][s, :, :np_s], atol=1e-3, rtol=1e-2)
            assert torch.allclose(o[s, :, :np_s], gold["tmp_output"][s, :, :np_s], atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("heads,ql,bs,kv", [((32, 8), 1, 16, "fp8"), ((16, 2), 2, 1024, "fp8"), ((8, 2), 1, 16, "bf16")])
def test_sink_tokens(heads, ql, bs, kv):
    """Sink logits join the softmax denominator in the reduce (pa_decode_triton_gluon_fp8.py:1117-1123)."""
    from oracle import pa_oracle
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, unpack_mtp
    hq, hkv = heads
    cfg = DecodeConfig("sink", 3, hq, hkv, bs, ql, ("fixed", 1), kv_dtype=kv, quant="per_tensor" if kv == "fp8" else "none")
    inp = make_inputs(cfg, seed=41, device=DEV, context_lens=torch.tensor([600, 1300, 40]))
    sinks = torch.linspace(-1.0, 3.0, hq).to(DEV)
    out = torch.full_like(inp.query, float("nan"))
    paged_attention_decode(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                           inp.softmax_scale, ql, inp.max_context, torch.bfloat16, None, inp.key_scale,
                           inp.value_scale, sink_tokens=sinks)
    torch.cuda.synchronize()
    ks, vs = inp.flat_scales()
    ref = pa_oracle.paged_attention(inp.query_tokens, inp.key_cache, inp.value_cache, inp.block_tables, inp.context_lens,
                                    inp.query_indptr(), ks, vs, sink_tokens=sinks)
    assert_close(unpack_mtp(out, cfg.num_seqs, ql, hkv), ref, what="sink tokens")


def test_operator_is_cuda_graph_capturable():
    """No allocation, no synchronisation, launches on the current stream: a decode call (both kernels,
    the reduce with its programmatic-launch attribute) can be captured once and replayed per step."""
    from triton_op_b200 import paged_attention_decode
    from triton_op_b200.inputs import DecodeConfig, make_inputs, unpack_mtp
    cfg = DecodeConfig("graph", 4, 16, 2, 16, 2, ("fixed", 1), quant="per_token")
    inp = make_inputs(cfg, seed=7, device=DEV, context_lens=torch.tensor([300, 1025, 16, 700]))
    out = torch.zeros_like(inp.query)

    def step():
        paged_attention_decode(out, inp.query, inp.key_cache, inp.value_cache, inp.context_lens, inp.block_tables,
                               inp.softmax_scale, 2, inp.max_context, torch.bfloat16, None, inp.key_scale, inp.value_scale)

    step()                                   # creates the cached workspaces outside the capture
    torch.cuda.synchronize()
    eager = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    # the graph reads lengths and tables from device memory at replay time: a shorter context changes the result
    inp.context_lens[1] = 512
    graph.replay()
    torch.cuda.synchronize()
    assert not torch.equal(out[1], eager[1]) and torch.equal(out[0], eager[0])
    assert_close(unpack_mtp(out, 4, 2, 2), oracle_output(inp), what="graph replay after a length change")


@pytest.mark.parametrize("name", ["cfg3_llama70b_mtp", "cfg4_longctx", "cfg5_serving_fp8", "cfg5_serving_bf16"])
def test_baseline_configs_full_size_properties(name):
    """The other baseline workloads at their full size.  The oracle checks a sample of sequences;
    the rest is covered by properties that do not depend on the size: a sequence's rows do not
    depend on which other sequences share the call (bit-identical in a sub-batch), and with a
    constant value cache every output equals that constant times the value scale."""
    import copy
    from triton_op_b200.inputs import CONFIGS, make_inputs
    cfg = CONFIGS[name]
    inp = make_inputs(cfg, seed=0, device=DEV)
    st = _status()
    out, _ = run_operator(inp, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and bool(torch.isfinite(out.float()).all())
    L = cfg.query_len
    g = torch.Generator().manual_seed(1)
    pick = sorted(torch.randperm(cfg.num_seqs, generator=g)[:min(6, cfg.num_seqs)].tolist())
    sub = copy.copy(inp)
    sub.cfg = type(cfg)(**{**cfg.__dict__, "num_seqs": len(pick)})
    rows = [s * L + t for s in pick for t in range(L)]
    sub.query_tokens = inp.query_tokens[rows]
    sub.query = inp.query[pick]
    sub.block_tables = inp.block_tables[pick]
    sub.context_lens = inp.context_lens[pick]
    assert_close(out[rows], oracle_output(sub), what=f"{name}: sampled sequences vs oracle")
    out_sub, _ = run_operator(sub, status=st)
    assert torch.equal(out_sub, out[rows])
    if cfg.quant != "per_token":          # (per-token value scales differ by token: no constant output)
        const = copy.copy(inp)
        const.value_cache = torch.full_like(inp.value_cache.float(), 0.75).to(inp.value_cache.dtype)
        out_c, _ = run_operator(const, status=st)
        expect = 0.75 * (float(inp.value_scale) if inp.value_scale is not None else 1.0)
        assert torch.allclose(out_c.float(), torch.full_like(out_c.float(), expect), rtol=1e-2, atol=0)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
