"""KV-cache write side.  CPU: the oracle's token-wise write reproduces the whole-cache builders
(layouts and quantisers the golden cases are made with).  GPU: the CUDA kernel writes the same
bytes and scales as the oracle, and a cache written by it decodes to the oracle's attention."""
from __future__ import annotations

import pytest
import torch

from triton_op_b200.inputs import (FP8, quantize_per_token, shuffle_value_cache_layout, to_paged_key, to_paged_value)


def _tokens(nb, hkv, bs, d, seed):
    g = torch.Generator()
    g.manual_seed(seed)
    k = torch.randn(nb, hkv, bs, d, generator=g).to(torch.bfloat16)
    v = torch.randn(nb, hkv, bs, d, generator=g).to(torch.bfloat16)
    return k, v


def _as_stream(x_tok):
    """[NB, Hkv, bs, D] -> ([NB*bs, Hkv, D] token stream, slots) with slot = block*bs + offset."""
    nb, hkv, bs, d = x_tok.shape
    return x_tok.permute(0, 2, 1, 3).reshape(nb * bs, hkv, d).contiguous()


@pytest.mark.parametrize("bs", [16, 64])
@pytest.mark.parametrize("mode", ["per_token", "per_tensor", "bf16"])
def test_oracle_write_reproduces_the_cache_builders(bs, mode):
    from oracle import pa_oracle
    nb, hkv, d = 5, 2, 128
    k_tok, v_tok = _tokens(nb, hkv, bs, d, seed=bs)
    slots = torch.randperm(nb * bs, generator=torch.Generator().manual_seed(1))      # every slot once, any order
    k_stream, v_stream = _as_stream(k_tok)[slots], _as_stream(v_tok)[slots]
    if mode == "bf16":
        kc = torch.zeros(nb, hkv, d // 8, bs, 8, dtype=torch.bfloat16)
        vc = torch.zeros(nb, hkv, d, bs, dtype=torch.bfloat16)
        pa_oracle.write_kv_cache(k_stream, v_stream, kc, vc, slots)
        assert torch.equal(kc, to_paged_key(k_tok)) and torch.equal(vc, to_paged_value(v_tok))
        return
    kc = torch.zeros(nb, hkv, d // 16, bs, 16).to(FP8)
    vc = torch.zeros(nb, hkv, d, bs).to(FP8)
    if mode == "per_token":
        ks, vs = torch.zeros(nb, hkv, bs, 1), torch.zeros(nb, hkv, bs, 1)
        pa_oracle.write_kv_cache(k_stream, v_stream, kc, vc, slots, ks, vs)
        qk, sk = quantize_per_token(k_tok.float())
        qv, sv = quantize_per_token(v_tok.float())
        assert torch.equal(ks, sk) and torch.equal(vs, sv)
    else:
        sk = (k_tok.float().abs().amax() / 448.0).clamp_min(1e-12)
        sv = (v_tok.float().abs().amax() / 448.0).clamp_min(1e-12)
        pa_oracle.write_kv_cache(k_stream, v_stream, kc, vc, slots, sk, sv)
        qk, qv = (k_tok.float() / sk).to(FP8), (v_tok.float() / sv).to(FP8)
    assert torch.equal(kc.view(torch.uint8), to_paged_key(qk).view(torch.uint8))
    assert torch.equal(vc.view(torch.uint8), to_paged_value(qv).view(torch.uint8))
    # shuffled value layout
    vt = torch.zeros(nb, hkv, bs // 16, d, 16).to(FP8)
    args = (ks.clone(), vs.clone()) if mode == "per_token" else (sk, sv)
    pa_oracle.write_kv_cache(k_stream, v_stream, kc.clone(), vt, slots, *args)
    assert torch.equal(vt.view(torch.uint8), shuffle_value_cache_layout(to_paged_value(qv)).view(torch.uint8))


@pytest.mark.gpu
@pytest.mark.parametrize("bs", [16, 64, 1024])
@pytest.mark.parametrize("mode", ["per_token", "per_tensor", "unscaled", "bf16", "per_token_trans"])
def test_cuda_write_is_bit_exact(bs, mode):
    from oracle import pa_oracle
    from triton_op_b200.cache_write import write_kv_cache
    dev = "cuda:0"
    nb, hkv, d = 6, 3, 128
    T = min(200, nb * bs - 5)
    g = torch.Generator().manual_seed(100 + bs)
    key = (torch.randn(T, hkv, d, generator=g) * 3).to(torch.bfloat16)
    value = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    key[7] = 0                                                   # an all-zero vector: scale clamps to 1e-12
    value[5, 1, 17] = 9.0                                        # beyond the range of a static scale: saturates
    slots = torch.randperm(nb * bs, generator=g)[:T].to(torch.int64)
    slots[11] = -1                                               # skipped token
    trans = mode.endswith("trans")
    if mode == "bf16":
        kc = torch.full((nb, hkv, d // 8, bs, 8), 7.0, dtype=torch.bfloat16)
        vc = torch.full((nb, hkv, d, bs), 7.0, dtype=torch.bfloat16)
        scales = (None, None)
    else:
        kc = torch.full((nb, hkv, d // 16, bs, 16), 1.0).to(FP8)
        vc = (torch.full((nb, hkv, bs // 16, d, 16), 1.0) if trans else torch.full((nb, hkv, d, bs), 1.0)).to(FP8)
        if mode.startswith("per_token"):
            scales = (torch.full((nb, hkv, bs, 1), -1.0), torch.full((nb, hkv, bs, 1), -1.0))
        elif mode == "per_tensor":
            scales = (torch.tensor(0.0371), torch.tensor(0.0093))
        else:
            scales = (None, None)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    sc_ref = tuple(None if s is None else s.clone() for s in scales)
    pa_oracle.write_kv_cache(key, value, kc_ref, vc_ref, slots, *sc_ref)
    kc_d, vc_d = kc.to(dev), vc.to(dev)
    sc_d = tuple(None if s is None else s.to(dev) for s in scales)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    write_kv_cache(key.to(dev), value.to(dev), kc_d, vc_d, slots.to(dev), *sc_d, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    as_bytes = lambda t: t.cpu().view(torch.uint8) if t.dtype != torch.bfloat16 else t.cpu().view(torch.int16)
    assert torch.equal(as_bytes(kc_d), as_bytes(kc_ref))
    assert torch.equal(as_bytes(vc_d), as_bytes(vc_ref))
    if mode.startswith("per_token"):
        assert torch.equal(sc_d[0].cpu(), sc_ref[0]) and torch.equal(sc_d[1].cpu(), sc_ref[1])


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["per_token", "per_tensor"])
def test_cuda_write_rounds_ties_and_tiny_values_like_the_oracle(mode):
    """Inputs made to land on the rounding boundaries: quotients that are exact halfway points
    between two e4m3 values (ties go to even), quotients in e4m3's subnormal range and below its
    smallest step, bf16 subnormals, and the largest finite bf16.  Bytes and scales as the oracle's."""
    from oracle import pa_oracle
    from triton_op_b200.cache_write import write_kv_cache
    dev = "cuda:0"
    nb, hkv, d, bs, T = 40, 2, 128, 16, 600
    g = torch.Generator().manual_seed(77)
    halfway = torch.tensor([1.0625, 1.1875, 1.3125, 1.4375, 1.5625, 1.6875, 1.8125, 1.9375])

    def adversarial():
        sign = torch.where(torch.rand(T, hkv, d, generator=g) < 0.5, -1.0, 1.0)
        m = halfway[torch.randint(0, 8, (T, hkv, d), generator=g)]
        e = torch.randint(-12, 8, (T, hkv, d), generator=g).float()
        x = sign * m * torch.exp2(e)
        x[:, :, 0] = 448.0 * torch.exp2(torch.randint(-3, 3, (T, hkv), generator=g).float())   # amax: a power-of-two scale
        x[::7, :, 5] = 1e-39                      # bf16 subnormal
        x[::11, :, 9] = 2.0 ** -30
        x[3::13, 0, :] *= 2.0 ** -11              # whole vectors of small quotients
        x[5, 1, 0] = 3.3895e38                    # largest finite bf16: the scale itself is huge
        return x.to(torch.bfloat16)

    key, value = adversarial(), adversarial()
    slots = torch.randperm(nb * bs, generator=g)[:T].to(torch.int64)
    slots[: 16 * 20] = torch.arange(16 * 20) + 16 * 3          # twenty full runs: the vector-store path too
    seen = set()
    keep = [i for i, v in enumerate(slots.tolist()) if not (v in seen or seen.add(v))]
    slots, key, value = slots[keep], key[keep], value[keep]
    kc = torch.full((nb, hkv, d // 16, bs, 16), 1.0).to(FP8)
    vc = torch.full((nb, hkv, d, bs), 1.0).to(FP8)
    if mode == "per_token":
        scales = (torch.full((nb, hkv, bs, 1), -1.0), torch.full((nb, hkv, bs, 1), -1.0))
    else:
        scales = (torch.tensor(2.0 ** -4), torch.tensor(0.173))
    kc_ref, vc_ref = kc.clone(), vc.clone()
    sc_ref = tuple(s.clone() for s in scales)
    pa_oracle.write_kv_cache(key, value, kc_ref, vc_ref, slots, *sc_ref)
    kc_d, vc_d = kc.to(dev), vc.to(dev)
    sc_d = tuple(s.to(dev) for s in scales)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    write_kv_cache(key.to(dev), value.to(dev), kc_d, vc_d, slots.to(dev), *sc_d, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.equal(kc_d.cpu().view(torch.uint8), kc_ref.view(torch.uint8))
    assert torch.equal(vc_d.cpu().view(torch.uint8), vc_ref.view(torch.uint8))
    if mode == "per_token":
        assert torch.equal(sc_d[0].cpu(), sc_ref[0]) and torch.equal(sc_d[1].cpu(), sc_ref[1])


def _prefill_slots(nb, bs, chunks, g):
    """Slots of token streams that walk pages the way a prefill chunk does: consecutive positions of a
    sequence from a start offset inside its first page, pages taken from a shuffled pool."""
    pool = torch.randperm(nb, generator=g).tolist()
    slots = []
    for start, n in chunks:
        pages = [pool.pop() for _ in range((start + n + bs - 1) // bs)]
        slots += [pages[(start + i) // bs] * bs + (start + i) % bs for i in range(n)]
    return slots


@pytest.mark.gpu
@pytest.mark.parametrize("bs,mode", [(16, "per_token"), (16, "per_tensor"), (64, "per_token"), (64, "per_token_trans"),
                                     (1024, "unscaled"), (16, "per_token_unaligned")])
def test_cuda_write_of_long_streams_is_bit_exact(bs, mode):
    """Streams with full runs of 16 consecutive slots, which one warp writes whole: prefill-style
    chunks with ragged ends, single scattered tokens between them, a skipped token and a slot outside
    the pool.  Same bytes and scales as the oracle's token-wise write."""
    from oracle import pa_oracle
    from triton_op_b200 import _lib
    from triton_op_b200.cache_write import write_kv_cache
    dev = "cuda:0"
    hkv, d = 8, 128
    nb = 400 if bs == 16 else (100 if bs == 64 else 12)
    g = torch.Generator().manual_seed(7 + bs)
    chunks = [(5, 700), (0, 512), (15, 33), (9, 1500), (3, 1), (0, 16), (1, 15), (8, 1290)]
    slots = _prefill_slots(nb, bs, chunks, g)
    used = set(slots)
    free = [s for s in range(nb * bs) if s not in used]
    singles = [free[i] for i in torch.randperm(len(free), generator=g)[:60].tolist()]
    slots = slots[:1200] + singles[:30] + slots[1200:] + singles[30:]
    slots[40] = -1                                               # skipped token inside a run
    slots.append(nb * bs + 3)                                    # outside the pool: reported, skipped
    T = len(slots)
    slots = torch.tensor(slots, dtype=torch.int64)
    key = (torch.randn(T, hkv, d, generator=g) * 3).to(torch.bfloat16)
    value = torch.randn(T, hkv, d, generator=g).to(torch.bfloat16)
    key[100] = 0
    trans = mode.endswith("trans")
    kc = torch.full((nb, hkv, d // 16, bs, 16), 1.0).to(FP8)
    vc = (torch.full((nb, hkv, bs // 16, d, 16), 1.0) if trans else torch.full((nb, hkv, d, bs), 1.0)).to(FP8)
    if mode.startswith("per_token"):
        scales = (torch.full((nb, hkv, bs, 1), -1.0), torch.full((nb, hkv, bs, 1), -1.0))
    elif mode == "per_tensor":
        scales = (torch.tensor(0.0371), torch.tensor(0.0093))
    else:
        scales = (None, None)
    kc_ref, vc_ref = kc.clone(), vc.clone()
    sc_ref = tuple(None if s is None else s.clone() for s in scales)
    pa_oracle.write_kv_cache(key[:-1], value[:-1], kc_ref, vc_ref, slots[:-1], *sc_ref)
    kc_d, vc_d = kc.to(dev), vc.to(dev)
    sc_d = tuple(None if s is None else s.to(dev) for s in scales)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    key_d = key.to(dev)
    if mode.endswith("unaligned"):      # rows 8 bytes off a 16-byte boundary: no vector accesses, every token written alone
        wide = torch.zeros(T, hkv, d + 8, dtype=torch.bfloat16, device=dev)
        wide[:, :, 4:4 + d] = key_d
        key_d = wide[:, :, 4:4 + d]
        assert key_d.data_ptr() % 16 == 8
    write_kv_cache(key_d, value.to(dev), kc_d, vc_d, slots.to(dev), *sc_d, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.PA_DEV_BAD_PAGE_ID
    assert torch.equal(kc_d.cpu().view(torch.uint8), kc_ref.view(torch.uint8))
    assert torch.equal(vc_d.cpu().view(torch.uint8), vc_ref.view(torch.uint8))
    if mode.startswith("per_token"):
        assert torch.equal(sc_d[0].cpu(), sc_ref[0]) and torch.equal(sc_d[1].cpu(), sc_ref[1])


@pytest.mark.gpu
def test_slot_outside_the_pool_is_reported_and_skipped():
    from triton_op_b200 import _lib
    from triton_op_b200.cache_write import write_kv_cache
    dev = "cuda:0"
    nb, hkv, d, bs = 2, 1, 128, 16
    kc = torch.zeros(nb, hkv, d // 16, bs, 16, device=dev).to(FP8)
    vc = torch.zeros(nb, hkv, d, bs, device=dev).to(FP8)
    key = torch.ones(2, hkv, d, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    write_kv_cache(key, key, kc, vc, torch.tensor([3, nb * bs + 5], device=dev), status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == _lib.PA_DEV_BAD_PAGE_ID
    assert int(kc.view(torch.uint8).ne(0).sum()) == d            # only the valid token was written


@pytest.mark.gpu
def test_decode_reads_what_the_write_kernel_wrote():
    """End to end over both sides of the path: tokens -> write kernel -> decode operator, against the
    oracle on the builder-made cache."""
    from _util import assert_close, oracle_output, run_operator
    from triton_op_b200.cache_write import slots_for, write_kv_cache
    from triton_op_b200.inputs import DecodeConfig, from_paged_key, from_paged_value, make_inputs
    dev = "cuda:0"
    cfg = DecodeConfig("rw", 3, 16, 2, 16, 2, ("fixed", 1), quant="per_token")
    lens = [700, 33, 2049]
    ref_inp = make_inputs(cfg, seed=31, device=dev, context_lens=torch.tensor(lens))
    # recover bf16 token vectors from the builder's cache (dequantised), then write them through the kernel
    nb, hkv, bs = ref_inp.key_cache.shape[0], 2, 16
    k_tok = (from_paged_key(ref_inp.key_cache).float() * ref_inp.key_scale).to(torch.bfloat16)
    v_tok = (from_paged_value(ref_inp.value_cache).float() * ref_inp.value_scale).to(torch.bfloat16)
    seq_ids = torch.cat([torch.full((n,), s) for s, n in enumerate(lens)]).to(dev)
    pos = torch.cat([torch.arange(n) for n in lens]).to(dev)
    slots = slots_for(ref_inp.block_tables, pos, seq_ids, bs)
    blk, off = slots // bs, slots % bs
    key = k_tok[blk, :, off, :].contiguous()
    value = v_tok[blk, :, off, :].contiguous()
    kc = torch.zeros_like(ref_inp.key_cache)
    vc = torch.zeros_like(ref_inp.value_cache)
    ks = torch.ones_like(ref_inp.key_scale)
    vs = torch.ones_like(ref_inp.value_scale)
    write_kv_cache(key, value, kc, vc, slots, ks, vs)
    import copy
    inp = copy.copy(ref_inp)
    inp.key_cache, inp.value_cache, inp.key_scale, inp.value_scale = kc, vc, ks, vs
    out, _ = run_operator(inp)
    torch.cuda.synchronize()
    assert_close(out, oracle_output(inp), what="decode after write")
