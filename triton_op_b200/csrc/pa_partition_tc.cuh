// Split-KV partition kernel on the tcgen05 tensor cores: e4m3fn KV cache, 16-token pages,
// 256-token partitions, up to 8 query rows per kv head (eqG = query_len * group <= 8).
//
// Same contract as paged_attention_decode_v2_gluon_fp8 of yanguahe/triton_op
// (pa_decode_triton_gluon_fp8.py:514-1002): per (sequence, kv head, partition) it stores
// m = max_j s_j, l = sum_j exp(s_j - m) and o = sum_j exp(s_j - m) v_j / l.
//
// Why this shape.  sm_100a has no native fp8 mma.sync: an e4m3 mma.sync is expanded into
// byte->half converts plus f16 tiles, and those converts (quarter-rate pipe) cap a register-level
// kernel near 65 % of HBM bandwidth.  tcgen05.mma kind::f8f6f4 multiplies e4m3 operands straight
// out of shared memory, so here no KV byte ever passes through a register:
//
//   bulk copy (page of one head = one contiguous 2 KB run)  ->  shared memory  ->  tensor core.
//
// The tiles are transposed so that the long axis fills M = 128:
//   S^T[128 tokens, N] = K[128 tokens, 128 d] . Q^T        (4 instructions, K = 32 each)
//   O^T[128 d,      N] = V^T[128 d, 256 tokens] . P^T      (8 instructions)
// with N = 16 columns = 8 query rows x {hi, lo}: the bf16 query and the probabilities are split
// into two e4m3 numbers each (x = hi + lo/16, 8 significant bits), so the products are exact and
// the result has bf16-level precision although the tensor core only sees e4m3.
//
// Both paged layouts are already what the tensor core wants (K-major "core matrices" of 8 rows
// x 16 bytes, no swizzle), so pages are copied verbatim and the descriptors do the gather:
//   K page [D/16][16 tok][16 B]: rows = tokens.  Pages sit 2 KB apart in the slot, so one M = 128
//     instruction takes tokens tg*8..tg*8+7 of each of the 16 pages (stride between 8-row groups =
//     2048 B, between the two 16-byte K units = 256 B); tg = 0, 1 covers the partition.
//   V page [D][16 tok]: rows = head dims (128 B between groups of 8), the two K units of an
//     instruction are two consecutive pages (2048 B apart).
//
// One CTA per SM, persistent over work items (an item = one partition of one kv head), 4*NG + 4
// warps with fixed roles joined by mbarriers (NG = 3):
//   warps 0 .. 4*NG-1   NG softmax + epilogue groups of four warps; a thread = one TMEM lane (a
//                       token of S^T, a head dim of O^T).  Group g takes the CTA's items g, g+NG,
//                       ... and owns its own S^T / O^T columns and P^T tile, so the per-item
//                       latency chain of a group (TMEM loads, reductions, P^T stores) overlaps
//                       the chains of the other groups.
//   warp 4*NG           tcgen05.mma issue (one elected lane) and TMEM allocation
//   warp 4*NG+1 / +2    K / V producers: one 2 KB bulk copy per page, page ids prefetched an item ahead
//   warp 4*NG+3         query producer: bf16 -> hi/lo e4m3 tile in the B-operand layout, per-token scales
// A ring of item slots (K 32 KB + V 32 KB each) keeps two items of copies in flight while a
// third is being consumed.  Every wait is bounded and reports PA_DEV_WAIT_TIMEOUT.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "pa_partition_fp8.cuh"  // Item, decode_item, build_partition_index
#include "pa_tcgen05.cuh"
#include "../../include/pa_decode_sm100.h"

namespace pa {
namespace tc {

constexpr int kItemTokens = 256;
constexpr int kItemPages = 16;
constexpr int kHalfSlot = kItemPages * kPageBytes;  // 32 KB: K (or V) of one item
constexpr int kSlotBytes = 2 * kHalfSlot;
constexpr int kNQ = 16;                             // MMA N: 8 query rows x {hi, lo}
constexpr int kQTileBytes = kNQ * kD;               // 2 KB: [2 row blocks][8 chunks][8 rows][16 B]
constexpr int kNG = 3;                              // softmax groups
constexpr int kMaxGroups = 4;
constexpr int kThreads = (4 * kNG + 4) * 32;
constexpr int kMaxSlots = 4;
// Query slot: the tile, 16 floats of per-row scales, and (per-token mode) 2 x 256 token scales.
__host__ __device__ constexpr int q_slot_bytes(bool per_token) {
  return kQTileBytes + 64 + (per_token ? 2 * kItemTokens * 4 : 0);
}
// P^T tile of one item: 8 k-steps x [2 row blocks (hi | lo)][2 K units][8 rows][16 tokens].  The
// strides are padded off the 128-byte grid so that the byte stores of a warp, which go to four
// different pages (= K units), fall into different banks.
constexpr int kPLbo = 144;                          // between the two K units of a k-step
constexpr int kPSbo = 288;                          // between the hi and the lo row block
constexpr int kPStep = 560;                         // between k-steps
constexpr int kPTileBytes = 8 * kPStep;
// TMEM columns: S^T of group g at 32*g (two 16-column halves), O^T of group g, parity b at
// 32*kMaxGroups + 32*g + 16*b.
constexpr int kTmemCols = 256;
constexpr int kTmemO = 32 * kMaxGroups;

// barrier indices inside the barrier block
// A parity wait is only meaningful while the waiter is at most one phase ahead of the barrier,
// so every barrier below is waited on either by one role in item order, or by a role that has
// first observed an event implying the previous phase (noted at the wait).
enum : int {
  kBarKQFull = 0,   // [slot] K pages landed (transaction bytes) + query tile written: 2 arrivals
  kBarVFull = 4,    // [slot] V pages landed
  kBarQEmpty = 8,   // [slot] the softmax group has read the slot's scales: 4 arrivals
  kBarSFull = 12,   // [group] QK^T of the group's current item is complete (commit); this also
                    //         frees the item's K pages and query tile
  kBarPFull = 16,   // [group] P^T stored, V cleared where needed, S^T consumed: 4 arrivals
  kBarOFull = 20,   // [group][parity] P.V complete (commit); this also frees the item's V pages
  kNumBars = 28
};
// fixed head of the shared-memory carve (bytes).  A softmax group keeps two items in flight (the
// softmax of its next item runs before the epilogue of the previous one), so what the epilogue
// reads is double buffered by the item's parity inside the group.
constexpr int kOffBars = 0;
constexpr int kOffTmemPtr = 384;
constexpr int kOffScan = 400;                     // 32 ints
constexpr int kOffRedMax = 640;                   // [groups][8 q][4 warps] floats
constexpr int kOffRedSum = 1152;                  // [groups][2 parities][8 q][4 warps] floats
constexpr int kOffMFin = 2176;                    // [groups][2 parities][8] floats (max, log2 domain)
constexpr int kOffVMax = 2432;                    // [groups][4 warps] floats (per-token V scale max)
constexpr int kOffVNorm = 2496;                   // [groups][2 parities] floats
constexpr int kHeadBytes = 2560;

// Walks the work items of one role: item k = first, first + step, ...  Decoding an item index
// into (sequence, partition, head) needs a search in the partition prefix sum; the cursor does
// that once and afterwards only steps forward.
struct ItemCursor {
  int sp, head, seq, step_sp, step_head;
  __device__ __forceinline__ void init(int k, int step, const KernelParams& p, const int* seq_off) {
    sp = k / p.Hkv;
    head = k - sp * p.Hkv;
    step_sp = step / p.Hkv;
    step_head = step - step_sp * p.Hkv;
    int lo = 0, hi = p.S;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_off[mid] <= sp) lo = mid; else hi = mid;
    }
    seq = lo;
  }
  __device__ __forceinline__ void advance(const KernelParams& p, const int* seq_off) {
    head += step_head;
    sp += step_sp;
    if (head >= p.Hkv) {
      head -= p.Hkv;
      ++sp;
    }
    while (seq < p.S - 1 && seq_off[seq + 1] <= sp) ++seq;
  }
  __device__ __forceinline__ Item item(const KernelParams& p, const int* seq_off, const int* seq_ctx) const {
    Item it;
    it.seq = seq;
    it.head = head;
    it.part = sp - seq_off[seq];
    it.ctx = seq_ctx[seq];
    it.tok0 = it.part * kItemTokens;
    it.ntok = min(kItemTokens, it.ctx - it.tok0);
    it.npages = (it.ntok + kPageTokens - 1) / kPageTokens;
    it.nstages = 0;
    return it;
  }
};

// Monotonic float <-> int map, so a float maximum can use the single-instruction integer
// warp reduction.
__device__ __forceinline__ int float_to_ordered(float x) {
  const int i = __float_as_int(x);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) {
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

// Nine shuffles reduce eight values over the warp; lane ends up with the result for
// q = (lane >> 2) & 7.
template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce8(const float (&v)[8], int lane) {
  auto op = [](float a, float b) { return IS_MAX ? fmaxf(a, b) : a + b; };
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float a[4], b[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float mine = b4 ? v[4 + j] : v[j];
    const float other = b4 ? v[j] : v[4 + j];
    a[j] = op(mine, __shfl_xor_sync(kFullMask, other, 16));
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b3 ? a[2 + j] : a[j];
    const float other = b3 ? a[j] : a[2 + j];
    b[j] = op(mine, __shfl_xor_sync(kFullMask, other, 8));
  }
  float c = op(b2 ? b[1] : b[0], __shfl_xor_sync(kFullMask, b2 ? b[0] : b[1], 4));
  c = op(c, __shfl_xor_sync(kFullMask, c, 2));
  c = op(c, __shfl_xor_sync(kFullMask, c, 1));
  return c;
}

// Six shuffles for four values; lane ends up with the result for q = (lane >> 3) & 3.
template <bool IS_MAX>
__device__ __forceinline__ float warp_reduce4(const float (&v)[4], int lane) {
  auto op = [](float a, float b) { return IS_MAX ? fmaxf(a, b) : a + b; };
  const bool b4 = lane & 16, b3 = lane & 8;
  float a[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b4 ? v[2 + j] : v[j];
    const float other = b4 ? v[j] : v[2 + j];
    a[j] = op(mine, __shfl_xor_sync(kFullMask, other, 16));
  }
  float c = op(b3 ? a[1] : a[0], __shfl_xor_sync(kFullMask, b3 ? a[0] : a[1], 8));
  c = op(c, __shfl_xor_sync(kFullMask, c, 4));
  c = op(c, __shfl_xor_sync(kFullMask, c, 2));
  c = op(c, __shfl_xor_sync(kFullMask, c, 1));
  return c;
}

// PER_TOKEN: per-token-per-head K/V scales.  TRACE: compile the clock stamps in (tuning builds).
// QR: query rows the softmax handles (4 or 8, >= eqG).  Row q sits in tile row / TMEM column q
// (hi half) and QR + q (lo half), so with QR = 4 only the first row block is ever touched.
template <bool PER_TOKEN, bool TRACE, int QR>
__global__ void __launch_bounds__(kThreads, 1)
pa_partition_fp8_tc_kernel(const __grid_constant__ KernelParams p) {
  constexpr int NG = kNG;
  constexpr int kWarpMma = 4 * NG, kWarpK = 4 * NG + 1, kWarpV = 4 * NG + 2, kWarpQ = 4 * NG + 3;
  constexpr int kQSlotBytes = q_slot_bytes(PER_TOKEN);
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int NS = p.num_stages;  // item slots in the KV ring (and query ring)

  const uint32_t sbase = smem_addr(smem);
  const uint32_t bars = sbase + kOffBars;
  auto bar = [&](int which, int idx) -> uint32_t { return bars + (which + idx) * 8; };
  int* seq_off = reinterpret_cast<int*>(smem + p.off_seq_offsets);
  int* seq_ctx = reinterpret_cast<int*>(smem + p.off_seq_ctx);
  float* red_max = reinterpret_cast<float*>(smem + kOffRedMax);
  float* red_sum = reinterpret_cast<float*>(smem + kOffRedSum);
  float* m_fin = reinterpret_cast<float*>(smem + kOffMFin);
  float* v_max = reinterpret_cast<float*>(smem + kOffVMax);
  float* v_norm = reinterpret_cast<float*>(smem + kOffVNorm);
  const uint32_t q_ring = sbase + p.off_q;             // NS x kQSlotBytes
  const uint32_t p_tiles = sbase + p.off_p;            // NG x kPTileBytes
  const uint32_t kv_ring = sbase + p.off_ring;         // NS x kSlotBytes

  if (tid == 0) {
    for (int s = 0; s < kMaxSlots; ++s) {
      mbar_init(bar(kBarKQFull, s), 2);
      mbar_init(bar(kBarVFull, s), 1);
      mbar_init(bar(kBarQEmpty, s), 4);
    }
    for (int g = 0; g < kMaxGroups; ++g) {
      mbar_init(bar(kBarSFull, g), 1);
      mbar_init(bar(kBarPFull, g), 4);
      for (int b = 0; b < 2; ++b) mbar_init(bar(kBarOFull, 2 * g + b), 1);
    }
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == kWarpMma) tmem_alloc(sbase + kOffTmemPtr, kTmemCols);
  const int n_sp = build_partition_index(p, seq_off, seq_ctx, reinterpret_cast<int*>(smem + kOffScan));
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  grid_launch_dependents();  // the reduce kernel may become resident; it waits for this grid to finish
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + kOffTmemPtr);
  const uint32_t tmem_s = tmem_base;            // S^T of group g at column 32*g (+16 for tg = 1)
  const uint32_t tmem_o = tmem_base + kTmemO;   // O^T of group g, parity b at column 32*g + 16*b

  const int n_items = n_sp * p.Hkv;
  const int first = blockIdx.x;
  const int stride = gridDim.x;
  const int n_local = first < n_items ? (n_items - first + stride - 1) / stride : 0;
  bool dead = false;

  // Tuning aid: when p.trace is set, lane 0 of each role of CTA 0 stamps the SM clock at a few
  // points of its first 64 items: trace[(role * 64 + item) * 4 + point].
  auto stamp = [&](int role, int item, int point) {
    if (TRACE && p.trace != nullptr && blockIdx.x == 0 && lane == 0 && item < 64)
      p.trace[(role * 64 + item) * 4 + point] = (unsigned long long)clock64();
  };
  auto fail = [&]() {
    dead = true;
    if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_WAIT_TIMEOUT);
  };
  // whole-warp bounded wait, uniform result
  auto wait = [&](uint32_t b, uint32_t parity) -> bool {
    return __all_sync(kFullMask, mbar_wait(b, parity));
  };

  if (warp == kWarpK || warp == kWarpV) {
    // ------------------------------------------------------------------ K / V producer
    const bool is_v = warp == kWarpV;
    const uint8_t* cache = is_v ? p.v : p.k;
    const int64_t stride_block = is_v ? p.v_stride_block : p.k_stride_block;
    const int64_t stride_head = is_v ? p.v_stride_head : p.k_stride_head;
    const int full0 = is_v ? kBarVFull : kBarKQFull;
    const uint64_t pol = l2_policy_evict_first();
    auto load_page_id = [&](const Item& it) -> int {
      int id = 0;
      if (lane < it.npages) {
        id = __ldg(p.block_tables + (int64_t)it.seq * p.bt_stride_seq + (int64_t)it.part * kItemPages + lane);
        if ((unsigned)id >= (unsigned)p.num_blocks) {
          id = 0;
          if (p.status) atomicOr(p.status, PA_DEV_BAD_PAGE_ID);
        }
      }
      return id;
    };
    ItemCursor cur;
    Item it_next{};
    int pid_next = 0;
    if (n_local > 0) {
      cur.init(first, stride, p, seq_off);
      it_next = cur.item(p, seq_off, seq_ctx);
      pid_next = load_page_id(it_next);
    }
    for (int i = 0; i < n_local && !dead; ++i) {
      const Item it = it_next;
      const int pid = pid_next;
      if (i + 1 < n_local) {
        cur.advance(p, seq_off);
        it_next = cur.item(p, seq_off, seq_ctx);
        pid_next = load_page_id(it_next);
      }
      const int slot = i % NS;
      stamp(is_v ? 1 : 0, i, 0);
      if (i >= NS) {
        // The slot is free once the product that read it (item i - NS) is complete: QK^T for K
        // pages, P.V for V pages.  This role has already seen the products of all earlier items,
        // so the barrier's previous phase is known to be complete.
        const int j = i - NS;
        const int g = j % NG;
        const uint32_t gu = (uint32_t)(j / NG);
        const bool ok = is_v ? wait(bar(kBarOFull, 2 * g + (int)(gu & 1)), (gu >> 1) & 1)
                             : wait(bar(kBarSFull, g), gu & 1);
        if (!ok) { fail(); break; }
      }
      stamp(is_v ? 1 : 0, i, 1);
      const uint32_t full = bar(full0, slot);
      if (lane == 0) mbar_arrive_expect_tx(full, it.npages * kPageBytes);
      __syncwarp();
      if (lane < it.npages) {
        bulk_g2s(kv_ring + slot * kSlotBytes + (is_v ? kHalfSlot : 0) + lane * kPageBytes,
                 cache + (int64_t)pid * stride_block + (int64_t)it.head * stride_head, kPageBytes, full, pol);
      }
      stamp(is_v ? 1 : 0, i, 2);
    }
  } else if (warp == kWarpQ) {
    // ------------------------------------------------------------------ query (+ scales) producer
    // lane -> query row n0 = lane / 4, quarter qq = lane % 4 of the head dims (32 each)
    const int n0 = lane >> 2, qq = lane & 3;
    const bool row_ok = n0 < p.eqG;
    auto load_q = [&](const Item& it, uint4 (&raw)[4]) {
#pragma unroll
      for (int e = 0; e < 4; ++e) raw[e] = make_uint4(0u, 0u, 0u, 0u);
      if (row_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q + (int64_t)it.seq * p.q_stride_seq + (int64_t)(it.head * p.eqG + n0) * p.q_stride_head + qq * 64);
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[e] = __ldg(src + e);
      }
    };
    // per-token scales: lanes 0-15 fetch the K scales of page `lane`, lanes 16-31 the V scales
    auto load_page_id = [&](const Item& it) -> int {
      int id = 0;
      const int pg = lane & 15;
      if (PER_TOKEN && pg < it.npages) {
        id = __ldg(p.block_tables + (int64_t)it.seq * p.bt_stride_seq + (int64_t)it.part * kItemPages + pg);
        if ((unsigned)id >= (unsigned)p.num_blocks) id = 0;
      }
      return id;
    };
    auto load_scales = [&](const Item& it, int pid, uint4 (&raw)[4]) {
#pragma unroll
      for (int e = 0; e < 4; ++e) raw[e] = make_uint4(0u, 0u, 0u, 0u);
      if (PER_TOKEN && (lane & 15) < it.npages) {
        const float* base = (lane < 16 ? p.k_scale : p.v_scale) + (int64_t)pid * p.kvs_stride_block +
                            (int64_t)it.head * p.kvs_stride_head;
        const uint4* src = reinterpret_cast<const uint4*>(base);
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[e] = __ldg(src + e);
      }
    };
    ItemCursor cur;
    Item it_next{}, it_next2{};
    uint4 q_next[4], sc_next[4];
    int pid_next2 = 0;
    if (n_local > 0) {
      cur.init(first, stride, p, seq_off);
      it_next = cur.item(p, seq_off, seq_ctx);
      load_q(it_next, q_next);
      load_scales(it_next, load_page_id(it_next), sc_next);
      if (n_local > 1) {
        cur.advance(p, seq_off);
        it_next2 = cur.item(p, seq_off, seq_ctx);
        pid_next2 = load_page_id(it_next2);
      }
    }
    for (int i = 0; i < n_local && !dead; ++i) {
      const Item it = it_next;
      uint4 qraw[4], sraw[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) { qraw[e] = q_next[e]; sraw[e] = sc_next[e]; }
      if (i + 1 < n_local) {
        it_next = it_next2;
        load_q(it_next, q_next);
        load_scales(it_next, pid_next2, sc_next);
        if (i + 2 < n_local) {
          cur.advance(p, seq_off);
          it_next2 = cur.item(p, seq_off, seq_ctx);
          pid_next2 = load_page_id(it_next2);
        }
      }
      const int slot = i % NS;
      const uint32_t use = (uint32_t)(i / NS);
      stamp(2, i, 0);
      if (!wait(bar(kBarQEmpty, slot), (use & 1) ^ 1)) { fail(); break; }
      stamp(2, i, 1);
      const uint32_t qt = q_ring + slot * kQSlotBytes;
      const uint32_t aux = qt + kQTileBytes;
      // row maximum -> power-of-two pre-scale putting it in [128, 256)
      float x[32];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t w[4] = {qraw[e].x, qraw[e].y, qraw[e].z, qraw[e].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[e * 8 + 2 * k] = bf16_lo_to_f32(w[k]);
          x[e * 8 + 2 * k + 1] = bf16_hi_to_f32(w[k]);
        }
      }
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < 32; ++e) amax = fmaxf(amax, fabsf(x[e]));
      amax = quad_max(amax);
      float pre = 1.0f, inv_pre = 1.0f;
      const int be = (int)((__float_as_uint(amax) >> 23) & 0xff);
      if (be > 30 && be < 225) {
        pre = __uint_as_float((uint32_t)(254 + 7 - be) << 23);
        inv_pre = __uint_as_float((uint32_t)(be - 7) << 23);
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {  // the two 16-dim chunks of this lane's quarter
        uint32_t hi4[4], lo4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float hi[4], lo[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) split_hi_lo(x[c * 16 + k * 4 + e] * pre, hi[e], lo[e]);
          hi4[k] = pack_e4m3x4(hi[0], hi[1], hi[2], hi[3]);
          lo4[k] = pack_e4m3x4(lo[0], lo[1], lo[2], lo[3]);
        }
        if (n0 < QR) {  // tile row n0 holds the hi half, tile row QR + n0 the lo half
          const int nl = QR + n0;
          const uint32_t dst = qt + (2 * qq + c) * 128;
          sts128(dst + n0 * 16, make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]));
          sts128(dst + (nl >> 3) * 1024 + (nl & 7) * 16, make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]));
        }
      }
      if (qq == 0 && n0 < QR) {
        float qs = 1.0f;
        if (p.q_quant_mode == PA_QUANT_PER_TENSOR) qs = __ldg(p.q_scale);
        if (p.q_quant_mode == PA_QUANT_PER_TOKEN && row_ok)
          qs = __ldg(p.q_scale + (int64_t)it.seq * p.q_scale_stride_seq + it.head * p.eqG + n0);
        sts32(aux + n0 * 4, __float_as_uint(inv_pre * qs));
      }
      if (PER_TOKEN) {
        const uint32_t dst = aux + 64 + (lane < 16 ? 0 : kItemTokens * 4) + (lane & 15) * 64;
#pragma unroll
        for (int e = 0; e < 4; ++e) sts128(dst + e * 16, sraw[e]);
      }
      fence_proxy_async();  // the tile is read by the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarKQFull, slot));
      stamp(2, i, 2);
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issue
    constexpr uint32_t kIdesc = idesc_f32acc(128, kNQ, 0, 0);
    const bool leader = elect_one();  // the one lane that issues every MMA and commit
    // per item i: group g = i % NG, use gu = i / NG of the group's buffers, O^T parity gu & 1.
    // P.V of an item is issued kLag items after its QK^T, so a softmax group has that long to
    // turn S^T into P^T before this in-order issue loop would have to wait for it.  The S^T
    // columns QK^T(i) overwrites were read by the softmax of item i - NG, whose P.V was issued
    // one iteration ago (kLag = NG - 1), after that group's arrival.
    constexpr int kLag = NG - 1;  // the host guarantees num_stages > kLag
    for (int i = 0; i < n_local + kLag && !dead; ++i) {
      if (i < n_local) {  // S^T(i) = K . Q^T
        const int slot = i % NS, g = i % NG;
        const uint32_t use = (uint32_t)(i / NS);
        stamp(3, i, 0);
        if (!wait(bar(kBarKQFull, slot), use & 1)) { fail(); break; }
        stamp(3, i, 1);
        fence_after_sync();
        const uint64_t kd = smem_desc(kv_ring + slot * kSlotBytes, 256, kPageBytes);
        const uint64_t qd = smem_desc(q_ring + slot * kQSlotBytes, 128, 1024);
        const uint32_t d0 = tmem_s + g * 32;
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t ad = kd + (uint64_t)(((2 * j) * 256 + tg * 128) >> 4);
            const uint64_t bd = qd + (uint64_t)(((2 * j) * 128) >> 4);
            if (leader) mma_f8_ss(d0 + tg * 16, ad, bd, kIdesc, j > 0);
          }
        }
        if (leader) mma_commit(bar(kBarSFull, g));
        __syncwarp();
      }
      if (i >= kLag) {  // O^T(j) = V^T . P^T
        const int j = i - kLag;
        const int slot = j % NS, g = j % NG;
        const uint32_t gu = (uint32_t)(j / NG);
        const int ob = 2 * g + (int)(gu & 1);
        // The group arrives here only after it has seen the item's V pages land and after its
        // epilogue of two items ago has read the O^T columns this product overwrites.
        if (!wait(bar(kBarPFull, g), gu & 1)) { fail(); break; }
        stamp(3, j, 2);
        fence_after_sync();
        const uint64_t vd = smem_desc(kv_ring + slot * kSlotBytes + kHalfSlot, kPageBytes, 128);
        const uint64_t pd = smem_desc(p_tiles + g * kPTileBytes, kPLbo, kPSbo);
        const uint32_t d0 = tmem_o + ob * 16;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ad = vd + (uint64_t)(((2 * ks) * kPageBytes) >> 4);
          const uint64_t bd = pd + (uint64_t)((ks * kPStep) >> 4);
          if (leader) mma_f8_ss(d0, ad, bd, kIdesc, ks > 0);
        }
        if (leader) mma_commit(bar(kBarOFull, ob));
        __syncwarp();
        stamp(3, j, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue groups
    const int grp = warp >> 2;         // softmax group: takes items grp, grp + NG, ...
    const int wq = warp & 3;           // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;      // TMEM lane: S^T row (token slot) / O^T row (head dim)
    const int pg = r >> 3;             // page of the tokens this thread owns in S^T
    const int bar_a = 1 + grp, bar_b = 1 + kMaxGroups + grp;  // named barriers of the group
    const uint32_t lane_field = (uint32_t)(wq * 32) << 16;
    float k_scale_t = 1.0f, v_scale_t = 1.0f;
    if (!PER_TOKEN && p.kv_quant_mode == PA_QUANT_PER_TENSOR) {
      k_scale_t = __ldg(p.k_scale);
      v_scale_t = __ldg(p.v_scale);
    }
    const float base_scale = p.softmax_scale * kLog2e * k_scale_t;
    // row q sees token j iff j < ctx - lim_off[q]; padding rows see nothing
    int lim_off[QR];
#pragma unroll
    for (int q = 0; q < QR; ++q) lim_off[q] = q < p.eqG ? (p.L - 1 - q / p.G) : -0x40000000;
    float* rm = red_max + grp * 32;

    auto softmax = [&](int i, const Item& it) -> bool {
      const int slot = i % NS;
      const uint32_t use = (uint32_t)(i / NS), gu = (uint32_t)(i / NG);
      const int par = grp * 2 + (int)(gu & 1);  // double-buffer index of what the epilogue reads
      if (wq == 0) stamp(4, i, 0);
      if (!wait(bar(kBarSFull, grp), gu & 1)) return false;
      if (wq == 0) stamp(4, i, 1);
      // QK^T of the item is done, so its query tile was complete: this wait returns at once and
      // orders the producer's scale writes before the reads below.
      if (!wait(bar(kBarKQFull, slot), use & 1)) return false;
      const uint32_t aux = q_ring + slot * kQSlotBytes + kQTileBytes;
      float row_scale[QR];
      {
        const uint4 a = lds128(aux);
        const uint4 b = QR > 4 ? lds128(aux + 16) : make_uint4(0u, 0u, 0u, 0u);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int q = 0; q < QR; ++q) row_scale[q] = __uint_as_float(w[q]) * base_scale;
      }
      float ks_tok[2] = {1.f, 1.f}, vs_tok[2] = {1.f, 1.f};
      if (PER_TOKEN) {
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
          const int tl = pg * 16 + tg * 8 + (r & 7);
          ks_tok[tg] = __uint_as_float(lds32(aux + 64 + tl * 4));
          vs_tok[tg] = __uint_as_float(lds32(aux + 64 + kItemTokens * 4 + tl * 4));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarQEmpty, slot));

      fence_after_sync();
      uint32_t sraw[2][2 * QR];  // columns: hi halves of the QR rows, then their lo halves
      tmem_ld(tmem_s + lane_field + grp * 32, sraw[0]);
      tmem_ld(tmem_s + lane_field + grp * 32 + 16, sraw[1]);
      tmem_ld_wait();
      if (wq == 0) stamp(6, i, 0);

      float s[2][QR];
      int key[QR];
#pragma unroll
      for (int tg = 0; tg < 2; ++tg) {
        const int tok = it.tok0 + pg * 16 + tg * 8 + (r & 7);  // global token index
        const int room = it.ctx - tok;                         // > lim_off[q]  <=>  visible
#pragma unroll
        for (int q = 0; q < QR; ++q) {
          float v = fmaf(__uint_as_float(sraw[tg][QR + q]), 0.0625f, __uint_as_float(sraw[tg][q])) * row_scale[q];
          if (PER_TOKEN) v *= ks_tok[tg];
          s[tg][q] = (room > lim_off[q] && lim_off[q] >= 0) ? v : -INFINITY;
        }
        if (PER_TOKEN && room <= 0) vs_tok[tg] = 0.f;
      }
      // partition maximum per row: integer warp reduction on order-preserving keys
#pragma unroll
      for (int q = 0; q < QR; ++q) key[q] = __reduce_max_sync(kFullMask, float_to_ordered(fmaxf(s[0][q], s[1][q])));
      if (lane == 0) {
#pragma unroll
        for (int q = 0; q < QR; ++q) rm[q * 4 + wq] = ordered_to_float(key[q]);
      }
      if (PER_TOKEN) {
        const int vk = __reduce_max_sync(kFullMask, float_to_ordered(fmaxf(vs_tok[0], vs_tok[1])));
        if (lane == 0) v_max[grp * 4 + wq] = ordered_to_float(vk);
      }
      if (wq == 0) stamp(6, i, 1);
      named_barrier_sync(bar_a, 128);
      if (wq == 0) stamp(6, i, 2);
      float vinv = 1.0f, vnorm = 1.0f;
      if (PER_TOKEN) {
        const float4 vm4 = *reinterpret_cast<const float4*>(v_max + grp * 4);
        vnorm = fmaxf(fmaxf(vm4.x, vm4.y), fmaxf(vm4.z, vm4.w));
        vinv = vnorm > 0.f ? 1.0f / vnorm : 0.f;
      }
      float psum[QR];
      uint32_t pbytes[2][QR / 2];  // [tg][hi rows (QR/4 words), lo rows (QR/4 words)], row q = byte q % 4
      {
        float hi[2][QR], lo[2][QR];
#pragma unroll
        for (int q = 0; q < QR; ++q) {
          const float4 m4 = *reinterpret_cast<const float4*>(rm + q * 4);
          const float m = fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w));
          const float m_use = (m == -INFINITY) ? 0.f : m;
          if (r == q) m_fin[par * 8 + q] = m;
          const float p0 = ex2(s[0][q] - m_use + 8.0f);
          const float p1 = ex2(s[1][q] - m_use + 8.0f);
          psum[q] = p0 + p1;
          split_hi_lo(PER_TOKEN ? p0 * (vs_tok[0] * vinv) : p0, hi[0][q], lo[0][q]);
          split_hi_lo(PER_TOKEN ? p1 * (vs_tok[1] * vinv) : p1, hi[1][q], lo[1][q]);
        }
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
          for (int w = 0; w < QR / 4; ++w) {
            pbytes[tg][w] = pack_e4m3x4(hi[tg][4 * w], hi[tg][4 * w + 1], hi[tg][4 * w + 2], hi[tg][4 * w + 3]);
            pbytes[tg][QR / 4 + w] = pack_e4m3x4(lo[tg][4 * w], lo[tg][4 * w + 1], lo[tg][4 * w + 2], lo[tg][4 * w + 3]);
          }
        }
      }
      // The group's P^T tile is still being read by P.V of the group's previous item until that
      // product's commit has arrived (normally long ago).
      if (gu > 0) {
        const uint32_t pu = gu - 1;
        if (!wait(bar(kBarOFull, 2 * grp + (int)(pu & 1)), (pu >> 1) & 1)) return false;
      }
      // P^T tile of k-step pg/2: [row block (hi | lo)][K unit = pg % 2][row q][token]
      const uint32_t pt = p_tiles + grp * kPTileBytes + (pg >> 1) * kPStep + (pg & 1) * kPLbo + (r & 7);
#pragma unroll
      for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
        for (int q = 0; q < QR; ++q) {
          constexpr int kLoBlock = (QR >= 8) ? kPSbo : 0;  // tile row QR + q: row block, then row
          sts8(pt + q * 16 + tg * 8, pbytes[tg][q >> 2] >> (8 * (q & 3)));
          sts8(pt + kLoBlock + ((QR + q) & 7) * 16 + tg * 8, pbytes[tg][QR / 4 + (q >> 2)] >> (8 * (q & 3)));
        }
      }
      if (wq == 0) stamp(6, i, 3);
      // Bytes of V past the context (absent pages, tokens past the end of the last page) may
      // hold anything, NaN patterns included, and 0 * NaN would poison O^T: clear them.
      // (P.V of the previous item in this slot was issued before QK^T of this one, so the V
      // barrier's previous phase is complete.)
      if (!wait(bar(kBarVFull, slot), use & 1)) return false;
      if (it.ntok < kItemTokens) {
        const uint32_t vrow = kv_ring + slot * kSlotBytes + kHalfSlot + r * 16;  // row = head dim r
        const int first_bad = it.ntok >> 4;           // page holding the first invalid token
        const int keep = it.ntok & 15;                // valid tokens in that page
        for (int pgi = first_bad; pgi < kItemPages; ++pgi) {
          uint4 val = make_uint4(0u, 0u, 0u, 0u);
          if (pgi == first_bad && keep > 0) {
            val = lds128(vrow + pgi * kPageBytes);
            uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int nk = min(max(keep - 4 * k, 0), 4);
              w[k] &= nk >= 4 ? 0xffffffffu : ((1u << (8 * nk)) - 1u);
            }
            val = make_uint4(w[0], w[1], w[2], w[3]);
          }
          sts128(vrow + pgi * kPageBytes, val);
        }
      }
      fence_proxy_async();   // P^T and the cleared V bytes are read by the tensor core
      fence_before_sync();   // the S^T loads above are complete (tmem_ld_wait)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull, grp));
      if (wq == 0) stamp(4, i, 2);
      // row sums, needed only by the epilogue of this item
      if constexpr (QR == 8) {
        const float wsum = warp_reduce8<false>(psum, lane);
        if ((lane & 3) == 0) red_sum[par * 32 + ((lane >> 2) & 7) * 4 + wq] = wsum;
      } else {
        const float wsum = warp_reduce4<false>(psum, lane);
        if ((lane & 7) == 0) red_sum[par * 32 + ((lane >> 3) & 3) * 4 + wq] = wsum;
      }
      if (PER_TOKEN && r == 0) v_norm[par] = vnorm;
      return true;
    };

    // `tail`: no softmax of a later item of this group ran in between, so the row sums of item j
    // still need a barrier of their own to be visible to the whole group.
    auto epilogue = [&](int j, const Item& it, bool tail) -> bool {
      const uint32_t gu = (uint32_t)(j / NG);
      const int par = grp * 2 + (int)(gu & 1);
      const float* rs = red_sum + par * 32;
      if (tail) named_barrier_sync(bar_b, 128);
      if (wq == 0) stamp(5, j, 0);
      if (!wait(bar(kBarOFull, par), (gu >> 1) & 1)) return false;
      if (wq == 0) stamp(5, j, 1);
      fence_after_sync();
      uint32_t oraw[2 * QR];
      tmem_ld(tmem_o + lane_field + par * 16, oraw);
      tmem_ld_wait();
      fence_before_sync();  // ordered before this warp's next arrival on the group's P barrier
      if (wq == 0) stamp(7, j, 0);

      const float vfin = PER_TOKEN ? v_norm[par] : v_scale_t;
      const int64_t ws_base = (int64_t)it.seq * p.ws_stride_seq + (int64_t)it.head * p.ws_stride_head +
                              (int64_t)it.part * p.ws_stride_part;
      unsigned short* tmp = reinterpret_cast<unsigned short*>(p.tmp_out) + (int64_t)it.seq * p.tmp_stride_seq +
                            (int64_t)it.head * p.tmp_stride_head + (int64_t)it.part * p.tmp_stride_part + r;
#pragma unroll
      for (int q = 0; q < QR; ++q) {
        if (q < p.eqG) {
          const float4 l4 = *reinterpret_cast<const float4*>(rs + q * 4);
          const float l = (l4.x + l4.y) + (l4.z + l4.w);   // in units of 1/256
          const float f = l > 0.f ? __fdividef(vfin, l) : 0.f;
          const float o = fmaf(__uint_as_float(oraw[QR + q]), 0.0625f, __uint_as_float(oraw[q])) * f;
          tmp[(int64_t)q * p.tmp_stride_row] = (unsigned short)(pack_bf16x2(o, 0.f) & 0xffffu);
          if (r == q) {
            p.max_logits[ws_base + q] = m_fin[par * 8 + q] * kLn2;
            p.exp_sums[ws_base + q] = l * (1.0f / 256.0f);
          }
        }
      }
      if (wq == 0) stamp(5, j, 2);
      return true;
    };

    // group g walks the CTA's items g, g+NG, ...; the epilogue of an item runs after the softmax
    // of the group's next item, by which time its P.V product has long been issued
    ItemCursor cur;
    if (grp < n_local) cur.init(first + grp * stride, NG * stride, p, seq_off);
    Item it_prev{};
    int prev = -1;
    for (int i = grp; i < n_local && !dead; i += NG) {
      const Item it = cur.item(p, seq_off, seq_ctx);
      cur.advance(p, seq_off);
      if (!softmax(i, it)) { fail(); break; }
      if (prev >= 0 && !epilogue(prev, it_prev, false)) { fail(); break; }
      it_prev = it;
      prev = i;
    }
    if (!dead && prev >= 0 && !epilogue(prev, it_prev, true)) fail();
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  fence_before_sync();
  __syncthreads();
  if (warp == kWarpMma) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace tc
}  // namespace pa
