// Split-KV partition kernel, e4m3fn KV cache, 16-token pages.
//
// Computes what paged_attention_decode_v2_gluon_fp8 computes
// (pa_decode_triton_gluon_fp8.py:514-1002 in yanguahe/triton_op): for every
// (sequence, kv head, partition) the running max m, the sum l = sum_j exp(s_j - m) and the
// partial output sum_j exp(s_j - m) v_j / l over the partition's tokens, stored to
// max_logits / exp_sums / tmp_out in the reference's layouts.
//
// Shape of the computation on B200
// --------------------------------
// The op streams every KV byte exactly once and does ~2*eqG flop per byte, so the only
// roofline that matters is HBM.  The kernel is therefore built around keeping a deep, steady
// queue of bulk copies in flight per SM:
//
//  * Persistent grid, one CTA per SM, NW warps per CTA.  A *work item* is one
//    (sequence, kv head, partition); items are dealt to warps round-robin over the whole grid.
//    Every CTA first builds, in shared memory, the prefix sum of partitions per sequence from
//    context_lens, so no host-side knowledge of the lengths and no scratch buffer is needed and
//    ragged batches cost nothing for the partitions that do not exist.
//  * Every warp owns a private ring of `num_stages` stages in shared memory.  One stage is two
//    pages (32 tokens): K page A | K page B | V page A | V page B (| per-token scales).  A page
//    of one head is a single contiguous 2 KB run in both caches ([D/16][16][16] for K,
//    [D][16] for V), so a stage is filled by four cp.async.bulk copies issued by four lanes of
//    the warp itself, completing on the stage's mbarrier.  The warp keeps issuing copies
//    `num_stages` ahead of what it computes, across work-item boundaries; page ids of the next
//    item are prefetched one item ahead so the dependent block-table load never stalls.
//    Because a ring is private to one warp there is no inter-warp synchronisation at all in
//    the steady state; the only waits are on the warp's own copies (bounded).
//  * Math is written as the e4m3 tile mma.sync.m16n8k32 on the fp8 bytes in shared memory, with
//    no dequantisation pass in the source.  sm_100a has no native e4m3 mma.sync, though: the
//    compiler expands each tile into byte->half converts plus f16 tiles, and that convert pipe
//    is what bounds this kernel near 4.2 TB/s (the tcgen05 kernel in pa_partition_tc.cuh, which
//    feeds e4m3 operands to the tensor core from shared memory, serves the 256-token partition
//    size for that reason; this kernel covers the other partition sizes).  The query (bf16) is split into
//    hi + lo/16, two e4m3 numbers per element, exactly (8 significant bits); hi rows live in
//    tile rows 0-7 and lo rows in rows 8-15, so one M=16 tile serves 8 query rows at bf16
//    precision.  The probabilities get the same hi/lo treatment for P.V.  Products are exact
//    and accumulate in fp32; scales (softmax, K, V) are applied in fp32 outside the tiles.
//  * Shared-memory reads are conflict-free 32-bit loads: the tile's N index (token for QK^T,
//    head dim for PV) is mapped onto lanes so that the eight lanes of a group touch eight
//    different 16-byte rows.  For QK^T this needs the two 8-token tiles of a page to take the
//    token sets {0,1,4,5,10,11,14,15} and {2,3,6,7,8,9,12,13}; a lane then owns four
//    consecutive tokens of the page (4t..4t+3), which is exactly the K-slot order P.V wants,
//    so probabilities never move between lanes.
#pragma once

#include <type_traits>

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "../../include/pa_decode_sm100.h"

namespace pa {

constexpr int kPageTokens = 16;               // tokens per page (this kernel)
constexpr int kPageBytes = kPageTokens * kD;  // 2048: one head's K (or V) page, e4m3
constexpr int kStageTokens = 32;              // two pages per stage
constexpr int kStageKV = 4 * kPageBytes;      // K A | K B | V A | V B
constexpr int kStageScales = 4 * kPageTokens * 4;  // k A | k B | v A | v B  (fp32 per token)
constexpr int kQRowBytes = kD * 2;            // bf16 query row

__host__ __device__ constexpr int stage_bytes(bool per_token) {
  return per_token ? kStageKV + kStageScales : kStageKV;
}

struct Item {
  int seq, head, part;
  int ctx;      // context length of the sequence (clamped)
  int tok0;     // first token of the partition
  int ntok;     // tokens of the partition that exist
  int npages;   // pages covering them
  int nstages;  // stages covering them
};

__device__ __forceinline__ Item decode_item(int k, const KernelParams& p, const int* seq_off,
                                            const int* seq_ctx) {
  Item it;
  const int sp = k / p.Hkv;
  it.head = k - sp * p.Hkv;
  int lo = 0, hi = p.S;  // seq_off[lo] <= sp < seq_off[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (seq_off[mid] <= sp) lo = mid; else hi = mid;
  }
  it.seq = lo;
  it.part = sp - seq_off[lo];
  it.ctx = seq_ctx[lo];
  it.tok0 = it.part * p.partition_size;
  it.ntok = min(p.partition_size, it.ctx - it.tok0);
  it.npages = (it.ntok + kPageTokens - 1) / kPageTokens;
  it.nstages = (it.npages + 1) >> 1;
  return it;
}

// Builds, cooperatively over the CTA, seq_off[0..S] (exclusive prefix sum of the number of
// partitions per sequence) and seq_ctx[0..S) (context lengths clamped to what the block table
// can address).  Returns the total number of (sequence, partition) pairs.
// (Run once per CTA: its loops stay rolled and it is not inlined, so that a cold start fetches a
// few hundred bytes of it instead of ten kilobytes of unrolled divisions.)
// A context length as the kernels use it: clamped to what the block table can address and to
// the workspaces' partition extent.  Returns the partition count through `np`.
__device__ __forceinline__ int clamp_context(const KernelParams& p, int c, int& np, bool& too_long) {
  if (c > p.ctx_cap) {
    c = p.ctx_cap;
    too_long = true;
  }
  if (c < 0) c = 0;
  np = (c + p.partition_size - 1) / p.partition_size;
  if (np > p.max_partitions) {  // workspace extent is the hard limit
    np = p.max_partitions;
    c = np * p.partition_size;
    too_long = true;
  }
  return c;
}

// `early`: the caller has not passed its dependency wait yet, so the lengths may still be written
// by the kernel before this one in the stream.  They are then read past the L1 (which must not
// keep a line that may change) and nothing is reported; the caller checks the index against the
// lengths as they are after the wait (partition_index_still_valid) before it relies on it.
__device__ __noinline__ int build_partition_index(const KernelParams& p, int* seq_off,
                                                  int* seq_ctx, int* scan_scratch, bool early = false) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5;
  if (tid == 0) seq_off[0] = 0;
  bool too_long = false;
#pragma unroll 1
  for (int i = tid; i < p.S; i += nthr) {
    int np;
    seq_ctx[i] = clamp_context(p, early ? __ldcg(p.context_lens + i) : p.context_lens[i], np, too_long);
    seq_off[i + 1] = np;
  }
  if (too_long && p.status && !early) atomicOr(p.status, PA_DEV_CTX_TOO_LONG);
  __syncthreads();
  const int chunk = (p.S + nthr - 1) / nthr;
  const int beg = min(tid * chunk, p.S), end = min(beg + chunk, p.S);
  int sum = 0;
#pragma unroll 1
  for (int i = beg; i < end; ++i) sum += seq_off[i + 1];
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(kFullMask, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) scan_scratch[warp] = incl;
  __syncthreads();
  int run = incl - sum;
#pragma unroll 1
  for (int w = 0; w < warp; ++w) run += scan_scratch[w];
#pragma unroll 1
  for (int i = beg; i < end; ++i) {
    run += seq_off[i + 1];
    seq_off[i + 1] = run;
  }
  __syncthreads();
  return seq_off[p.S];
}

// True (for the whole CTA) when the lengths, read now, are the ones an early index was built from.
// Also does the reporting the early build left out.  Contains a block-wide barrier.
__device__ __noinline__ bool partition_index_still_valid(const KernelParams& p, const int* seq_ctx) {
  bool changed = false, too_long = false;
#pragma unroll 1
  for (int i = threadIdx.x; i < p.S; i += blockDim.x) {
    int np;
    if (clamp_context(p, p.context_lens[i], np, too_long) != seq_ctx[i]) changed = true;
  }
  if (too_long && p.status) atomicOr(p.status, PA_DEV_CTX_TOO_LONG);
  return __syncthreads_or(changed) == 0;
}

// MT: 8-row query tiles per warp (eqG <= 8*MT).  PER_TOKEN: per-token-per-head K/V scales.
template <int NW, int MT, bool PER_TOKEN>
__global__ void __launch_bounds__(NW * 32, 1)
pa_partition_fp8_p16_kernel(const __grid_constant__ KernelParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int STAGE = stage_bytes(PER_TOKEN);
  constexpr int QBUF = MT * 8 * kQRowBytes;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2;   // group id: tile row (A/C) or tile column (B)
  const int t = lane & 3;    // thread in group
  const bool sw = (t >> 1) != 0;

  int* scan_scratch = reinterpret_cast<int*>(smem + kMaxWarps * kBarBytesPerWarp);
  int* seq_off = reinterpret_cast<int*>(smem + p.off_seq_offsets);
  int* seq_ctx = reinterpret_cast<int*>(smem + p.off_seq_ctx);
  const uint32_t bars = smem_addr(smem) + warp * kBarBytesPerWarp;  // [num_stages] full + 1 query
  const uint32_t qbar = bars + kMaxStages * 8;
  const uint32_t qbuf = smem_addr(smem + p.off_q) + warp * QBUF;
  const uint32_t ring = smem_addr(smem + p.off_ring) + warp * p.num_stages * STAGE;
  const int NS = p.num_stages;

  if (lane == 0) {
    for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8, 1);
    mbar_init(qbar, 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  const int n_sp = build_partition_index(p, seq_off, seq_ctx, scan_scratch);  // has __syncthreads
  grid_launch_dependents();  // the reduce kernel may become resident; it waits for this grid to finish
  const int n_items = n_sp * p.Hkv;
  const int wtot = gridDim.x * NW;
  const int k_first = blockIdx.x * NW + warp;
  if (k_first >= n_items) return;

  const uint64_t pol_stream = l2_policy_evict_first();
  const uint64_t pol_keep = l2_policy_evict_last();

  // Per-lane shared-memory offsets.  QK^T B operand: lane group g supplies token tok(tau, g)
  // of 8-token tile tau; the quad's lane t supplies bytes 4t..4t+3 of a 16-byte chunk.
  uint32_t koff[2];
#pragma unroll
  for (int tau = 0; tau < 2; ++tau) {
    const int tok = 4 * (g >> 1) + 2 * (tau ^ (g >> 2)) + (g & 1);
    koff[tau] = tok * 16 + 4 * t;
  }
  const uint32_t voff = g * 16 + 4 * t;  // PV B operand: head dim 8i+g, tokens 4t..4t+3

  float k_scale_t = 1.0f, v_scale_t = 1.0f;
  if (!PER_TOKEN && p.kv_quant_mode == PA_QUANT_PER_TENSOR) {
    k_scale_t = __ldg(p.k_scale);
    v_scale_t = __ldg(p.v_scale);
  }

  bool dead = false;  // set when a bounded wait ran out

  // ------------------------------------------------------------------ producer side
  int pk = k_first;  // item the next stage to issue belongs to
  Item pit = decode_item(pk, p, seq_off, seq_ctx);
  int ps = 0;        // stage within pit
  int pslot = 0;     // ring slot of the next stage to issue
  int issued = 0, consumed = 0;

  auto load_page_ids = [&](const Item& it) -> int {
    int id = 0;
    if (lane < it.npages) {
      id = __ldg(p.block_tables + (int64_t)it.seq * p.bt_stride_seq +
                 (int64_t)it.part * p.pages_per_partition + lane);
      if ((unsigned)id >= (unsigned)p.num_blocks) {
        id = 0;
        if (p.status) atomicOr(p.status, PA_DEV_BAD_PAGE_ID);
      }
    }
    return id;
  };
  int ppages = load_page_ids(pit);
  int ppages_next = 0;
  if (pk + wtot < n_items) ppages_next = load_page_ids(decode_item(pk + wtot, p, seq_off, seq_ctx));

  auto issue_stage = [&]() {
    if (pk >= n_items) return;
    const uint32_t bar = bars + pslot * 8;
    const uint32_t dst = ring + pslot * STAGE;
    const int pgA = 2 * ps;
    const bool hasB = (pgA + 1) < pit.npages;
    const int idA = __shfl_sync(kFullMask, ppages, pgA & 31);
    const int idB = __shfl_sync(kFullMask, ppages, (pgA + 1) & 31);
    if (lane == 0)
      mbar_arrive_expect_tx(bar, (hasB ? 2u : 1u) * (PER_TOKEN ? 2 * kPageBytes + 2 * kPageTokens * 4
                                                                 : 2 * kPageBytes));
    __syncwarp();
    const bool second = lane & 1;
    if (!second || hasB) {
      const int64_t id = second ? idB : idA;
      if (lane < 4) {
        const bool is_v = lane >> 1;
        const uint8_t* src = is_v ? p.v + id * p.v_stride_block + (int64_t)pit.head * p.v_stride_head
                                  : p.k + id * p.k_stride_block + (int64_t)pit.head * p.k_stride_head;
        bulk_g2s(dst + (is_v ? 2 * kPageBytes : 0) + (second ? kPageBytes : 0), src, kPageBytes,
                 bar, pol_stream);
      } else if (PER_TOKEN && lane < 8) {
        const bool is_v = (lane - 4) >> 1;
        const float* src = (is_v ? p.v_scale : p.k_scale) + id * p.kvs_stride_block +
                           (int64_t)pit.head * p.kvs_stride_head;
        bulk_g2s(dst + kStageKV + (lane - 4) * (kPageTokens * 4), src, kPageTokens * 4, bar,
                 pol_stream);
      }
    }
    ++issued;
    if (++pslot == NS) pslot = 0;
    if (++ps == pit.nstages) {
      ps = 0;
      pk += wtot;
      if (pk < n_items) {
        pit = decode_item(pk, p, seq_off, seq_ctx);
        ppages = ppages_next;
        if (pk + wtot < n_items)
          ppages_next = load_page_ids(decode_item(pk + wtot, p, seq_off, seq_ctx));
      }
    }
  };

  auto issue_query = [&](const Item& it) {
    if (lane == 0) {
      const uint32_t bytes = p.eqG * kQRowBytes;
      mbar_arrive_expect_tx(qbar, bytes);
      bulk_g2s(qbuf,
               p.q + (int64_t)it.seq * p.q_stride_seq + (int64_t)it.head * p.eqG * p.q_stride_head,
               bytes, qbar, pol_keep);
    }
  };

  {
    issue_query(pit);
    for (int s = 0; s < NS; ++s) issue_stage();
  }

  // ------------------------------------------------------------------ consumer side
  int cslot = 0;
  uint32_t cphase = 0, qphase = 0;

  for (int ck = k_first; ck < n_items && !dead; ck += wtot) {
    const Item it = decode_item(ck, p, seq_off, seq_ctx);

    // ---- query fragments (A operand of QK^T), rows 8*mt+g: hi in tile rows 0-7, lo in 8-15
    uint32_t qf[MT][4][4];
    float row_scale[MT];  // softmax_scale * log2e * k_scale / (query pre-scale)
    int row_lim[MT];      // first token index the row may NOT see
    float row_slope[MT];  // ALiBi slope of the row's query head, base-2 logit domain (0 without ALiBi)
    if (!__all_sync(kFullMask, mbar_wait(qbar, qphase))) {
      dead = true;
      break;
    }
    qphase ^= 1;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r = mt * 8 + g;
      const bool row_ok = r < p.eqG;
      uint2 raw[4][2];
      float amax = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          raw[j][h] = row_ok ? lds64(qbuf + r * kQRowBytes + (32 * j + 16 * h + 4 * t) * 2)
                             : make_uint2(0u, 0u);
          amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf16_lo_to_f32(raw[j][h].x)), fabsf(bf16_hi_to_f32(raw[j][h].x))),
                                   fmaxf(fabsf(bf16_lo_to_f32(raw[j][h].y)), fabsf(bf16_hi_to_f32(raw[j][h].y)))));
        }
      }
      amax = quad_max(amax);
      // Power-of-two pre-scale that puts the row maximum in [128, 256): exact, and both halves
      // of the split then fit e4m3 (max 448).
      float pre = 1.0f, inv_pre = 1.0f;
      const int be = (int)((__float_as_uint(amax) >> 23) & 0xff);
      if (be > 30 && be < 225) {
        pre = __uint_as_float((uint32_t)(254 + 7 - be) << 23);
        inv_pre = __uint_as_float((uint32_t)(be - 7) << 23);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float hi[4], lo[4];
          split_hi_lo(bf16_lo_to_f32(raw[j][h].x) * pre, hi[0], lo[0]);
          split_hi_lo(bf16_hi_to_f32(raw[j][h].x) * pre, hi[1], lo[1]);
          split_hi_lo(bf16_lo_to_f32(raw[j][h].y) * pre, hi[2], lo[2]);
          split_hi_lo(bf16_hi_to_f32(raw[j][h].y) * pre, hi[3], lo[3]);
          qf[mt][j][2 * h + 0] = pack_e4m3x4(hi[0], hi[1], hi[2], hi[3]);
          qf[mt][j][2 * h + 1] = pack_e4m3x4(lo[0], lo[1], lo[2], lo[3]);
        }
      }
      float qs = 1.0f;
      if (p.q_quant_mode == PA_QUANT_PER_TENSOR) qs = __ldg(p.q_scale);
      if (p.q_quant_mode == PA_QUANT_PER_TOKEN && row_ok)
        qs = __ldg(p.q_scale + (int64_t)it.seq * p.q_scale_stride_seq + it.head * p.eqG + r);
      row_scale[mt] = p.softmax_scale * kLog2e * k_scale_t * inv_pre * qs;
      const int trow = row_ok ? r / p.G : 0;
      row_lim[mt] = it.ctx - (p.L - 1 - trow);
      row_slope[mt] = (p.alibi != nullptr && row_ok) ? __ldg(p.alibi + it.head * p.G + r % p.G) * kLog2e : 0.f;
    }
    const bool alibi = p.alibi != nullptr;   // bias slope * (key position - (context - 1)), pa_decode_triton_gluon_fp8.py:905-908
    __syncwarp();
    fence_proxy_async();
    if (ck + wtot < n_items) issue_query(decode_item(ck + wtot, p, seq_off, seq_ctx));

    // ---- running softmax state
    float m_run[MT], l_run[MT];
    float acc[MT][16][4];
    float vmax_run = 0.f;  // per-token V scales: running max of the scales folded into P
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      m_run[mt] = -INFINITY;
      l_run[mt] = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][i][e] = 0.f;
    }

    auto compute_stage = [&](const uint32_t st, const int stok0, auto tail_tag) {
      constexpr bool TAIL = decltype(tail_tag)::value;
      // ---------------- S = Q K^T for 2 pages x 16 tokens; lane keeps tokens 4t..4t+3 of each
      float sv[MT][8];
      float vs[8];
#pragma unroll
      for (int pg = 0; pg < 2; ++pg) {
        float c[MT][2][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int tau = 0; tau < 2; ++tau)
#pragma unroll
            for (int e = 0; e < 4; ++e) c[mt][tau][e] = 0.f;
        const uint32_t kb = st + pg * kPageBytes;
        uint32_t kw[4][2][2];  // all B fragments of the page first, then the tiles
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int tau = 0; tau < 2; ++tau) {
            kw[j][tau][0] = lds32(kb + (2 * j) * 256 + koff[tau]);
            kw[j][tau][1] = lds32(kb + (2 * j + 1) * 256 + koff[tau]);
          }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int tau = 0; tau < 2; ++tau)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) mma_e4m3(c[mt][tau], qf[mt][j], kw[j][tau][0], kw[j][tau][1]);
        float ks[4] = {1.f, 1.f, 1.f, 1.f};
        if (PER_TOKEN) {
          const uint4 kraw = lds128(st + kStageKV + pg * (kPageTokens * 4) + t * 16);
          const uint4 vraw = lds128(st + kStageKV + (2 + pg) * (kPageTokens * 4) + t * 16);
          ks[0] = __uint_as_float(kraw.x); ks[1] = __uint_as_float(kraw.y);
          ks[2] = __uint_as_float(kraw.z); ks[3] = __uint_as_float(kraw.w);
          vs[pg * 4 + 0] = __uint_as_float(vraw.x); vs[pg * 4 + 1] = __uint_as_float(vraw.y);
          vs[pg * 4 + 2] = __uint_as_float(vraw.z); vs[pg * 4 + 3] = __uint_as_float(vraw.w);
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          // natural token order: tokens 4t,4t+1 come from tile (sw ? 1 : 0), 4t+2,4t+3 from the other
          float hi[4], lo[4];
          hi[0] = sw ? c[mt][1][0] : c[mt][0][0];
          hi[1] = sw ? c[mt][1][1] : c[mt][0][1];
          hi[2] = sw ? c[mt][0][0] : c[mt][1][0];
          hi[3] = sw ? c[mt][0][1] : c[mt][1][1];
          lo[0] = sw ? c[mt][1][2] : c[mt][0][2];
          lo[1] = sw ? c[mt][1][3] : c[mt][0][3];
          lo[2] = sw ? c[mt][0][2] : c[mt][1][2];
          lo[3] = sw ? c[mt][0][3] : c[mt][1][3];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float s = fmaf(lo[i], 0.0625f, hi[i]) * row_scale[mt];
            if (PER_TOKEN) s *= ks[i];
            if (alibi) s = fmaf(row_slope[mt], (float)(stok0 + pg * kPageTokens + 4 * t + i - (it.ctx - 1)), s);
            if (TAIL) {
              const int tok = stok0 + pg * kPageTokens + 4 * t + i;
              if (tok >= row_lim[mt]) s = -INFINITY;
            }
            sv[mt][pg * 4 + i] = s;
          }
        }
      }
      if (PER_TOKEN && TAIL) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int tok = stok0 + (i >> 2) * kPageTokens + 4 * t + (i & 3);
          if (tok >= it.ctx) vs[i] = 0.f;
        }
      }

      // ---------------- online softmax; P = exp2(s - m) * 256 split into hi/lo e4m3
      float vfac[8];
      float vbeta = 1.0f;
      if (PER_TOKEN) {
        float vm = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) vm = fmaxf(vm, vs[i]);
        vm = quad_max(vm);
        const float vnew = fmaxf(vmax_run, vm);
        const float vinv = vnew > 0.f ? 1.0f / vnew : 0.f;
        vbeta = vmax_run * vinv;  // 0 on the first stage (accumulators are zero)
        if (vnew == vmax_run) vbeta = 1.0f;
        vmax_run = vnew;
#pragma unroll
        for (int i = 0; i < 8; ++i) vfac[i] = vs[i] * vinv;
      }
      uint32_t pa[MT][4];
      float alpha[MT];
      bool rescale = PER_TOKEN && (vbeta != 1.0f);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float mx = sv[mt][0];
#pragma unroll
        for (int i = 1; i < 8; ++i) mx = fmaxf(mx, sv[mt][i]);
        mx = quad_max(mx);
        const float m_new = fmaxf(m_run[mt], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[mt] = ex2(m_run[mt] - m_use);
        if (m_new == m_run[mt]) alpha[mt] = 1.0f;  // also covers -inf == -inf
        m_run[mt] = m_new;
        rescale = rescale || (alpha[mt] != 1.0f);
        float psum = 0.f;
        float hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float pv = ex2(sv[mt][i] - m_use + 8.0f);
          psum += pv;
          if (PER_TOKEN) pv *= vfac[i];
          split_hi_lo(pv, hi[i], lo[i]);
        }
        l_run[mt] = l_run[mt] * alpha[mt] + psum;
        pa[mt][0] = pack_e4m3x4(hi[0], hi[1], hi[2], hi[3]);  // page A, tile rows 0-7 (hi)
        pa[mt][1] = pack_e4m3x4(lo[0], lo[1], lo[2], lo[3]);  // page A, tile rows 8-15 (lo)
        pa[mt][2] = pack_e4m3x4(hi[4], hi[5], hi[6], hi[7]);  // page B
        pa[mt][3] = pack_e4m3x4(lo[4], lo[5], lo[6], lo[7]);
      }
      if (__any_sync(kFullMask, rescale)) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const float f = alpha[mt] * vbeta;
#pragma unroll
          for (int i = 0; i < 16; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[mt][i][e] *= f;
        }
      }

      // ---------------- O += P V ; B operand = V[d = 8i+g][tokens 4t..4t+3] of page A / page B
      uint32_t maskA = 0xffffffffu, maskB = 0xffffffffu;
      if (TAIL) {
        // bytes of tokens >= ctx may hold anything (NaN patterns included): zero them
        const int nA = min(max(it.ctx - (stok0 + 4 * t), 0), 4);
        const int nB = min(max(it.ctx - (stok0 + kPageTokens + 4 * t), 0), 4);
        maskA = nA >= 4 ? 0xffffffffu : ((1u << (8 * nA)) - 1u);
        maskB = nB >= 4 ? 0xffffffffu : ((1u << (8 * nB)) - 1u);
      }
      const uint32_t vb = st + 2 * kPageBytes + voff;
#pragma unroll
      for (int i0 = 0; i0 < 16; i0 += 4) {
        uint32_t vw[4][2];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          vw[ii][0] = lds32(vb + (i0 + ii) * 128);
          vw[ii][1] = lds32(vb + kPageBytes + (i0 + ii) * 128);
          if (TAIL) {
            vw[ii][0] &= maskA;
            vw[ii][1] &= maskB;
          }
        }
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_e4m3(acc[mt][i0 + ii], pa[mt], vw[ii][0], vw[ii][1]);
      }
    };

    // ---- stream the item's stages
    const int full_lim = it.ctx - (p.L - 1);  // tokens below this are visible to every row
    for (int s = 0; s < it.nstages; ++s) {
      if (!__all_sync(kFullMask, mbar_wait(bars + cslot * 8, cphase))) {
        dead = true;
        break;
      }
      const uint32_t st = ring + cslot * STAGE;
      const int stok0 = it.tok0 + s * kStageTokens;
      if (stok0 + kStageTokens > full_lim)
        compute_stage(st, stok0, std::true_type{});
      else
        compute_stage(st, stok0, std::false_type{});
      __syncwarp();
      fence_proxy_async();
      ++consumed;
      if (++cslot == NS) {
        cslot = 0;
        cphase ^= 1;
      }
      issue_stage();  // refill the slot just drained with the stage NS ahead
    }
    if (dead) break;

    // ---- store the partition's (m, l, o)
    const int64_t ws_base = (int64_t)it.seq * p.ws_stride_seq + (int64_t)it.head * p.ws_stride_head +
                            (int64_t)it.part * p.ws_stride_part;
    const int64_t tmp_base = (int64_t)it.seq * p.tmp_stride_seq + (int64_t)it.head * p.tmp_stride_head +
                             (int64_t)it.part * p.tmp_stride_part;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r = mt * 8 + g;
      const float l = quad_sum(l_run[mt]);
      if (r < p.eqG) {
        const float vfin = PER_TOKEN ? vmax_run : v_scale_t;
        const float f = l > 0.f ? vfin / l : 0.f;
        if (t == 0) {
          p.max_logits[ws_base + r] = m_run[mt] * kLn2;
          p.exp_sums[ws_base + r] = l * (1.0f / 256.0f);
        }
        uint32_t* orow = reinterpret_cast<uint32_t*>(p.tmp_out) +
                         ((tmp_base + (int64_t)r * p.tmp_stride_row) >> 1);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float o0 = fmaf(acc[mt][i][2], 0.0625f, acc[mt][i][0]) * f;
          const float o1 = fmaf(acc[mt][i][3], 0.0625f, acc[mt][i][1]) * f;
          orow[(8 * i + 2 * t) >> 1] = pack_bf16x2(o0, o1);
        }
      }
    }
  }

  if (dead) {
    if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_WAIT_TIMEOUT);
    // Copies already issued may still land in this CTA's shared memory: give each one more
    // bounded wait before the CTA retires.
    while (consumed < issued) {
      mbar_wait(bars + cslot * 8, cphase);
      ++consumed;
      if (++cslot == NS) {
        cslot = 0;
        cphase ^= 1;
      }
    }
  }
}

}  // namespace pa
