// Split-KV partition kernel for bf16 KV caches (16-token pages).
//
// Semantics of the reference's bf16 path (pa_decode_gluon.py:47-460 / pa_decode_triton.py:26-224 in
// yanguahe/triton_op, driven by pa_decode_gluon.py:655-756): key cache [NB, Hkv, D/8, bs, 8],
// value cache [NB, Hkv, D, bs], optional per-tensor k / v scales, one query token per sequence
// (the causal MTP rule is honoured too).  Outputs as in the fp8 kernels: per partition
// m = max_j s_j, l = sum_j exp(s_j - m), o = sum_j exp(s_j - m) v_j / l.
//
// bf16 x bf16 -> f32 is a native tensor-core tile (m16n8k16), so this kernel stays at register
// level: every warp owns a private ring of one-page stages (K 4 KB | V 4 KB) filled by two bulk
// copies per page, and runs QK^T, the online softmax and P.V from shared memory with
// conflict-free (K) / two-way (V) 32-bit loads.  Up to 16 query rows form the M = 16 tile.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "pa_partition_fp8.cuh"  // Item, decode_item, build_partition_index
#include "../../include/pa_decode_sm100.h"

namespace pa {

constexpr int kBf16PageBytes = kPageTokens * kD * 2;   // 4096: one head's K (or V) page
constexpr int kBf16Stage = 2 * kBf16PageBytes;         // K page | V page
constexpr int kBf16QBuf = 16 * kQRowBytes;             // 16 query rows, bf16

template <int NW>
__global__ void __launch_bounds__(NW * 32, 1)
pa_partition_bf16_p16_kernel(const __grid_constant__ KernelParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int g = lane >> 2;   // group id: tile row (A/C) or tile column (B)
  const int t = lane & 3;    // thread in group
  const int sw = t >> 1;

  int* scan_scratch = reinterpret_cast<int*>(smem + kMaxWarps * kBarBytesPerWarp);
  int* seq_off = reinterpret_cast<int*>(smem + p.off_seq_offsets);
  int* seq_ctx = reinterpret_cast<int*>(smem + p.off_seq_ctx);
  const uint32_t bars = smem_addr(smem) + warp * kBarBytesPerWarp;
  const uint32_t qbar = bars + kMaxStages * 8;
  const uint32_t qbuf = smem_addr(smem + p.off_q) + warp * kBf16QBuf;
  const uint32_t ring = smem_addr(smem + p.off_ring) + warp * p.num_stages * kBf16Stage;
  const int NS = p.num_stages;

  if (lane == 0) {
    for (int s = 0; s < NS; ++s) mbar_init(bars + s * 8, 1);
    mbar_init(qbar, 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  const int n_sp = build_partition_index(p, seq_off, seq_ctx, scan_scratch);  // has __syncthreads
  grid_launch_dependents();
  const int n_items = n_sp * p.Hkv;
  const int wtot = gridDim.x * NW;
  const int k_first = blockIdx.x * NW + warp;
  if (k_first >= n_items) return;

  const uint64_t pol_stream = l2_policy_evict_first();
  const uint64_t pol_keep = l2_policy_evict_last();

  // The two 8-token tiles of a page take the token sets {0,1,4,5,10,11,14,15} and
  // {2,3,6,7,8,9,12,13}: lane group g supplies token tok(tau, g) to QK^T (conflict-free loads of
  // the [chunk][token][16 B] page) and thread t then owns tokens tok(tau, 2t), tok(tau, 2t) + 1.
  uint32_t koff[2], voff[2];
  int mytok[2];
#pragma unroll
  for (int tau = 0; tau < 2; ++tau) {
    const int tok = 4 * (g >> 1) + 2 * (tau ^ (g >> 2)) + (g & 1);
    koff[tau] = tok * 16 + 4 * t;
    mytok[tau] = 4 * t + 2 * (tau ^ sw);           // first of this thread's two tokens in tile tau
    voff[tau] = g * 32 + mytok[tau] * 2;           // V row = head dim 8i+g, 16 tokens x 2 B
  }
  float k_scale_t = 1.0f, v_scale_t = 1.0f;
  if (p.kv_quant_mode == PA_QUANT_PER_TENSOR) {
    k_scale_t = __ldg(p.k_scale);
    v_scale_t = __ldg(p.v_scale);
  }
  const float row_scale = p.softmax_scale * kLog2e * k_scale_t;
  bool dead = false;

  // ------------------------------------------------------------------ producer side
  int pk = k_first;
  Item pit = decode_item(pk, p, seq_off, seq_ctx);
  int ps = 0, pslot = 0, issued = 0, consumed = 0;
  auto load_page_ids = [&](const Item& it) -> int {
    int id = 0;
    if (lane < it.npages) {
      id = __ldg(p.block_tables + (int64_t)it.seq * p.bt_stride_seq + (int64_t)it.part * p.pages_per_partition + lane);
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
    const uint32_t dst = ring + pslot * kBf16Stage;
    const int64_t id = __shfl_sync(kFullMask, ppages, ps & 31);
    if (lane == 0) mbar_arrive_expect_tx(bar, kBf16Stage);
    __syncwarp();
    if (lane < 2) {
      const uint8_t* src = lane ? p.v + id * p.v_stride_block + (int64_t)pit.head * p.v_stride_head
                                : p.k + id * p.k_stride_block + (int64_t)pit.head * p.k_stride_head;
      bulk_g2s(dst + lane * kBf16PageBytes, src, kBf16PageBytes, bar, pol_stream);
    }
    ++issued;
    if (++pslot == NS) pslot = 0;
    if (++ps == pit.npages) {
      ps = 0;
      pk += wtot;
      if (pk < n_items) {
        pit = decode_item(pk, p, seq_off, seq_ctx);
        ppages = ppages_next;
        if (pk + wtot < n_items) ppages_next = load_page_ids(decode_item(pk + wtot, p, seq_off, seq_ctx));
      }
    }
  };
  auto issue_query = [&](const Item& it) {
    if (lane == 0) {
      const uint32_t bytes = p.eqG * kQRowBytes;
      mbar_arrive_expect_tx(qbar, bytes);
      bulk_g2s(qbuf, p.q + (int64_t)it.seq * p.q_stride_seq + (int64_t)it.head * p.eqG * p.q_stride_head, bytes,
               qbar, pol_keep);
    }
  };
  issue_query(pit);
  for (int s = 0; s < NS; ++s) issue_stage();

  // ------------------------------------------------------------------ consumer side
  int cslot = 0;
  uint32_t cphase = 0, qphase = 0;
  for (int ck = k_first; ck < n_items && !dead; ck += wtot) {
    const Item it = decode_item(ck, p, seq_off, seq_ctx);
    if (!__all_sync(kFullMask, mbar_wait(qbar, qphase))) { dead = true; break; }
    qphase ^= 1;
    // query fragments: tile rows g and g+8 are query rows g and g+8, K index = head dim
    uint32_t qf[8][4];
    const bool ok0 = g < p.eqG, ok1 = (g + 8) < p.eqG;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t c = (16 * j + 2 * t) * 2;
      qf[j][0] = ok0 ? lds32(qbuf + g * kQRowBytes + c) : 0u;
      qf[j][1] = ok1 ? lds32(qbuf + (g + 8) * kQRowBytes + c) : 0u;
      qf[j][2] = ok0 ? lds32(qbuf + g * kQRowBytes + c + 16) : 0u;
      qf[j][3] = ok1 ? lds32(qbuf + (g + 8) * kQRowBytes + c + 16) : 0u;
    }
    int lim[2];  // first token the row may not see
    lim[0] = it.ctx - (p.L - 1 - (ok0 ? g / p.G : 0));
    lim[1] = it.ctx - (p.L - 1 - (ok1 ? (g + 8) / p.G : 0));
    // ALiBi (pa_decode_triton.py:92-99, 148-151): slope[query head] * (key position - (context - 1)) on
    // the scaled scores; here in the base-2 logit domain
    const bool alibi = p.alibi != nullptr;
    float slope[2] = {0.f, 0.f};
    if (alibi) {
      if (ok0) slope[0] = __ldg(p.alibi + it.head * p.G + g % p.G) * kLog2e;
      if (ok1) slope[1] = __ldg(p.alibi + it.head * p.G + (g + 8) % p.G) * kLog2e;
    }
    __syncwarp();
    fence_proxy_async();
    if (ck + wtot < n_items) issue_query(decode_item(ck + wtot, p, seq_off, seq_ctx));

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    const int full_lim = it.ctx - (p.L - 1);  // tokens below this are visible to every row
    for (int s = 0; s < it.npages; ++s) {
      if (!__all_sync(kFullMask, mbar_wait(bars + cslot * 8, cphase))) { dead = true; break; }
      const uint32_t st = ring + cslot * kBf16Stage;
      const int tok0 = it.tok0 + s * kPageTokens;
      const bool tail = tok0 + kPageTokens > full_lim;
      // ---- S = Q K^T: two 8-token tiles, rows g (c[.][0..1]) and g+8 (c[.][2..3])
      float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int tau = 0; tau < 2; ++tau) {
          const uint32_t b0 = lds32(st + (2 * j) * 256 + koff[tau]);
          const uint32_t b1 = lds32(st + (2 * j + 1) * 256 + koff[tau]);
          mma_bf16(c[tau], qf[j], b0, b1);
        }
      }
      float sv[2][4];  // [row half][tile * 2 + e]
#pragma unroll
      for (int tau = 0; tau < 2; ++tau)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = tok0 + mytok[tau] + e;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v = c[tau][2 * h + e] * row_scale;
            if (alibi) v = fmaf(slope[h], (float)(tok - (it.ctx - 1)), v);
            if (tail && tok >= lim[h]) v = -INFINITY;
            sv[h][tau * 2 + e] = v;
          }
        }
      // ---- online softmax for the two rows
      uint32_t pa[4];
      float alpha[2];
      bool rescale = false;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float mx = fmaxf(fmaxf(sv[h][0], sv[h][1]), fmaxf(sv[h][2], sv[h][3]));
        mx = quad_max(mx);
        const float m_new = fmaxf(m_run[h], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[h] = (m_new == m_run[h]) ? 1.0f : ex2(m_run[h] - m_use);
        m_run[h] = m_new;
        rescale = rescale || (alpha[h] != 1.0f);
        float pv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) pv[e] = ex2(sv[h][e] - m_use);
        l_run[h] = l_run[h] * alpha[h] + (pv[0] + pv[1]) + (pv[2] + pv[3]);
        pa[h] = pack_bf16x2(pv[0], pv[1]);      // K slots 2t, 2t+1   <-> this thread's tile-0 tokens
        pa[2 + h] = pack_bf16x2(pv[2], pv[3]);  // K slots 8+2t, 9+2t <-> tile-1 tokens
      }
      if (__any_sync(kFullMask, rescale)) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          acc[i][0] *= alpha[0];
          acc[i][1] *= alpha[0];
          acc[i][2] *= alpha[1];
          acc[i][3] *= alpha[1];
        }
      }
      // ---- O += P V: B operand = V[d = 8i+g][this thread's tokens of tile 0 | tile 1]
      uint32_t vmask[2] = {0xffffffffu, 0xffffffffu};
      if (tail) {  // tokens past the context may hold anything (NaN patterns included)
#pragma unroll
        for (int tau = 0; tau < 2; ++tau) {
          const int n = min(max(it.ctx - (tok0 + mytok[tau]), 0), 2);
          vmask[tau] = n >= 2 ? 0xffffffffu : (n == 1 ? 0x0000ffffu : 0u);
        }
      }
      const uint32_t vb = st + kBf16PageBytes;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t b0 = lds32(vb + i * 256 + voff[0]) & vmask[0];
        const uint32_t b1 = lds32(vb + i * 256 + voff[1]) & vmask[1];
        mma_bf16(acc[i], pa, b0, b1);
      }
      __syncwarp();
      fence_proxy_async();
      ++consumed;
      if (++cslot == NS) { cslot = 0; cphase ^= 1; }
      issue_stage();
    }
    if (dead) break;

    // ---- store the partition's (m, l, o) for rows g and g+8
    const int64_t ws_base = (int64_t)it.seq * p.ws_stride_seq + (int64_t)it.head * p.ws_stride_head +
                            (int64_t)it.part * p.ws_stride_part;
    const int64_t tmp_base = (int64_t)it.seq * p.tmp_stride_seq + (int64_t)it.head * p.tmp_stride_head +
                             (int64_t)it.part * p.tmp_stride_part;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = g + 8 * h;
      const float l = quad_sum(l_run[h]);
      if (r < p.eqG) {
        const float f = l > 0.f ? v_scale_t / l : 0.f;
        if (t == 0) {
          p.max_logits[ws_base + r] = m_run[h] * kLn2;
          p.exp_sums[ws_base + r] = l;
        }
        uint32_t* orow = reinterpret_cast<uint32_t*>(p.tmp_out) + ((tmp_base + (int64_t)r * p.tmp_stride_row) >> 1);
#pragma unroll
        for (int i = 0; i < 16; ++i)
          orow[(8 * i + 2 * t) >> 1] = pack_bf16x2(acc[i][2 * h] * f, acc[i][2 * h + 1] * f);
      }
    }
  }

  if (dead) {
    if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_WAIT_TIMEOUT);
    while (consumed < issued) {  // copies already issued may still land: give each a bounded wait
      mbar_wait(bars + cslot * 8, cphase);
      ++consumed;
      if (++cslot == NS) { cslot = 0; cphase ^= 1; }
    }
  }
}

}  // namespace pa
