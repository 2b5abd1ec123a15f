// KV-cache write side: quantise new key / value tokens and scatter them into the paged layouts
// the decode kernels read.
//
// The reference builds its caches offline with torch permutes (test_pa_mtp.py:109-172 for the
// layouts, :294-369 quantize_kv_cache_symmetric for per-token e4m3 quantisation); a serving
// loop does the same per new token.  Layouts written here:
//   keys   [NB, Hkv, D/x, bs, x]   (x = 16 for e4m3fn, 8 for bf16)
//   values [NB, Hkv, D, bs]   or   [NB, Hkv, bs/16, D, 16] (transposed, e4m3fn only)
//   per-token scales [NB, Hkv, bs, 1] fp32: scale = max(amax(vector) / 448, 1e-12), q = x / scale
// Quantisation uses IEEE division and round-to-nearest-even e4m3fn conversion, so the bytes are
// the ones torch's `(x.float() / scale).to(torch.float8_e4m3fn)` gives for in-range values.
#pragma once

#include "../../include/pa_decode_sm100.h"
#include "pa_common.cuh"
#include "pa_params.cuh"

namespace pa {

struct CacheWriteParams {
  const uint8_t* key;          // new tokens [T, Hkv, D] bf16
  const uint8_t* value;
  const int64_t* slots;        // [T]: block * block_size + offset; negative = skip the token
  uint8_t* key_cache;
  uint8_t* value_cache;
  float* k_scale;              // per-token: written [NB, Hkv, bs]; per-tensor: read [1]; else null
  float* v_scale;
  int32_t T, Hkv, block_size, num_blocks;
  int32_t kv_is_fp8, quant_mode, v_trans;      // quant_mode: PaQuantMode
  int64_t key_stride_tok, key_stride_head;     // elements
  int64_t value_stride_tok, value_stride_head;
  int64_t kc_stride_block, kc_stride_head;     // elements of the cache dtype
  int64_t vc_stride_block, vc_stride_head;
  int64_t ks_stride_block, ks_stride_head;     // per-token scales, elements
  int32_t* status;
};

// One warp per (token, kv head); lane owns head dims 4*lane .. 4*lane+3 of the key and of the value.
__global__ void __launch_bounds__(128) pa_cache_write_kernel(const __grid_constant__ CacheWriteParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t pair = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (pair >= (int64_t)p.T * p.Hkv) return;
  const int t = (int)(pair / p.Hkv), h = (int)(pair % p.Hkv);
  const int64_t slot = p.slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / p.block_size;
  const int off = (int)(slot - blk * p.block_size);
  if (blk >= p.num_blocks) {   // a slot outside the pool: report, write nothing
    if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_BAD_PAGE_ID);
    return;
  }
  const int bs = p.block_size;
  const int d0 = 4 * lane;

#pragma unroll
  for (int kv = 0; kv < 2; ++kv) {
    const bool is_v = kv == 1;
    const uint8_t* src = (is_v ? p.value : p.key) +
                         2 * ((int64_t)t * (is_v ? p.value_stride_tok : p.key_stride_tok) +
                              (int64_t)h * (is_v ? p.value_stride_head : p.key_stride_head) + d0);
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    float x[4] = {bf16_lo_to_f32(raw.x), bf16_hi_to_f32(raw.x), bf16_lo_to_f32(raw.y), bf16_hi_to_f32(raw.y)};
    uint8_t* cache = is_v ? p.value_cache : p.key_cache;
    const int64_t base = blk * (is_v ? p.vc_stride_block : p.kc_stride_block) + (int64_t)h * (is_v ? p.vc_stride_head : p.kc_stride_head);

    if (!p.kv_is_fp8) {        // bf16 cache: the same bits, other places
      if (!is_v) {             // [D/8][bs][8]: this lane's 4 dims are half of one 16-byte run
        const int64_t e = base + ((int64_t)(d0 >> 3) * bs + off) * 8 + (d0 & 7);
        *reinterpret_cast<uint2*>(cache + 2 * e) = raw;
      } else {                 // [D][bs]
        const unsigned short w[4] = {(unsigned short)(raw.x & 0xffffu), (unsigned short)(raw.x >> 16),
                                     (unsigned short)(raw.y & 0xffffu), (unsigned short)(raw.y >> 16)};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          *reinterpret_cast<unsigned short*>(cache + 2 * (base + (int64_t)(d0 + e) * bs + off)) = w[e];
      }
      continue;
    }

    float scale = 1.0f;
    if (p.quant_mode == PA_QUANT_PER_TOKEN) {
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, o));
      scale = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
      if (lane == 0) {
        float* dst = is_v ? p.v_scale : p.k_scale;
        dst[blk * p.ks_stride_block + (int64_t)h * p.ks_stride_head + off] = scale;
      }
    } else if (p.quant_mode == PA_QUANT_PER_TENSOR) {
      scale = *(is_v ? p.v_scale : p.k_scale);
    }
    const uint32_t q = pack_e4m3x4(__fdiv_rn(x[0], scale), __fdiv_rn(x[1], scale), __fdiv_rn(x[2], scale),
                                   __fdiv_rn(x[3], scale));
    if (!is_v) {               // [D/16][bs][16]: 4 consecutive bytes of one 16-byte run
      *reinterpret_cast<uint32_t*>(cache + base + ((int64_t)(d0 >> 4) * bs + off) * 16 + (d0 & 15)) = q;
    } else if (!p.v_trans) {   // [D][bs]: one byte per head dim, bs apart
#pragma unroll
      for (int e = 0; e < 4; ++e) cache[base + (int64_t)(d0 + e) * bs + off] = (uint8_t)(q >> (8 * e));
    } else {                   // [bs/16][D][16]
#pragma unroll
      for (int e = 0; e < 4; ++e)
        cache[base + ((int64_t)(off >> 4) * kD + (d0 + e)) * 16 + (off & 15)] = (uint8_t)(q >> (8 * e));
    }
  }
}

}  // namespace pa
