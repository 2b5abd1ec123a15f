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
  int32_t vec_ok;                              // sources, caches and their strides allow 16-byte accesses
  int64_t key_stride_tok, key_stride_head;     // elements
  int64_t value_stride_tok, value_stride_head;
  int64_t kc_stride_block, kc_stride_head;     // elements of the cache dtype
  int64_t vc_stride_block, vc_stride_head;
  int64_t ks_stride_block, ks_stride_head;     // per-token scales, elements
  int32_t* status;
};

// Tokens t .. t+15 of kv head h fill slots off .. off+15 (off a multiple of 16) of block blk.
__device__ __forceinline__ void write_full_run(const CacheWriteParams& p, int t, int h, int64_t blk, int off, int lane) {
  const int bs = p.block_size;
  const int64_t sbase = blk * p.ks_stride_block + (int64_t)h * p.ks_stride_head + off;
  const bool per_token = p.quant_mode == PA_QUANT_PER_TOKEN;

  // ---- keys: lane = (chunk c of 16 head dims, phase ph); it takes tokens ph, ph+4, ph+8, ph+12
  {
    const int c = lane >> 2, ph = lane & 3;
    const int64_t kbase = blk * p.kc_stride_block + (int64_t)h * p.kc_stride_head;
    uint4 ra[4], rb[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const uint8_t* src = p.key + 2 * ((int64_t)(t + 4 * m + ph) * p.key_stride_tok + (int64_t)h * p.key_stride_head + 16 * c);
      ra[m] = *reinterpret_cast<const uint4*>(src);
      rb[m] = *reinterpret_cast<const uint4*>(src + 16);
    }
    float sk = p.quant_mode == PA_QUANT_PER_TENSOR ? *p.k_scale : 1.0f;
#pragma unroll
    for (int m = 0; m < 4; ++m) {
      const uint32_t w[8] = {ra[m].x, ra[m].y, ra[m].z, ra[m].w, rb[m].x, rb[m].y, rb[m].z, rb[m].w};
      float x[16];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[2 * e] = bf16_lo_to_f32(w[e]);
        x[2 * e + 1] = bf16_hi_to_f32(w[e]);
      }
      if (per_token) {
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(x[e]));
#pragma unroll
        for (int o = 4; o <= 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, o));   // over the 8 chunks
        sk = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
        if (c == 0) p.k_scale[sbase + 4 * m + ph] = sk;
      }
      uint4 q;
      q.x = pack_e4m3x4(__fdiv_rn(x[0], sk), __fdiv_rn(x[1], sk), __fdiv_rn(x[2], sk), __fdiv_rn(x[3], sk));
      q.y = pack_e4m3x4(__fdiv_rn(x[4], sk), __fdiv_rn(x[5], sk), __fdiv_rn(x[6], sk), __fdiv_rn(x[7], sk));
      q.z = pack_e4m3x4(__fdiv_rn(x[8], sk), __fdiv_rn(x[9], sk), __fdiv_rn(x[10], sk), __fdiv_rn(x[11], sk));
      q.w = pack_e4m3x4(__fdiv_rn(x[12], sk), __fdiv_rn(x[13], sk), __fdiv_rn(x[14], sk), __fdiv_rn(x[15], sk));
      *reinterpret_cast<uint4*>(p.key_cache + kbase + ((int64_t)c * bs + off + 4 * m + ph) * 16) = q;
    }
  }

  // ---- values: lane owns head dims 4*lane .. 4*lane+3 of all 16 tokens
  const int d0 = 4 * lane;
  const int64_t vbase = blk * p.vc_stride_block + (int64_t)h * p.vc_stride_head;
  uint2 rv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i)
    rv[i] = *reinterpret_cast<const uint2*>(p.value + 2 * ((int64_t)(t + i) * p.value_stride_tok + (int64_t)h * p.value_stride_head + d0));
  float sv = p.quant_mode == PA_QUANT_PER_TENSOR ? *p.v_scale : 1.0f;
  uint32_t qv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float x[4] = {bf16_lo_to_f32(rv[i].x), bf16_hi_to_f32(rv[i].x), bf16_lo_to_f32(rv[i].y), bf16_hi_to_f32(rv[i].y)};
    if (per_token) {
      float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, o));
      sv = fmaxf(__fdiv_rn(amax, 448.0f), 1e-12f);
      if (lane == 0) p.v_scale[sbase + i] = sv;
    }
    qv[i] = pack_e4m3x4(__fdiv_rn(x[0], sv), __fdiv_rn(x[1], sv), __fdiv_rn(x[2], sv), __fdiv_rn(x[3], sv));
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {   // row d0 + e of the block: byte e of the 16 tokens
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = __byte_perm(qv[4 * j], qv[4 * j + 1], 0x0040 + 0x0011 * e);       // tokens 4j, 4j+1
      const uint32_t hi = __byte_perm(qv[4 * j + 2], qv[4 * j + 3], 0x0040 + 0x0011 * e);   // tokens 4j+2, 4j+3
      w[j] = __byte_perm(lo, hi, 0x5410);
    }
    uint8_t* dst = p.v_trans ? p.value_cache + vbase + ((int64_t)(off >> 4) * kD + (d0 + e)) * 16
                             : p.value_cache + vbase + (int64_t)(d0 + e) * bs + off;
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Token-wise write: one warp per (token, kv head); lane owns head dims 4*lane .. 4*lane+3 of the
// key and of the value.  Used for bf16 caches and when 16-byte accesses are not possible.
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

// e4m3 caches: one warp per (window of 16 consecutive token indices, kv head).
//
// A value row of the cache holds one head dim of 16 neighbouring slots in 16 consecutive bytes,
// and a key chunk holds 16 head dims of neighbouring slots in consecutive 16-byte pieces; a token
// written alone stores 128 single value bytes, each into a different sector, and eight half
// sectors of keys.  When the 16 slots of an aligned slot block are written by 16 consecutive
// tokens of the stream in order (a prefill chunk walking a page) that is a full run, and the
// warp whose window holds its first token writes it whole (write_full_run: 16-byte vector stores
// into whole sectors).  The window's other tokens (ragged ends of a chunk, scattered decode-step
// slots) are written one by one, with all their rows requested up front.  Bytes and scales are
// the same either way.
__global__ void __launch_bounds__(128) pa_cache_write_fp8_kernel(const __grid_constant__ CacheWriteParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t windows = ((int64_t)p.T + 15) / 16;
  if (wid >= windows * p.Hkv) return;
  const int64_t g = wid / p.Hkv;
  const int h = (int)(wid - g * p.Hkv);
  const int bs = p.block_size;
  const int d0 = 4 * lane;

  // slots of token indices 16 g - 16 + k, k = 0..63 (lane holds k = lane and k = lane + 32): the
  // window is k = 16..31; a run through a window token begins at most 15 before it and ends at
  // most 15 after it
  const int64_t ia = 16 * g - 16 + lane, ib = ia + 32;
  const int64_t sa = (ia >= 0 && ia < p.T) ? p.slots[ia] : -1;
  const int64_t sb = (ib >= 0 && ib < p.T) ? p.slots[ib] : -1;
  // bit k: token k's slot follows token k - 1's
  const int64_t sa_prev = __shfl_up_sync(kFullMask, sa, 1);
  int64_t sb_prev = __shfl_up_sync(kFullMask, sb, 1);
  const int64_t sa_last = __shfl_sync(kFullMask, sa, 31);
  if (lane == 0) sb_prev = sa_last;
  const uint32_t fa = __ballot_sync(kFullMask, lane > 0 && sa >= 0 && sa_prev >= 0 && sa == sa_prev + 1);
  const uint32_t fb = __ballot_sync(kFullMask, sb >= 0 && sb_prev >= 0 && sb == sb_prev + 1);
  const unsigned long long follows = ((unsigned long long)fb << 32) | fa;

  // lanes 16..31 are the window: is my token inside a full run, and is it the run's first token?
  bool in_full = false;
  if (lane >= 16 && sa >= 0) {
    const int first = lane - (int)(sa & 15);          // k of the token that would hold slot (sa & ~15); >= 1
    in_full = ((follows >> (first + 1)) & 0x7fffull) == 0x7fffull;
  }
  const uint32_t full_mask = __ballot_sync(kFullMask, in_full);
  const uint32_t lead_mask = __ballot_sync(kFullMask, in_full && (sa & 15) == 0);      // at most one bit
  const uint32_t single_mask = __ballot_sync(kFullMask, lane >= 16 && sa >= 0 && !in_full) >> 16;

  if (p.vec_ok && lead_mask != 0) {
    const int lk = __ffs(lead_mask) - 1;
    const int64_t slot0 = __shfl_sync(kFullMask, sa, lk);
    const int64_t blk = slot0 / bs;
    if (blk >= p.num_blocks) {
      if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_BAD_PAGE_ID);
    } else {
      write_full_run(p, (int)(16 * g - 16 + lk), h, blk, (int)(slot0 - blk * bs), lane);
    }
  }
  // tokens written one by one: all of the window without 16-byte accesses, else those outside full runs
  const uint32_t todo = p.vec_ok ? single_mask : (single_mask | (full_mask >> 16));
  if (todo == 0) return;
  uint2 rk[16], rv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if ((todo >> i) & 1u) {
      const int64_t t = 16 * g + i;
      rk[i] = *reinterpret_cast<const uint2*>(p.key + 2 * (t * p.key_stride_tok + (int64_t)h * p.key_stride_head + d0));
      rv[i] = *reinterpret_cast<const uint2*>(p.value + 2 * (t * p.value_stride_tok + (int64_t)h * p.value_stride_head + d0));
    }
  }
  float sk = 1.0f, sv = 1.0f;
  if (p.quant_mode == PA_QUANT_PER_TENSOR) {
    sk = *p.k_scale;
    sv = *p.v_scale;
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (!((todo >> i) & 1u)) continue;
    const int64_t slot = __shfl_sync(kFullMask, sa, 16 + i);
    const int64_t blk = slot / bs;
    const int off = (int)(slot - blk * bs);
    if (blk >= p.num_blocks) {   // a slot outside the pool: report, write nothing
      if (lane == 0 && p.status) atomicOr(p.status, PA_DEV_BAD_PAGE_ID);
      continue;
    }
    const float xk[4] = {bf16_lo_to_f32(rk[i].x), bf16_hi_to_f32(rk[i].x), bf16_lo_to_f32(rk[i].y), bf16_hi_to_f32(rk[i].y)};
    const float xv[4] = {bf16_lo_to_f32(rv[i].x), bf16_hi_to_f32(rv[i].x), bf16_lo_to_f32(rv[i].y), bf16_hi_to_f32(rv[i].y)};
    if (p.quant_mode == PA_QUANT_PER_TOKEN) {
      float ak = fmaxf(fmaxf(fabsf(xk[0]), fabsf(xk[1])), fmaxf(fabsf(xk[2]), fabsf(xk[3])));
      float av = fmaxf(fmaxf(fabsf(xv[0]), fabsf(xv[1])), fmaxf(fabsf(xv[2]), fabsf(xv[3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ak = fmaxf(ak, __shfl_xor_sync(kFullMask, ak, o));
        av = fmaxf(av, __shfl_xor_sync(kFullMask, av, o));
      }
      sk = fmaxf(__fdiv_rn(ak, 448.0f), 1e-12f);
      sv = fmaxf(__fdiv_rn(av, 448.0f), 1e-12f);
      if (lane == 0) {
        const int64_t si = blk * p.ks_stride_block + (int64_t)h * p.ks_stride_head + off;
        p.k_scale[si] = sk;
        p.v_scale[si] = sv;
      }
    }
    const uint32_t qk = pack_e4m3x4(__fdiv_rn(xk[0], sk), __fdiv_rn(xk[1], sk), __fdiv_rn(xk[2], sk), __fdiv_rn(xk[3], sk));
    const uint32_t qv = pack_e4m3x4(__fdiv_rn(xv[0], sv), __fdiv_rn(xv[1], sv), __fdiv_rn(xv[2], sv), __fdiv_rn(xv[3], sv));
    const int64_t kbase = blk * p.kc_stride_block + (int64_t)h * p.kc_stride_head;
    const int64_t vbase = blk * p.vc_stride_block + (int64_t)h * p.vc_stride_head;
    *reinterpret_cast<uint32_t*>(p.key_cache + kbase + ((int64_t)(d0 >> 4) * bs + off) * 16 + (d0 & 15)) = qk;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      uint8_t* dst = p.v_trans ? p.value_cache + vbase + ((int64_t)(off >> 4) * kD + (d0 + e)) * 16 + (off & 15)
                               : p.value_cache + vbase + (int64_t)(d0 + e) * bs + off;
      *dst = (uint8_t)(qv >> (8 * e));
    }
  }
}

}  // namespace pa
