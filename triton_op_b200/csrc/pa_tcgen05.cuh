// tcgen05 (5th-generation tensor core) and tensor-memory wrappers for sm_100a.
//
// Operands of tcgen05.mma live in shared memory and are described by 64-bit matrix
// descriptors; the accumulator lives in tensor memory (TMEM), 128 lanes x 512 32-bit columns
// per SM.  Everything here is the single-CTA form (cta_group::1); no cluster multicast is used.
#pragma once

#include <stdint.h>

#include "pa_common.cuh"

namespace pa {
namespace tc {

// ---- shared-memory matrix descriptor, no swizzle, K-major ------------------------------------
// The operand tile is (rows x 2) units of 16 bytes: rows are 16 bytes apart inside a group of 8
// (a 128-byte "core matrix"), groups of 8 rows are `sbo` bytes apart, and the two 16-byte units
// along K are `lbo` bytes apart.  All three of address, lbo and sbo are multiples of 16.
//   bits [0,14)  start address >> 4        bits [16,30) lbo >> 4       bits [32,46) sbo >> 4
//   bits [46,48) descriptor version (1 on sm_100)                      bits [61,64) swizzle (0 = none)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// Swizzled K-major operand (what a tiled TMA copy with CU_TENSOR_MAP_SWIZZLE_{64,128}B writes):
// rows are `span` bytes apart (span = 64 or 128), the 16-byte chunks of a row are XOR-ed with
// the row number inside each group of 8 rows, groups are 8 * span bytes apart.  The tile base
// is aligned to 8 * span.  layout code: 4 = 64-byte swizzle, 2 = 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_swizzled(uint32_t addr, uint32_t span) {
  const uint64_t layout = span == 128 ? 2ull : 4ull;
  return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(((8 * span) >> 4) & 0x3fffu) << 32) |
         (1ull << 46) | (layout << 61);
}

// Tiled TMA load of one 4-D box into this CTA's shared memory (no multicast), completion
// counted on `bar`.  c0 is the innermost coordinate and must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int c0, int c1, int c2, int c3,
                                            uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
      : "memory");
}

// ---- instruction descriptor (upper 32 bits of the "idesc" operand) ----------------------------
//   bits [4,6)  accumulator format (1 = f32)      bits [7,10) A format     bits [10,13) B format
//   bit 15 / 16 A / B major (0 = K-major)          bits [17,23) N >> 3      bits [24,29) M >> 4
// kind::f8f6f4 formats: 0 = e4m3.  kind::f16 formats: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t idesc_f32acc(int m, int n, int a_fmt, int b_fmt, bool b_mn_major = false) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], e4m3 operands, K = 32 per instruction.  One thread issues.
__device__ __forceinline__ void mma_f8_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u)  // no output lane disabled
      : "memory");
}

// bf16 / f16 operands, K = 16 per instruction.
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u)  // no output lane disabled
      : "memory");
}

// The mbarrier gets one arrival when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// True in exactly one lane of a converged warp.  The tensor-core instructions take their
// operands from warp-uniform registers, so the issuing warp keeps its control flow uniform,
// computes descriptors in every lane and predicates only the instruction itself on this.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Whole-warp, converged.  `columns` is a power of two >= 32; the base address is written to
// shared memory at `dst`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

// Warp-wide load of 16 consecutive 32-bit columns of this warp's 32 TMEM lanes: thread i gets
// lane (lane field of taddr) + i, register j gets column (column field) + j.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
      : "r"(taddr)
      : "memory");
}
// Eight registers of every lane back into eight tensor-memory columns (this warp's 32 lanes).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
               "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
               "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7]))
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[16]) { tmem_ld16(taddr, v); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[8]) { tmem_ld8(taddr, v); }
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// A counter in shared memory that one set of warps bumps (release) and another polls (acquire):
// what the bumping thread wrote, or saw written through a warp barrier, before the bump is
// visible to the thread that reads the bumped value.
__device__ __forceinline__ void red_release_cta_add(uint32_t addr, uint32_t v) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_cta_shared(uint32_t addr, uint32_t v) {
  asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// A counter in global memory that other CTAs bump after a fence: read past the L1.
__device__ __forceinline__ int ld_relaxed_gpu(const int32_t* ptr) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_cta_shared(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void sts8(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t lo, uint32_t hi) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(lo), "r"(hi) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace tc
}  // namespace pa
