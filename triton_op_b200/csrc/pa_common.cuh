// Device-side helpers shared by the paged-attention decode kernels (sm_100a).
//
// Thin wrappers over the PTX the kernels are built from: mbarrier + cp.async.bulk (the
// non-tensor form of TMA: one thread moves a contiguous run of bytes global -> shared and the
// hardware signals an mbarrier with the byte count), the e4m3 / bf16 mma.sync tiles, and the
// packed fp8 converts.  No multicast form of any copy is used anywhere in this library.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pa {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned kFullMask = 0xffffffffu;

// Upper bound on polls of one mbarrier phase.  A poll is a try_wait with a suspend-time hint:
// the hardware parks the thread until the phase completes or the hint runs out, so a waiting
// warp takes few issue slots from the warps that compute (back-to-back polls of the four
// waiting roles were more than half of all instructions the kernel issued), and wakes as soon
// as the phase completes.  After kSpinPolls polls the waiter also sleeps between polls.  The
// limit is of the order of seconds if every poll runs its full hint and tens of milliseconds
// if the hint is ignored, while a healthy copy completes in microseconds.  When the limit runs
// out the warp records PA_DEV_WAIT_TIMEOUT and stops issuing work, so a lost copy can never
// spin a GPU forever.
constexpr uint32_t kSpinPolls = 1u << 15;
constexpr uint32_t kWaitPollLimit = 1u << 20;
constexpr uint32_t kPollSuspendNs = 4096;

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// start while its predecessor still runs; it must call grid_dependency_wait() before touching
// the predecessor's results.  The predecessor calls grid_launch_dependents() once it no longer
// minds sharing the SMs.
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// async-proxy (bulk copy) accesses to the same bytes.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// More bytes to wait for in the barrier's current phase, without arriving.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return done != 0;
}

// Bounded wait; false when the limit ran out.  The polling loop is one shared out-of-line
// function: inlined at every wait site (and unrolled) it made up almost half of the kernel's
// code, and the kernels' hot loops should stay inside the instruction cache.  (A tighter loop,
// four instructions a poll in one asm block, measured slower: the waiting roles then poll more
// often and take more issue slots from the warps that compute.)
__device__ __noinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity) {
#pragma unroll 1
  for (uint32_t it = 0; it < kWaitPollLimit; ++it) {
    if (mbar_try_wait_hint(bar, parity, kPollSuspendNs)) return true;
    if (it > kSpinPolls) __nanosleep(200);
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_poll(bar, parity);
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// Contiguous global -> shared copy of `bytes` (multiple of 16; both addresses 16-byte
// aligned), completion counted on `bar`.  The destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// D(16x8,f32) += A(16x32,e4m3,row) * B(32x8,e4m3,col).  Register/element map (PTX ISA,
// m16n8k32 8-bit): with g = lane/4, t = lane%4 and byte i of a register = element i,
//   a[0]: row g   k 4t+i      a[1]: row g+8 k 4t+i      a[2]: row g   k 16+4t+i   a[3]: row g+8 k 16+4t+i
//   b0  : k 4t+i  col g       b1  : k 16+4t+i col g
//   c[0],c[1]: row g cols 2t,2t+1                       c[2],c[3]: row g+8 cols 2t,2t+1
__device__ __forceinline__ void mma_e4m3(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col).  With g = lane/4, t = lane%4 and the
// low half of a register = the lower index,
//   a[0]: row g   k 2t,2t+1   a[1]: row g+8 k 2t,2t+1   a[2]: row g   k 8+2t,9+2t   a[3]: row g+8 k 8+2t,9+2t
//   b0  : k 2t,2t+1 col g     b1  : k 8+2t,9+2t col g
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four fp32 -> four e4m3 (round to nearest even, saturating), x0 in the lowest byte.
__device__ __forceinline__ uint32_t pack_e4m3x4(float x0, float x1, float x2, float x3) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
      "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
      "mov.b32 %0, {lo, hi};\n\t}"
      : "=r"(r)
      : "f"(x0), "f"(x1), "f"(x2), "f"(x3));
  return r;
}

// Two fp32 -> packed bf16x2 (round to nearest even), x0 in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float x0, float x1) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(x0), "f"(x1));
  return r;
}

// Splits x into hi + lo/16 where hi keeps the top 4 significant bits of x (exactly an e4m3
// value while |x| is in e4m3's normal range) and lo carries the next bits.  Two e4m3 numbers
// then hold 8 significant bits, the precision of bf16, which lets an e4m3 tensor-core tile
// multiply a bf16-precision operand: the operand occupies two rows of the tile.
__device__ __forceinline__ void split_hi_lo(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xfff00000u);
  lo = (x - hi) * 16.0f;
}

// The same split with the low part unscaled (x = hi + lo) when UNSCALED: for operands whose two
// parts are multiplied separately and added by the tensor core itself.
template <bool UNSCALED>
__device__ __forceinline__ void split_parts(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xfff00000u);
  lo = UNSCALED ? x - hi : (x - hi) * 16.0f;
}

__device__ __forceinline__ float bf16_lo_to_f32(uint32_t packed) {
  return __uint_as_float(packed << 16);
}
__device__ __forceinline__ float bf16_hi_to_f32(uint32_t packed) {
  return __uint_as_float(packed & 0xffff0000u);
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
  v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
  return v;
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(kFullMask, v, 1);
  v += __shfl_xor_sync(kFullMask, v, 2);
  return v;
}

}  // namespace pa
