// Read-only streaming probe: what HBM gives a kernel that only reads, through the same mechanism
// the partition kernels use (cp.async.bulk of 2 KB runs into shared-memory rings, one persistent
// CTA per SM, nothing computed).  The benchmark quotes the decode call against this ceiling next
// to the read+write copy bandwidth.  No counterpart in the reference.
#pragma once

#include "pa_common.cuh"
#include "../../include/pa_decode_sm100.h"

namespace pa {

constexpr int kProbeWarps = 8;
constexpr int kProbeSlots = 3;
constexpr int kProbeSlotBytes = 8192;            // four 2 KB runs per slot
constexpr int kProbeRun = 2048;
constexpr int kProbeSmem = 1024 + kProbeWarps * kProbeSlots * kProbeSlotBytes;

// Units of 8 KB are dealt round-robin over all warps of the grid; unit u of region r starts at
// base[r] + u * 8 KB.  Every wait is bounded (PA_DEV_WAIT_TIMEOUT in *status).
__global__ void __launch_bounds__(kProbeWarps * 32, 1)
pa_stream_probe_kernel(const uint8_t* a, const uint8_t* b, long long units_each, int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t bars = smem_addr(smem) + warp * kProbeSlots * 8;
  const uint32_t ring = smem_addr(smem) + 1024 + warp * kProbeSlots * kProbeSlotBytes;
  if (lane == 0) {
    for (int s = 0; s < kProbeSlots; ++s) mbar_init(bars + s * 8, 1);
    mbar_fence_init();
    fence_proxy_async();
  }
  __syncthreads();
  const uint64_t pol = l2_policy_evict_first();
  const long long total = 2 * units_each;
  const long long wtot = (long long)gridDim.x * kProbeWarps;
  long long next = (long long)blockIdx.x * kProbeWarps + warp;   // next unit to request
  int slot_p = 0;
  auto issue = [&]() {
    if (next >= total) return;
    const uint8_t* src = (next < units_each ? a + next * kProbeSlotBytes : b + (next - units_each) * kProbeSlotBytes);
    const uint32_t bar = bars + slot_p * 8;
    if (lane == 0) mbar_arrive_expect_tx(bar, kProbeSlotBytes);
    __syncwarp();
    if (lane < kProbeSlotBytes / kProbeRun)
      bulk_g2s(ring + slot_p * kProbeSlotBytes + lane * kProbeRun, src + lane * kProbeRun, kProbeRun, bar, pol);
    next += wtot;
    if (++slot_p == kProbeSlots) slot_p = 0;
  };
  for (int s = 0; s < kProbeSlots; ++s) issue();
  int slot_c = 0;
  uint32_t phase = 0;
  for (long long u = (long long)blockIdx.x * kProbeWarps + warp; u < total; u += wtot) {
    if (!__all_sync(kFullMask, mbar_wait(bars + slot_c * 8, phase))) {
      if (lane == 0 && status) atomicOr(status, PA_DEV_WAIT_TIMEOUT);
      break;
    }
    if (++slot_c == kProbeSlots) {
      slot_c = 0;
      phase ^= 1;
    }
    issue();
  }
}

}  // namespace pa
