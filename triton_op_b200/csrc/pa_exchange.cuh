// Cross-GPU exchange of (max, sum, output) triples over NVLink peer stores, for KV-partition-
// sharded decode (no counterpart in the single-GPU reference; the reduce it completes is
// pa_decode_triton_gluon_fp8.py:1187-1333 applied across GPUs).
//
// Every rank owns a receive buffer [2 parities][world][rows][kLinesPerRow] of flagged 16-byte
// lines, mapped into its peers (CUDA IPC).  One decode step (1, 2, ...):
//   the reduce kernel     stores each row's triple, as lines flagged with the step number, into
//                         slot [step & 1][rank] of EVERY rank's buffer (plain stores; nothing to
//                         fence, the flag travels inside each 8-byte half line);
//   pa_merge_wait_kernel  reads the `world` triples of its row from the local buffer, waiting
//                         (bounded) for lines whose flag is not the step's yet, and merges them
//                         like pa_merge_triples_kernel.
// A rank cannot run two steps ahead of a peer (its next reduce comes after its own merge, which
// waited for that peer's lines of the same step), so two parities of buffers are enough.  Remote
// data is always WRITTEN into the consumer's memory and read locally; nothing here waits on a
// kernel of the same GPU.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "pa_reduce.cuh"
#include "../../include/pa_decode_sm100.h"

namespace pa {

struct MergeWaitParams {
  uint8_t* out;                     // bf16 [num_rows, head_size], row stride out_stride_row elements
  int64_t out_stride_row;
  const uint4* recv;                // local receive buffer
  int32_t* counters;                // [0] warps done (zero between launches), [1] steps merged so far
  int32_t* status;                  // optional
  int32_t world, step, num_rows;
};

constexpr uint32_t kLinePolls = 1u << 20;   // with the sleep below: about a second, then give up

// Waits until both halves of the line carry `step`; false when the wait ran out.
__device__ __forceinline__ bool wait_line(const uint4* src, int step, uint4& v) {
  for (uint32_t poll = 0; poll < kLinePolls; ++poll) {
    if ((int)v.y == step && (int)v.w == step) return true;
    __nanosleep(100);
    v = ld_line(src);
  }
  return (int)v.y == step && (int)v.w == step;
}

// One warp per output row, four rows per CTA; lane owns head dims 4*lane .. 4*lane+3.
__global__ void __launch_bounds__(128) pa_merge_wait_kernel(const __grid_constant__ MergeWaitParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  // step 0: counted on the device.  counters[1] changes only after every warp of this launch
  // has counted itself in below, i.e. after every warp has read it here.
  const int step = p.step ? p.step : p.counters[1] + 1;
  bool ok = true;
  if (row < p.num_rows) {
    const uint4* base = p.recv + (int64_t)(step & 1) * p.world * p.num_rows * kLinesPerRow + row * kLinesPerRow;
    const int64_t src_stride = (int64_t)p.num_rows * kLinesPerRow;
    float M = -INFINITY, W = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr int kBatch = 8;   // sources whose lines are requested together
    for (int s0 = 0; s0 < p.world && ok; s0 += kBatch) {
      uint4 h[kBatch], a[kBatch], b[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (s0 + j < p.world) {
          const uint4* src = base + (s0 + j) * src_stride;
          h[j] = ld_line(src);
          a[j] = ld_line(src + 1 + 2 * lane);
          b[j] = ld_line(src + 2 + 2 * lane);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (s0 + j < p.world && ok) {
          const uint4* src = base + (s0 + j) * src_stride;
          ok = wait_line(src, step, h[j]) && wait_line(src + 1 + 2 * lane, step, a[j]) &&
               wait_line(src + 2 + 2 * lane, step, b[j]);
          ok = __all_sync(kFullMask, ok);
          const float ms = __uint_as_float(h[j].x), ls = __uint_as_float(h[j].z);
          if (ok && ls > 0.f && ms > -INFINITY) {
            const float newM = fmaxf(M, ms);
            const float f = (M == -INFINITY) ? 0.f : expf(M - newM);
            const float w = ls * expf(ms - newM);
            W = fmaf(W, f, w);
            acc[0] = fmaf(acc[0], f, w * __uint_as_float(a[j].x));
            acc[1] = fmaf(acc[1], f, w * __uint_as_float(a[j].z));
            acc[2] = fmaf(acc[2], f, w * __uint_as_float(b[j].x));
            acc[3] = fmaf(acc[3], f, w * __uint_as_float(b[j].z));
            M = newM;
          }
        }
      }
    }
    if (ok) {
      const float inv = W > 0.f ? 1.0f / W : 0.f;
      uint2 res;
      res.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
      res.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<uint2*>(p.out + 2 * (row * p.out_stride_row + 4 * lane)) = res;
    } else if (lane == 0 && p.status) {
      atomicOr(p.status, PA_DEV_WAIT_TIMEOUT);
    }
  }
  // the last warp of the launch closes the step (device-counted steps only)
  if (p.step == 0 && lane == 0) {
    const int total = (int)gridDim.x * 4;
    if (atomicAdd(p.counters, 1) == total - 1) {
      p.counters[0] = 0;
      p.counters[1] = step;
    }
  }
}

}  // namespace pa
