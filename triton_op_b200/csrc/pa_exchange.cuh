// Cross-GPU exchange of (max, sum, output) triples over NVLink peer stores, for KV-partition-
// sharded decode (no counterpart in the single-GPU reference; the reduce it completes is
// pa_decode_triton_gluon_fp8.py:1187-1333 applied across GPUs).
//
// Every rank owns a receive buffer [2 parities][world][message] and a flag word per source
// rank, both mapped into its peers (CUDA IPC).  One decode step `epoch` (1, 2, ...):
//   pa_push_message_kernel   copies this rank's packed message (m | l | pad | o, as the reduce
//                            kernel left it) into slot [epoch & 1][rank] of EVERY rank's
//                            buffer with plain 16-byte stores, fences, and then stores `epoch`
//                            into flag[rank] of every rank;
//   pa_merge_wait_kernel     waits (bounded) until all its flags have reached `epoch`, then
//                            merges the `world` messages of parity epoch & 1 like
//                            pa_merge_triples_kernel.
// A rank cannot run two steps ahead of a peer (its next push comes after its own merge, which
// waited for that peer's push of the same step), so two parities of buffers are enough and the
// flags only ever grow.  Remote data is always WRITTEN into the consumer's memory and read
// locally; nothing here waits on a kernel of the same GPU.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "../../include/pa_decode_sm100.h"

namespace pa {

constexpr int kMaxPeers = 16;

struct ExchangeParams {
  const float* msg;                 // this rank's message, msg_floats floats (a multiple of 4)
  float* recv[kMaxPeers];           // rank g's receive buffer [2][world][msg_floats] (g == rank: the local one)
  int* flags[kMaxPeers];            // rank g's flag words [world]
  int* done;                        // local: [0] CTA arrival count (zero between launches), [1] steps pushed so far
  int32_t* status;                  // optional
  int32_t world, rank, epoch;
  int64_t msg_floats;
};

__global__ void __launch_bounds__(256) pa_push_message_kernel(const __grid_constant__ ExchangeParams p) {
  // epoch 0: the step number lives on the device (a captured launch replays with the same
  // arguments).  done[1] only changes after every CTA has counted itself in, below.
  int epoch = p.epoch;
  if (epoch == 0) epoch = *reinterpret_cast<volatile int*>(p.done + 1) + 1;
  const int64_t n16 = p.msg_floats / 4;
  const float4* src = reinterpret_cast<const float4*>(p.msg);
  const int64_t slot = ((int64_t)(epoch & 1) * p.world + p.rank) * p.msg_floats;
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n16; v += (int64_t)gridDim.x * blockDim.x) {
    const float4 x = src[v];
    for (int g = 0; g < p.world; ++g) reinterpret_cast<float4*>(p.recv[g] + slot)[v] = x;
  }
  // every CTA publishes its stores system-wide before it counts itself in; the last one to do so
  // (having seen all the others) raises the flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.done, 1) == (int)gridDim.x - 1) {
      p.done[0] = 0;
      p.done[1] = epoch;
      __threadfence_system();
      for (int g = 0; g < p.world; ++g) {
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.flags[g] + p.rank), "r"(epoch) : "memory");
      }
    }
  }
}

struct MergeWaitParams {
  uint8_t* out;                     // bf16 [num_rows, head_size], row stride out_stride_row elements
  int64_t out_stride_row;
  const float* recv;                // local receive buffer [2][world][msg_floats]
  const int* flags;                 // local flag words [world]
  const int* counters;              // the push kernel's counters (epoch 0: step number = counters[1])
  int32_t* status;                  // optional
  int32_t world, epoch, num_rows;
  int64_t msg_floats;
};

// One warp per output row, four rows per CTA.
__global__ void __launch_bounds__(128) pa_merge_wait_kernel(const __grid_constant__ MergeWaitParams p) {
  __shared__ int s_ok;
  const int epoch = p.epoch ? p.epoch : p.counters[1];   // written by the push launched before this one
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world) {
    // bounded wait for this source's message of the step (about a second, then give up)
    bool ok = false;
    for (uint32_t poll = 0; poll < (1u << 20); ++poll) {
      int f;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(f) : "l"(p.flags + threadIdx.x) : "memory");
      if (f >= epoch) { ok = true; break; }
      __nanosleep(200);
    }
    if (!ok) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, PA_DEV_WAIT_TIMEOUT);
    return;
  }
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= p.num_rows) return;
  const float* base = p.recv + (int64_t)(epoch & 1) * p.world * p.msg_floats;
  const int64_t o_off = p.msg_floats - (int64_t)p.num_rows * kD;
  float M = -INFINITY;
  for (int s = 0; s < p.world; ++s) {
    const float* msg = base + (int64_t)s * p.msg_floats;
    const float ls = __ldcg(msg + p.num_rows + row);
    const float ms = __ldcg(msg + row);
    if (ls > 0.f) M = fmaxf(M, ms);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float W = 0.f;
  for (int s = 0; s < p.world; ++s) {
    const float* msg = base + (int64_t)s * p.msg_floats;
    const float ls = __ldcg(msg + p.num_rows + row);
    const float ms = __ldcg(msg + row);
    if (!(ls > 0.f) || !(ms > -INFINITY)) continue;
    const float w = ls * expf(ms - M);
    const float4 v = __ldcg(reinterpret_cast<const float4*>(msg + o_off + row * kD + 4 * lane));
    W += w;
    acc[0] = fmaf(w, v.x, acc[0]);
    acc[1] = fmaf(w, v.y, acc[1]);
    acc[2] = fmaf(w, v.z, acc[2]);
    acc[3] = fmaf(w, v.w, acc[3]);
  }
  const float inv = W > 0.f ? 1.0f / W : 0.f;
  uint2 res;
  res.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
  res.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
  *reinterpret_cast<uint2*>(p.out + 2 * (row * p.out_stride_row + 4 * lane)) = res;
}

}  // namespace pa
