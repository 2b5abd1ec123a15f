// Cross-partition log-sum-exp reduce and the cross-shard triple merge.
//
// pa_reduce_kernel restates paged_attention_decode_v2_reduce_kernel
// (pa_decode_triton_gluon_fp8.py:1187-1333 in yanguahe/triton_op):
//   np = ceil(ctx / partition_size); M = max_p m_p; w_p = l_p * exp(m_p - M);
//   out = sum_p (w_p / sum w) * o_p   (fp32 accumulate, bf16 store).
// Differences by design: it loops over the partitions with a running sum instead of loading a
// [P_pow2, eqG, D] tile at once, so the partition count is unbounded; a partition whose l is 0
// (every key masked for that row) gets weight 0 instead of relying on zero-filled workspaces.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"

namespace pa {

// Triples that cross GPUs travel as flagged 16-byte lines {value, step, value, step}.  Each
// {value, step} pair is ONE naturally aligned 64-bit element of a two-element vector access: the
// memory model makes no promise about the order in which the elements of a vector access become
// visible, but every element is written and read whole, so a reader that finds the step number it
// waits for in a half has that half's value too -- no fence, no separate flag, one trip over the
// link.  A row's triple is 1 + kD / 2 lines: {m, l}, then {o[2i], o[2i+1]}.
constexpr int kMaxPeers = 16;
constexpr int kLinesPerRow = 1 + kD / 2;

__device__ __forceinline__ void st_line(uint4* dst, float a, float b, int step) {
  const uint64_t hi = (uint64_t)(uint32_t)step << 32;
  asm volatile("st.volatile.global.v2.b64 [%0], {%1, %2};" ::"l"(dst), "l"(hi | __float_as_uint(a)),
               "l"(hi | __float_as_uint(b))
               : "memory");
}
// Returns the line as {value a, step of a, value b, step of b}.
__device__ __forceinline__ uint4 ld_line(const uint4* src) {
  uint64_t a, b;
  asm volatile("ld.volatile.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(src) : "memory");
  return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}

struct ReduceParams {
  uint8_t* out;                 // bf16 [S, Hkv*eqG, D]; may be null when triples are stored
  const float* exp_sums;
  const float* max_logits;
  const uint8_t* tmp_out;       // bf16
  const int32_t* context_lens;
  const float* sink;            // optional [Hkv*G]: sink logit per query head, added to the row's weight sum
  float* tri_m;                 // optional fp32 triples
  float* tri_l;
  float* tri_o;
  // optional: the triples also go, as flagged lines, into slot [step & 1][push_rank] of every
  // rank's receive buffer [2][push_world][rows][kLinesPerRow] (entry push_rank: the local one)
  uint4* push[kMaxPeers];
  const int32_t* push_counter;  // push_step == 0: the step is push_counter[1] + 1 (steps merged so far, + 1)
  int32_t push_world, push_rank, push_step;
  int32_t S, Hkv, eqG, G, partition_size, max_partitions, ctx_cap;
  int64_t out_stride_seq, out_stride_head;
  int64_t ws_stride_seq, ws_stride_head, ws_stride_part;
  int64_t tmp_stride_seq, tmp_stride_head, tmp_stride_part, tmp_stride_row;
};

// One output row whose partitions (at most 32) all lie in one chunk, merged by one warp: the
// arithmetic of pa_reduce_kernel<1> below, operation for operation, so that a decode call gives
// the same bits whether its partitions are merged by that kernel or, in the single-launch form,
// by a warp of the partition kernel itself.  Loads go to L2 (ld.global.cg): the partitions were
// written by other SMs during the same launch.  lane owns head dims 4*lane..4*lane+3.
__device__ __noinline__ void merge_row_one_chunk(const float* __restrict__ max_logits, const float* __restrict__ exp_sums,
                                                 const uint8_t* __restrict__ tmp_out, int64_t ws_row, int64_t ws_stride_part,
                                                 int64_t tmp_row, int64_t tmp_stride_part, int np, float sink_logit,
                                                 bool has_sink, uint8_t* out_row, int lane) {
  float m = -INFINITY, l = 0.f;
  if (lane < np) {
    m = __ldcg(max_logits + ws_row + (int64_t)lane * ws_stride_part);
    l = __ldcg(exp_sums + ws_row + (int64_t)lane * ws_stride_part);
  }
  constexpr int kFlight = 16;
  uint2 raw[kFlight];
#pragma unroll
  for (int j = 0; j < kFlight; ++j)
    raw[j] = j < np ? __ldcg(reinterpret_cast<const uint2*>(tmp_out + 2 * (tmp_row + (int64_t)j * tmp_stride_part)))
                    : make_uint2(0u, 0u);
  float cm = (l > 0.f) ? m : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(kFullMask, cm, o));
  const float M = cm;
  const float w = (l > 0.f && m > -INFINITY) ? l * expf(m - M) : 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float W = 0.f;
  for (int j0 = 0; j0 < np; j0 += kFlight) {
    if (j0 > 0) {
#pragma unroll
      for (int j = 0; j < kFlight; ++j)
        raw[j] = (j0 + j) < np
                     ? __ldcg(reinterpret_cast<const uint2*>(tmp_out + 2 * (tmp_row + (int64_t)(j0 + j) * tmp_stride_part)))
                     : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < kFlight; ++j) {
      const float wj = __shfl_sync(kFullMask, w, (j0 + j) & 31);
      if ((j0 + j) < np && wj != 0.f) {
        W += wj;
        acc[0] = fmaf(wj, bf16_lo_to_f32(raw[j].x), acc[0]);
        acc[1] = fmaf(wj, bf16_hi_to_f32(raw[j].x), acc[1]);
        acc[2] = fmaf(wj, bf16_lo_to_f32(raw[j].y), acc[2]);
        acc[3] = fmaf(wj, bf16_hi_to_f32(raw[j].y), acc[3]);
      }
    }
  }
  float Wout = W;
  if (has_sink && W > 0.f) Wout += expf(sink_logit - M);
  const float inv_out = Wout > 0.f ? 1.0f / Wout : 0.f;
  uint2 o;
  o.x = pack_bf16x2(acc[0] * inv_out, acc[1] * inv_out);
  o.y = pack_bf16x2(acc[2] * inv_out, acc[3] * inv_out);
  *reinterpret_cast<uint2*>(out_row + 8 * lane) = o;
}

// ---- pieces shared by the reduce kernels --------------------------------------------------------
// Where one output row (sequence, kv head, row r) finds its partitions.
struct RowRef {
  int seq, head, r, np;
  int64_t ws_base, tmp_base;   // element offsets of partition 0 (tmp_base includes this lane's 4 head dims)
};

__device__ __forceinline__ RowRef row_ref(const ReduceParams& p, int64_t row, bool active, int lane) {
  RowRef a;
  // (32-bit divisions: the host refuses more than 2^31 - 1 rows, and a 64-bit division is a few
  // hundred instructions of a kernel that is a few hundred instructions per row otherwise)
  const unsigned row32 = (unsigned)row, per_head = (unsigned)p.eqG, per_seq = per_head * (unsigned)p.Hkv;
  const unsigned seq_u = row32 / per_seq, in_seq = row32 - seq_u * per_seq;
  a.head = (int)(in_seq / per_head);
  a.r = (int)(in_seq - (unsigned)a.head * per_head);
  a.seq = active ? (int)seq_u : 0;
  int ctx = active ? p.context_lens[a.seq] : 0;
  ctx = max(0, min(ctx, p.ctx_cap));
  a.np = min((ctx + p.partition_size - 1) / p.partition_size, p.max_partitions);
  a.ws_base = (int64_t)a.seq * p.ws_stride_seq + (int64_t)a.head * p.ws_stride_head + a.r;
  a.tmp_base = (int64_t)a.seq * p.tmp_stride_seq + (int64_t)a.head * p.tmp_stride_head +
               (int64_t)a.r * p.tmp_stride_row + 4 * lane;
  return a;
}

// Loads from the workspaces, stated as global loads (the compiler cannot tell from a pointer inside
// the parameter block, and generic loads cost it a handful of extra instructions each).
__device__ __forceinline__ uint2 ld_global_u2(const void* ptr) {
  uint2 v;
  asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ float ld_global_f32(const void* ptr) {
  float v;
  asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(ptr) : "memory");
  return v;
}

// One warp's share of a row: the 32-partition chunks `first`, `first + step`, ... folded into a
// running (maximum M, weight sum W, weighted output acc).  Partitions are taken 32 at a time
// (lane = partition for the max / weight, then FLIGHT partial-output rows in flight per step).
// The first FLIGHT rows of a chunk are requested together with the maxima and sums, so the usual
// row (at most 16 partitions) costs one memory round trip.
template <int FLIGHT>
__device__ __forceinline__ void reduce_chunks(const ReduceParams& p, const RowRef& a, int first, int step, int lane,
                                              float& M, float& W, float (&acc)[4]) {
  for (int p0 = first * 32; p0 < a.np; p0 += 32 * step) {
    const int pi = p0 + lane;
    const int cnt = min(32, a.np - p0);
    float m = -INFINITY, l = 0.f;
    if (pi < a.np) {
      m = ld_global_f32(p.max_logits + a.ws_base + (int64_t)pi * p.ws_stride_part);
      l = ld_global_f32(p.exp_sums + a.ws_base + (int64_t)pi * p.ws_stride_part);
    }
    const uint8_t* part0 = p.tmp_out + 2 * (a.tmp_base + (int64_t)p0 * p.tmp_stride_part);   // this lane's bytes of partition p0
    const int64_t part_bytes = 2 * p.tmp_stride_part;
    uint2 raw[FLIGHT];  // requested before the maximum is known
#pragma unroll
    for (int j = 0; j < FLIGHT; ++j) raw[j] = j < cnt ? ld_global_u2(part0 + j * part_bytes) : make_uint2(0u, 0u);
    float cm = (l > 0.f) ? m : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cm = fmaxf(cm, __shfl_xor_sync(kFullMask, cm, o));
    const float newM = fmaxf(M, cm);
    if (newM > M) {  // rescale what has been accumulated so far (M = -inf: nothing yet)
      const float f = (M == -INFINITY) ? 0.f : expf(M - newM);
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] *= f;
      W *= f;
      M = newM;
    }
    const float w = (l > 0.f && m > -INFINITY) ? l * expf(m - M) : 0.f;
    for (int j0 = 0; j0 < cnt; j0 += FLIGHT) {
      if (j0 > 0) {
#pragma unroll
        for (int j = 0; j < FLIGHT; ++j)
          raw[j] = (j0 + j) < cnt ? ld_global_u2(part0 + (j0 + j) * part_bytes) : make_uint2(0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < FLIGHT; ++j) {
        const float wj = __shfl_sync(kFullMask, w, (j0 + j) & 31);
        if ((j0 + j) < cnt && wj != 0.f) {  // a zero-weight partition may hold anything
          W += wj;
          acc[0] = fmaf(wj, bf16_lo_to_f32(raw[j].x), acc[0]);
          acc[1] = fmaf(wj, bf16_hi_to_f32(raw[j].x), acc[1]);
          acc[2] = fmaf(wj, bf16_lo_to_f32(raw[j].y), acc[2]);
          acc[3] = fmaf(wj, bf16_hi_to_f32(raw[j].y), acc[3]);
        }
      }
    }
  }
}

// Folds one more warp's (maximum, weight sum, weighted output) into a combination relative to the
// common maximum mx (the order of these calls is the order of the additions).
__device__ __forceinline__ void fold_partial(float ms, float ws, const float4& a, float mx, float& W, float (&acc)[4]) {
  if (!(ms > -INFINITY)) return;    // that warp saw no partition with weight
  const float f = expf(ms - mx);
  W = fmaf(ws, f, W);
  acc[0] = fmaf(a.x, f, acc[0]);
  acc[1] = fmaf(a.y, f, acc[1]);
  acc[2] = fmaf(a.z, f, acc[2]);
  acc[3] = fmaf(a.w, f, acc[3]);
}

// A finished row: sink weight, normalisation, and the stores (bf16 output, fp32 triple, peer lines).
__device__ __forceinline__ void finish_row(const ReduceParams& p, const RowRef& a, int64_t row, int64_t n_rows, int lane,
                                           float M, float W, float (&acc)[4]) {
  // sink token: a weight without a value, relative to the same maximum (triples stay without it)
  float Wout = W;
  if (p.sink != nullptr && W > 0.f) Wout += expf(p.sink[a.head * p.G + a.r % p.G] - M);
  const float inv = W > 0.f ? 1.0f / W : 0.f;
  const float inv_out = Wout > 0.f ? 1.0f / Wout : 0.f;
  float res[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    res[e] = acc[e] * inv_out;
    acc[e] *= inv;
  }
  if (p.out) {
    uint2 o;
    o.x = pack_bf16x2(res[0], res[1]);
    o.y = pack_bf16x2(res[2], res[3]);
    *reinterpret_cast<uint2*>(p.out + 2 * ((int64_t)a.seq * p.out_stride_seq +
                                           ((int64_t)a.head * p.eqG + a.r) * p.out_stride_head + 4 * lane)) = o;
  }
  if (p.tri_o) {
    if (lane == 0) {
      p.tri_m[row] = M;
      p.tri_l[row] = W;
    }
    *reinterpret_cast<float4*>(p.tri_o + row * kD + 4 * lane) =
        make_float4(acc[0], acc[1], acc[2], acc[3]);
  }
  if (p.push_world > 0) {
    const int step = p.push_step ? p.push_step : p.push_counter[1] + 1;
    const int64_t line0 = (((int64_t)(step & 1) * p.push_world + p.push_rank) * n_rows + row) * kLinesPerRow;
    for (int g = 0; g < p.push_world; ++g) {
      uint4* dst = p.push[g] + line0;
      if (lane == 0) st_line(dst, M, W, step);
      st_line(dst + 1 + 2 * lane, acc[0], acc[1], step);
      st_line(dst + 2 + 2 * lane, acc[2], acc[3], step);
    }
  }
}

// WPR warps per output row (sequence, kv head, row r); lane owns head dims 4*lane..4*lane+3.
// WPR = 1: four rows per CTA, the usual case (np <= 32: one chunk).  Long contexts have few rows
// and hundreds of partitions each, and a single warp would walk them one memory round trip
// after the other; with WPR = 16 the warps of a CTA take the 32-partition chunks of ONE row
// round-robin and combine their running (max, sum, weighted output) through shared memory.
// (Rows of up to 128 partitions have a kernel of their own below.)
template <int WPR>
__global__ void __launch_bounds__(WPR == 1 ? 128 : 512) pa_reduce_kernel(const __grid_constant__ ReduceParams p) {
  static_assert(WPR == 1 || WPR == 16, "one warp per row (four rows per CTA) or sixteen");
  constexpr int kWarps = WPR == 1 ? 4 : 16;
  constexpr int kRowsPerCta = kWarps / WPR;
  // the next kernel in the stream (the next step's partition kernel) may become resident now; it
  // waits for this grid to finish before it touches global memory
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int slice = warp % WPR;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + warp / WPR;
  const int64_t n_rows = (int64_t)p.S * p.Hkv * p.eqG;
  if (row >= n_rows) return;   // WPR = 16: one row per CTA, so the whole CTA leaves together
  const RowRef a = row_ref(p, row, true, lane);

  // The launch may overlap the tail of the partition kernel (programmatic dependent launch):
  // nothing that kernel wrote is read before this point.
  grid_dependency_wait();

  float M = -INFINITY;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float W = 0.f;
  // rows in flight: a 16-warp row has one 32-partition chunk per warp, taken in one round trip
  reduce_chunks<WPR == 16 ? 32 : 16>(p, a, slice, WPR, lane, M, W, acc);
  if (WPR > 1) {
    // combine the warps' partial results: warp `slice` holds (M, W, acc) of its chunks
    __shared__ float s_m[kWarps], s_w[kWarps];
    __shared__ float4 s_acc[kWarps][32];
    if (lane == 0) {
      s_m[slice] = M;
      s_w[slice] = W;
    }
    s_acc[slice][lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (slice != 0) return;
    float mx = -INFINITY;
#pragma unroll
    for (int s = 0; s < WPR; ++s) mx = fmaxf(mx, s_m[s]);
    W = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = 0.f;
#pragma unroll
    for (int s = 0; s < WPR; ++s) fold_partial(s_m[s], s_w[s], s_acc[s][lane], mx, W, acc);
    M = mx;
  }
  finish_row(p, a, row, n_rows, lane, M, W, acc);
}

// Rows of 33 to 128 partitions (two to four chunks) among, typically, thousands of rows of one
// chunk: a serving mix with a few long contexts.  Eight rows per CTA, one warp each: the warp
// reduces its row's first chunk; the further chunks of the CTA's long rows are then dealt over
// all eight warps, and each long row's warp folds its chunks' results in chunk order.  (Four
// warps per row, one chunk each, gives the same numbers with three of four warps idle on every
// short row.)
constexpr int kMidRows = 8;           // rows (= warps) per CTA
constexpr int kMidChunks = 4;         // chunks per row at most (128 partitions)
// one chunk of one row
__device__ __forceinline__ void reduce_one_chunk(const ReduceParams& p, const RowRef& a, int chunk, int lane,
                                                 float* M, float* W, float* acc) {
  float m = -INFINITY, w = 0.f;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  reduce_chunks<16>(p, a, chunk, kMidChunks, lane, m, w, v);
  *M = m;
  *W = w;
  acc[0] = v[0], acc[1] = v[1], acc[2] = v[2], acc[3] = v[3];
}
__global__ void __launch_bounds__(kMidRows * 32, 3) pa_reduce_mid_kernel(const __grid_constant__ ReduceParams p) {
  __shared__ int s_extra[kMidRows];                                   // further chunks of each row
  __shared__ float s_m[kMidRows * (kMidChunks - 1)], s_w[kMidRows * (kMidChunks - 1)];
  __shared__ float4 s_acc[kMidRows * (kMidChunks - 1)][32];
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t row0 = (int64_t)blockIdx.x * kMidRows;
  const int64_t row = row0 + warp;
  const int64_t n_rows = (int64_t)p.S * p.Hkv * p.eqG;
  const bool active = row < n_rows;
  const RowRef a = row_ref(p, row, active, lane);
  const int extra = active ? max(0, min((a.np + 31) / 32, kMidChunks) - 1) : 0;
  if (lane == 0) s_extra[warp] = extra;
  grid_dependency_wait();

  // the row's first chunk
  float M, W, acc[4];
  reduce_one_chunk(p, a, 0, lane, &M, &W, acc);
  __syncthreads();
  // further chunks of the CTA's rows, numbered row by row: task t = chunk 1 + (t - first task of its row)
  int first_task = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kMidRows; ++w) {
    const int e = s_extra[w];
    if (w < warp) first_task += e;
    total += e;
  }
  for (int t = warp; t < total; t += kMidRows) {
    int owner = -1, before = 0, pre = 0;    // the row whose tasks [pre, pre + extra) hold t
#pragma unroll
    for (int w = 0; w < kMidRows; ++w) {
      const int e = s_extra[w];
      if (owner < 0 && t < pre + e) {
        owner = w;
        before = pre;
      }
      pre += e;
    }
    const RowRef b = row_ref(p, row0 + owner, true, lane);
    float m2, w2, a2[4];
    reduce_one_chunk(p, b, 1 + (t - before), lane, &m2, &w2, a2);
    if (lane == 0) {
      s_m[t] = m2;
      s_w[t] = w2;
    }
    s_acc[t][lane] = make_float4(a2[0], a2[1], a2[2], a2[3]);
  }
  __syncthreads();
  if (!active) return;
  if (extra > 0) {   // chunk 0 from this warp's registers, then the row's further chunks in order
    float mx = M;
    for (int c = 0; c < extra; ++c) mx = fmaxf(mx, s_m[first_task + c]);
    const float m0 = M, w0 = W;
    const float4 a0 = make_float4(acc[0], acc[1], acc[2], acc[3]);
    W = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] = 0.f;
    fold_partial(m0, w0, a0, mx, W, acc);
    for (int c = 0; c < extra; ++c) fold_partial(s_m[first_task + c], s_w[first_task + c], s_acc[first_task + c][lane], mx, W, acc);
    M = mx;
  }
  finish_row(p, a, row, n_rows, lane, M, W, acc);
}

// One warp per row; merges `num_shards` (m, l, o) triples.  Shard s keeps its m and l rows
// ml_stride floats and its o rows o_stride floats after those of shard s - 1.
__global__ void __launch_bounds__(128)
pa_merge_triples_kernel(uint8_t* out, int64_t out_stride_row, const float* __restrict__ m,
                        const float* __restrict__ l, const float* __restrict__ o, int num_shards,
                        int num_rows, int64_t ml_stride, int64_t o_stride) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= num_rows) return;
  float M = -INFINITY;
  for (int s = 0; s < num_shards; ++s) {
    const float ls = l[(int64_t)s * ml_stride + row];
    const float ms = m[(int64_t)s * ml_stride + row];
    if (ls > 0.f) M = fmaxf(M, ms);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float W = 0.f;
  for (int s = 0; s < num_shards; ++s) {
    const float ls = l[(int64_t)s * ml_stride + row];
    const float ms = m[(int64_t)s * ml_stride + row];
    if (!(ls > 0.f) || !(ms > -INFINITY)) continue;
    const float w = ls * expf(ms - M);
    const float4 v = *reinterpret_cast<const float4*>(o + (int64_t)s * o_stride + row * kD + 4 * lane);
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
  *reinterpret_cast<uint2*>(out + 2 * (row * out_stride_row + 4 * lane)) = res;
}

}  // namespace pa
