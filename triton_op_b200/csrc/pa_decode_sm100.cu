// Host side of the C ABI declared in include/pa_decode_sm100.h: argument validation, the
// shared-memory carve and grid of the partition kernel, and the launches.  Nothing here
// allocates device memory, synchronises or touches any stream but the caller's.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

#include "../../include/pa_decode_sm100.h"
#include "pa_partition_bf16.cuh"
#include "pa_partition_fp8.cuh"
#include "pa_partition_tc.cuh"
#include "pa_reduce.cuh"
#include "pa_cache_write.cuh"
#include "pa_exchange.cuh"
#include "pa_stream_probe.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

struct DeviceInfo {
  int sm_count = 0;
  int max_smem_optin = 0;
  bool ready = false;
};
constexpr int kMaxDevices = 64;
DeviceInfo g_dev[kMaxDevices];

int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return PA_ERR_CUDA;
}

// Device attributes are immutable, so a benign race between threads writes the same values.
int device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return PA_ERR_UNSUPPORTED;
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    int sm = 0, smem = 0;
    e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    d.sm_count = sm;
    d.max_smem_optin = smem;
    d.ready = true;
  }
  *out = &d;
  return PA_OK;
}

// cuTensorMapEncodeTiled, looked up through the runtime so that the library does not link libcuda.
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = []() -> TensorMapEncodeFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &st) != cudaSuccess ||
        st != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<TensorMapEncodeFn>(ptr);
  }();
  return fn;
}

// Descriptor of the value cache [NB, Hkv, 128, bs] (e4m3) for boxes of [128 head dims][span tokens],
// written to shared memory with the swizzle the tensor core reads.
int encode_value_map(const PaDecodeParams* p, CUtensorMap* out) {
  TensorMapEncodeFn enc = tensor_map_encoder();
  if (!enc) return PA_ERR_CUDA;
  const cuuint32_t span = p->block_size == 64 ? 64 : 128;
  const cuuint64_t dims[4] = {(cuuint64_t)p->block_size, (cuuint64_t)pa::kD, (cuuint64_t)p->num_kv_heads,
                              (cuuint64_t)p->num_blocks};
  const cuuint64_t strides[3] = {(cuuint64_t)p->block_size, (cuuint64_t)p->v_stride_head, (cuuint64_t)p->v_stride_block};
  const cuuint32_t box[4] = {span, (cuuint32_t)pa::kD, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(p->value_cache), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         span == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return PA_ERR_CUDA;
  }
  return PA_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int round_up(int v, int a) { return (v + a - 1) / a * a; }

struct LaunchPlan {
  pa::KernelParams kp;
  CUtensorMap vmap;   // tiled-copy descriptor of the value cache (pages of 64 tokens or more)
  int warps = 0;      // consumer warps per CTA
  int mtiles = 0;     // 8-row query tiles per warp
  bool per_token = false;
  bool tensor_path = false;  // tcgen05 kernel (else the mma.sync kernel)
  bool fused = false;        // tcgen05 kernel in its single-launch form: it also merges the partitions
  bool pair = false;         // tcgen05 kernel on 512-token partitions (two work items per partition)
  bool staged = false;       // tcgen05 kernel: per-token scales are staged in the query slots
  bool bf16_kv = false;      // bf16 KV cache (mma.sync bf16 kernel)
  int rows = 0;              // query rows per work item (tcgen05 kernel)
  int grid = 0;
  int smem = 0;
};

// Validation common to every entry point that reads PaDecodeParams.
int validate(const PaDecodeParams* p, bool need_partition_inputs, bool need_out) {
  if (!p) return PA_ERR_NULL_POINTER;
  if (p->struct_size != sizeof(PaDecodeParams) || p->abi_version != PA_ABI_VERSION) return PA_ERR_ABI;
  if (p->num_seqs < 0 || p->num_kv_heads <= 0 || p->query_group_size <= 0 || p->query_len <= 0 ||
      p->block_size <= 0 || p->partition_size <= 0 || p->max_partitions <= 0 ||
      p->max_blocks_per_seq <= 0 || p->num_blocks <= 0)
    return PA_ERR_BAD_SHAPE;
  if (p->head_size != pa::kD) return PA_ERR_UNSUPPORTED;
  if (p->query_len > 4) return PA_ERR_UNSUPPORTED;  // reference: QUERY_SEQ_LEN <= 4
  if (p->out_dtype != PA_DT_BF16) return PA_ERR_UNSUPPORTED;
  if (!p->context_lens || !p->exp_sums || !p->max_logits || !p->tmp_out) return PA_ERR_NULL_POINTER;
  if (need_out && !p->out) return PA_ERR_NULL_POINTER;
  if (p->partition_size % p->block_size != 0 && p->block_size % p->partition_size != 0)
    return PA_ERR_BAD_SHAPE;
  if (need_partition_inputs) {
    if (!p->query || !p->key_cache || !p->value_cache || !p->block_tables) return PA_ERR_NULL_POINTER;
    if (p->kv_quant_mode != PA_QUANT_NONE && (!p->key_scale || !p->value_scale))
      return PA_ERR_NULL_POINTER;
    if (p->q_quant_mode != PA_QUANT_NONE && !p->query_scale) return PA_ERR_NULL_POINTER;
  }
  if ((p->tmp_stride_row & 7) || (p->tmp_stride_part & 7) || (p->tmp_stride_head & 7) ||
      (p->tmp_stride_seq & 7) || !aligned16(p->tmp_out))
    return PA_ERR_ALIGNMENT;
  if (need_out && ((p->out_stride_head & 3) || (p->out_stride_seq & 3) ||
                   (reinterpret_cast<uintptr_t>(p->out) & 7u)))
    return PA_ERR_ALIGNMENT;
  return PA_OK;
}

// allow_fuse: the caller wants the whole decode (partitions and their merge) and would take it as
// one launch where the kernel has that form.
int make_plan(const PaDecodeParams* p, LaunchPlan* plan, bool allow_fuse = false) {
  int rc = validate(p, true, false);
  if (rc != PA_OK) return rc;
  DeviceInfo* dev = nullptr;
  rc = device_info(&dev);
  if (rc != PA_OK) return rc;

  const int eqG = p->query_group_size * p->query_len;
  if (p->q_dtype != PA_DT_BF16 && p->q_dtype != PA_DT_E4M3FN) return PA_ERR_UNSUPPORTED;
  const int q_item = p->q_dtype == PA_DT_BF16 ? 2 : 1;   // bytes per query element
  if (p->kv_dtype != PA_DT_E4M3FN && p->kv_dtype != PA_DT_BF16) return PA_ERR_UNSUPPORTED;
  const bool bf16_kv = p->kv_dtype == PA_DT_BF16;
  const int kv_item = bf16_kv ? 2 : 1;  // bytes per cache element
  if (bf16_kv && p->kv_quant_mode == PA_QUANT_PER_TOKEN) return PA_ERR_UNSUPPORTED;
  if (p->block_size != 16 && p->block_size != 64 && p->block_size != 1024) return PA_ERR_UNSUPPORTED;
  // Transposed values [NB, Hkv, bs/16, D, 16] (e4m3): a 16-token page is the same bytes as the
  // normal layout; longer pages are served by the tcgen05 kernel as 2 KB runs.
  const bool v_trans = p->v_layout == PA_V_TRANSPOSED && p->block_size != 16;
  if (p->v_layout != PA_V_NORMAL && p->v_layout != PA_V_TRANSPOSED) return PA_ERR_UNSUPPORTED;
  if (p->v_layout == PA_V_TRANSPOSED && p->kv_dtype != PA_DT_E4M3FN) return PA_ERR_UNSUPPORTED;
  if (eqG > 64) return PA_ERR_UNSUPPORTED;
  // tcgen05 kernel: 256-token partitions.  tune_warps == 4 / 8 explicitly asks for the mma.sync
  // kernel, which also covers other partition sizes for 16-token pages and up to 16 query rows.
  // 512-token partitions run on it too (as pairs of 256-token items merged in the epilogue) with
  // up to 16 query rows and no ALiBi.
  const bool pair = !bf16_kv && p->partition_size == 2 * pa::tc::kItemTokens && p->tune_warps == 0 && eqG <= 16 &&
                    p->alibi_slopes == nullptr && p->trace == nullptr;
  const bool tensor_path = !bf16_kv && (p->partition_size == pa::tc::kItemTokens || pair) && p->tune_warps == 0;
  if (!tensor_path) {
    if (p->block_size != 16 || eqG > 16 || q_item != 2) return PA_ERR_UNSUPPORTED;
    if (p->partition_size % (bf16_kv ? pa::kPageTokens : pa::kStageTokens) != 0 ||
        p->partition_size / p->block_size > 32)
      return PA_ERR_UNSUPPORTED;
  }
  // bulk copies: 16-byte aligned sources, contiguous page-of-one-head runs
  if (!aligned16(p->key_cache) || !aligned16(p->value_cache) || !aligned16(p->query))
    return PA_ERR_ALIGNMENT;
  if (((p->k_stride_block * kv_item) & 15) || ((p->k_stride_head * kv_item) & 15) ||
      ((p->v_stride_block * kv_item) & 15) || ((p->v_stride_head * kv_item) & 15))
    return PA_ERR_ALIGNMENT;
  if (p->q_stride_head != pa::kD || ((p->q_stride_seq * q_item) & 15)) return PA_ERR_ALIGNMENT;
  const bool per_token = p->kv_quant_mode == PA_QUANT_PER_TOKEN;
  if (per_token) {
    if (!aligned16(p->key_scale) || !aligned16(p->value_scale) || (p->kv_scale_stride_block & 3) ||
        (p->kv_scale_stride_head & 3))
      return PA_ERR_ALIGNMENT;
  }

  pa::KernelParams& k = plan->kp;
  memset(&k, 0, sizeof(k));
  k.q = static_cast<const uint8_t*>(p->query);
  k.k = static_cast<const uint8_t*>(p->key_cache);
  k.v = static_cast<const uint8_t*>(p->value_cache);
  k.block_tables = p->block_tables;
  k.context_lens = p->context_lens;
  k.q_scale = p->query_scale;
  k.k_scale = p->key_scale;
  k.v_scale = p->value_scale;
  k.alibi = p->alibi_slopes;
  k.exp_sums = p->exp_sums;
  k.max_logits = p->max_logits;
  k.tmp_out = static_cast<uint8_t*>(p->tmp_out);
  k.status = p->status;
  k.trace = reinterpret_cast<unsigned long long*>(p->trace);
  k.S = p->num_seqs;
  k.Hkv = p->num_kv_heads;
  k.G = p->query_group_size;
  k.L = p->query_len;
  k.eqG = eqG;
  k.block_size = p->block_size;
  k.num_blocks = p->num_blocks;
  k.max_blocks_per_seq = p->max_blocks_per_seq;
  k.partition_size = p->partition_size;
  k.max_partitions = p->max_partitions;
  k.pages_per_partition = p->partition_size / p->block_size;
  const int64_t cap = (int64_t)p->max_blocks_per_seq * p->block_size;
  k.ctx_cap = cap > 0x7fffffff ? 0x7fffffff : (int32_t)cap;
  k.q_stride_seq = p->q_stride_seq * q_item;    // elements -> bytes
  k.q_stride_head = p->q_stride_head * q_item;
  k.q_is_fp8 = q_item == 1;
  k.k_stride_block = p->k_stride_block * kv_item;   // elements -> bytes
  k.k_stride_head = p->k_stride_head * kv_item;
  k.v_stride_block = p->v_stride_block * kv_item;
  k.v_stride_head = p->v_stride_head * kv_item;
  k.bt_stride_seq = p->bt_stride_seq;
  k.q_scale_stride_seq = p->q_scale_stride_seq;
  k.kvs_stride_block = p->kv_scale_stride_block;
  k.kvs_stride_head = p->kv_scale_stride_head;
  k.ws_stride_seq = p->ws_stride_seq;
  k.ws_stride_head = p->ws_stride_head;
  k.ws_stride_part = p->ws_stride_part;
  k.tmp_stride_seq = p->tmp_stride_seq;
  k.tmp_stride_head = p->tmp_stride_head;
  k.tmp_stride_part = p->tmp_stride_part;
  k.tmp_stride_row = p->tmp_stride_row;
  k.q_quant_mode = p->q_quant_mode;
  k.kv_quant_mode = p->kv_quant_mode;
  k.softmax_scale = p->softmax_scale;

  plan->per_token = per_token;
  plan->mtiles = eqG <= 8 ? 1 : 2;

  // upper bound on work items, for the grid
  int64_t parts_cap = (cap + p->partition_size - 1) / p->partition_size;
  if (parts_cap > p->max_partitions) parts_cap = p->max_partitions;
  const int64_t items_cap = (int64_t)p->num_seqs * p->num_kv_heads * parts_cap;
  const int index_bytes = round_up((p->num_seqs + 1) * 4, 16) + round_up(p->num_seqs * 4 + 4, 16);

  plan->tensor_path = tensor_path;
  memset(&plan->vmap, 0, sizeof(plan->vmap));
  if (plan->tensor_path) {
    k.v_trans = v_trans ? 1 : 0;
    if (p->block_size >= 64 && !v_trans) {
      rc = encode_value_map(p, &plan->vmap);
      if (rc != PA_OK) return rc;
    }
    const int qr = eqG <= 4 ? 4 : (eqG <= 8 ? 8 : 16);   // query rows per work item
    const int nrb = (eqG + qr - 1) / qr;                  // row blocks per (partition, head)
    plan->rows = qr;
    k.num_row_blocks = nrb;
    k.early_start = p->tune_early >= 0 ? 1 : 0;
    plan->warps = pa::tc::kThreads / 32;
    // Single launch: one row block per (partition, head), every row's partitions within one chunk
    // of the merge (32), and a counter array for the row sets that are cut by the end of a team's range.
    plan->pair = pair;
    plan->fused = allow_fuse && !pair && p->merge_counters != nullptr && p->out != nullptr && nrb == 1 && qr <= 8 &&
                  p->max_partitions <= 32 && p->alibi_slopes == nullptr && p->trace == nullptr && p->tune_fuse > 0;
    if (plan->fused) {
      k.out = static_cast<uint8_t*>(p->out);
      k.sink = p->sink_tokens;
      k.merge_counters = p->merge_counters;
      k.out_stride_seq = p->out_stride_seq;
      k.out_stride_head = p->out_stride_head;
    }
    int off = pa::tc::kHeadBytes;
    k.off_seq_offsets = off;
    k.off_seq_ctx = off + round_up((p->num_seqs + 1) * 4, 16);
    off = round_up(off + index_bytes, 128);
    k.off_q = off;
    // Per-token scales of pages of 64 tokens or more are staged in the query slots (2 KB each)
    // while that fits; a batch whose index leaves no room runs the form whose softmax threads
    // fetch the scales themselves.  (The 16-row form for 512-token partitions never stages: its
    // slots and its halves' buffers do not fit together.)
    const bool want_staged = pa::tc::staged_token_scales(p->block_size, per_token) && !(pair && qr == 16);
    // Ring depths (K ring, V ring), deepest that fits.  The K ring is never shallower than the
    // three softmax groups (P.V trails QK^T by two items in the issue loop, and a group's waits
    // on the ring barriers assume a slot is not refilled within that lag), the V ring never
    // shallower than two; a batch whose in-kernel index leaves no room for that is refused.
    static const int kDepths[][2] = {{4, 4}, {4, 3}, {3, 3}, {3, 2}};
    if (p->tune_stages > 0 && p->tune_stages < 3) return PA_ERR_UNSUPPORTED;
    if (p->tune_vstages > 0 && p->tune_vstages < 2) return PA_ERR_UNSUPPORTED;
    bool placed = false;
    for (int attempt = 0; attempt < 2 && !placed; ++attempt) {
    const bool staged = want_staged && attempt == 0;
    if (attempt == 1 && (!want_staged || pair)) break;     // nothing else to try
    const int qslot = pa::tc::q_slot_bytes(qr, staged);
    for (const auto& d : kDepths) {
      if (p->tune_stages > 0 && d[0] > p->tune_stages) continue;
      if (p->tune_vstages > 0 && d[1] != p->tune_vstages) continue;
      const int off_p = round_up(off + pa::tc::kQSlots * qslot, 128);
      const int off_stash = round_up(off_p + pa::tc::kNG * pa::tc::p_tile_bytes(qr), 16);
      const int stash = pair ? 2 * (qr * pa::kD * 2 + 2 * 16 * 4) + pa::tc::kNG * 2 * 16 * 4 : 0;
      const int ring = round_up(off_stash + stash, 1024);
      const int total = ring + (d[0] + d[1]) * pa::tc::kHalfSlot;
      if (total <= dev->max_smem_optin) {
        k.off_p = off_p;
        k.off_stash = off_stash;
        k.off_ring = ring;
        k.off_vring = ring + d[0] * pa::tc::kHalfSlot;
        k.num_stages = d[0];
        k.num_vstages = d[1];
        plan->smem = total;
        plan->staged = staged;
        placed = true;
        break;
      }
    }
    }
    if (!placed) return PA_ERR_TOO_LARGE;  // num_seqs too large for the in-kernel index
    if (want_staged && !plan->staged) plan->fused = false;   // (the single-launch form exists staged only)
    int64_t items = items_cap * nrb * (pair ? 2 : 1);
    int64_t grid = items < dev->sm_count ? items : dev->sm_count;
    if (p->tune_ctas > 0 && p->tune_ctas < grid) grid = p->tune_ctas;
    if (grid < 1) grid = 1;
    k.team_size = 1;
    if (plan->fused) {
      // teams of CTAs that share the kv heads of a (sequence, partition) row: the largest size
      // that divides both the head count and the grid, or what the caller asks for
      int team = p->tune_fuse > 1 ? p->tune_fuse - 1 : 0;
      if (team == 0) {
        int a = (int)grid, b = p->num_kv_heads;
        while (b != 0) {
          const int t = a % b;
          a = b;
          b = t;
        }
        team = a;
      }
      if (team > grid || p->num_kv_heads % team != 0) return PA_ERR_UNSUPPORTED;
      grid -= grid % team;
      k.team_size = team;
    }
    plan->grid = (int)grid;
    return PA_OK;
  }

  plan->bf16_kv = bf16_kv;
  plan->warps = p->tune_warps > 0 ? p->tune_warps : 8;
  if (plan->warps != 4 && plan->warps != 8) return PA_ERR_UNSUPPORTED;
  if (bf16_kv) plan->warps = 8;

  // shared-memory carve
  const int stage = bf16_kv ? pa::kBf16Stage : pa::stage_bytes(per_token);
  const int qbuf = bf16_kv ? pa::kBf16QBuf : plan->mtiles * 8 * pa::kQRowBytes;
  int off = pa::kSmemHeadBytes;
  k.off_seq_offsets = off;
  off += round_up((p->num_seqs + 1) * 4, 16);
  k.off_seq_ctx = off;
  off += round_up(p->num_seqs * 4 + 4, 16);
  off = round_up(off, 128);
  k.off_q = off;
  off += plan->warps * qbuf;
  off = round_up(off, 128);
  k.off_ring = off;
  int stages = (dev->max_smem_optin - off) / (plan->warps * stage);
  if (stages > pa::kMaxStages) stages = pa::kMaxStages;
  if (p->tune_stages > 0 && p->tune_stages < stages) stages = p->tune_stages;
  if (stages < 2) return PA_ERR_TOO_LARGE;  // num_seqs too large for the in-kernel index
  k.num_stages = stages;
  plan->smem = off + plan->warps * stages * stage;

  // persistent grid: one CTA per SM, fewer when there cannot be that many work items
  int64_t grid = (items_cap + plan->warps - 1) / plan->warps;
  if (grid > dev->sm_count) grid = dev->sm_count;
  if (p->tune_ctas > 0 && p->tune_ctas < grid) grid = p->tune_ctas;
  if (grid < 1) grid = 1;
  plan->grid = (int)grid;
  return PA_OK;
}

template <int NW, int MT, bool PT>
int launch_partition_t(const LaunchPlan& plan, cudaStream_t stream) {
  auto kern = pa::pa_partition_fp8_p16_kernel<NW, MT, PT>;
  // Raising the dynamic shared-memory limit is per function and per device; repeating the
  // call is cheap and keeps the library free of per-device mutable state.
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem);
  if (e != cudaSuccess) return cuda_fail(e);
  kern<<<plan.grid, NW * 32, plan.smem, stream>>>(plan.kp);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}

template <int BS, int QR, bool PT, bool TRACE, bool ALIBI = false, bool FUSE = false, bool PAIR = false, bool STAGE = true>
int launch_tensor_t(const LaunchPlan& plan, cudaStream_t stream) {
  auto kern = pa::tc::pa_partition_fp8_tc_kernel<BS, QR, PT, TRACE, ALIBI, FUSE, PAIR, STAGE>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem);
  if (e != cudaSuccess) return cuda_fail(e);
  // Programmatic dependent launch: in a decode loop the CTAs may become resident and set up their
  // barriers and tensor memory while the kernel before this one in the stream (the previous step's
  // reduce) drains; the kernel waits (griddepcontrol.wait) before it reads or writes global memory.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)plan.grid);
  cfg.blockDim = dim3(pa::tc::kThreads);
  cfg.dynamicSmemBytes = (size_t)plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, plan.kp, plan.vmap);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}

template <int BS, bool TRACE>
int launch_tensor_bs(const LaunchPlan& plan, cudaStream_t stream) {
  const bool pt = plan.per_token;
  if (!TRACE && plan.fused) {                 // the single-launch instantiations (4 or 8 rows per item)
    if (plan.rows == 4)
      return pt ? launch_tensor_t<BS, 4, true, false, false, true>(plan, stream) : launch_tensor_t<BS, 4, false, false, false, true>(plan, stream);
    if (plan.rows == 8)
      return pt ? launch_tensor_t<BS, 8, true, false, false, true>(plan, stream) : launch_tensor_t<BS, 8, false, false, false, true>(plan, stream);
    return PA_ERR_UNSUPPORTED;
  }
  if (!TRACE && plan.pair) {                  // 512-token partitions
    switch (plan.rows) {
      case 4: return pt ? launch_tensor_t<BS, 4, true, false, false, false, true>(plan, stream) : launch_tensor_t<BS, 4, false, false, false, false, true>(plan, stream);
      case 8: return pt ? launch_tensor_t<BS, 8, true, false, false, false, true>(plan, stream) : launch_tensor_t<BS, 8, false, false, false, false, true>(plan, stream);
      case 16: return pt ? launch_tensor_t<BS, 16, true, false, false, false, true>(plan, stream) : launch_tensor_t<BS, 16, false, false, false, false, true>(plan, stream);
      default: return PA_ERR_UNSUPPORTED;
    }
  }
  if constexpr (!TRACE && BS >= 64) {
  if (pt && !plan.staged && !plan.pair) {     // per-token scales fetched by the softmax threads
    const bool al = plan.kp.alibi != nullptr;
    switch (plan.rows) {
      case 4: return al ? launch_tensor_t<BS, 4, true, false, true, false, false, false>(plan, stream) : launch_tensor_t<BS, 4, true, false, false, false, false, false>(plan, stream);
      case 8: return al ? launch_tensor_t<BS, 8, true, false, true, false, false, false>(plan, stream) : launch_tensor_t<BS, 8, true, false, false, false, false, false>(plan, stream);
      case 16: return al ? launch_tensor_t<BS, 16, true, false, true, false, false, false>(plan, stream) : launch_tensor_t<BS, 16, true, false, false, false, false, false>(plan, stream);
      default: return PA_ERR_UNSUPPORTED;
    }
  }
  }
  if (!TRACE && plan.kp.alibi != nullptr) {   // the ALiBi instantiations
    switch (plan.rows) {
      case 4: return pt ? launch_tensor_t<BS, 4, true, false, true>(plan, stream) : launch_tensor_t<BS, 4, false, false, true>(plan, stream);
      case 8: return pt ? launch_tensor_t<BS, 8, true, false, true>(plan, stream) : launch_tensor_t<BS, 8, false, false, true>(plan, stream);
      case 16: return pt ? launch_tensor_t<BS, 16, true, false, true>(plan, stream) : launch_tensor_t<BS, 16, false, false, true>(plan, stream);
      default: return PA_ERR_UNSUPPORTED;
    }
  }
  switch (plan.rows) {
    case 4: return pt ? launch_tensor_t<BS, 4, true, TRACE>(plan, stream) : launch_tensor_t<BS, 4, false, TRACE>(plan, stream);
    case 8: return pt ? launch_tensor_t<BS, 8, true, TRACE>(plan, stream) : launch_tensor_t<BS, 8, false, TRACE>(plan, stream);
    case 16: return pt ? launch_tensor_t<BS, 16, true, TRACE>(plan, stream) : launch_tensor_t<BS, 16, false, TRACE>(plan, stream);
    default: return PA_ERR_UNSUPPORTED;
  }
}

int launch_partition(const LaunchPlan& plan, cudaStream_t stream) {
  if (plan.kp.S == 0) return PA_OK;
  if (plan.tensor_path) {
    switch (plan.kp.block_size) {
      case 16:
#ifdef PA_TRACE_BUILD   // tuning builds (-DPA_TRACE_BUILD): clock stamps compiled in (pages of 16 and of 1024 tokens)
        if (plan.kp.trace != nullptr) return launch_tensor_bs<16, true>(plan, stream);
#endif
        return launch_tensor_bs<16, false>(plan, stream);
      case 64: return launch_tensor_bs<64, false>(plan, stream);
      case 1024:
#ifdef PA_TRACE_BUILD
        if (plan.kp.trace != nullptr) return launch_tensor_bs<1024, true>(plan, stream);
#endif
        return launch_tensor_bs<1024, false>(plan, stream);
      default: return PA_ERR_UNSUPPORTED;
    }
  }
  if (plan.bf16_kv) {
    auto kern = pa::pa_partition_bf16_p16_kernel<8>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, plan.smem);
    if (e != cudaSuccess) return cuda_fail(e);
    kern<<<plan.grid, 8 * 32, plan.smem, stream>>>(plan.kp);
    e = cudaGetLastError();
    return e != cudaSuccess ? cuda_fail(e) : PA_OK;
  }
#define PA_CASE(NW, MT, PT) \
  if (plan.warps == NW && plan.mtiles == MT && plan.per_token == PT) return launch_partition_t<NW, MT, PT>(plan, stream);
  PA_CASE(8, 1, false)
  PA_CASE(8, 1, true)
  PA_CASE(8, 2, false)
  PA_CASE(8, 2, true)
  PA_CASE(4, 1, false)
  PA_CASE(4, 1, true)
  PA_CASE(4, 2, false)
  PA_CASE(4, 2, true)
#undef PA_CASE
  return PA_ERR_UNSUPPORTED;
}

struct PushTarget {   // where the reduce kernel also sends its triples (KV-partition sharding)
  void* const* peer_recv;
  const int32_t* counters;
  int32_t world, rank, step;
};

int launch_reduce(const PaDecodeParams* p, float* tri_m, float* tri_l, float* tri_o,
                  cudaStream_t stream, const PushTarget* push = nullptr) {
  pa::ReduceParams r;
  memset(&r, 0, sizeof(r));
  if (push) {
    for (int g = 0; g < push->world; ++g) r.push[g] = static_cast<uint4*>(push->peer_recv[g]);
    r.push_counter = push->counters;
    r.push_world = push->world;
    r.push_rank = push->rank;
    r.push_step = push->step;
  }
  r.out = static_cast<uint8_t*>(p->out);
  r.exp_sums = p->exp_sums;
  r.max_logits = p->max_logits;
  r.tmp_out = static_cast<const uint8_t*>(p->tmp_out);
  r.context_lens = p->context_lens;
  r.tri_m = tri_m;
  r.tri_l = tri_l;
  r.tri_o = tri_o;
  r.S = p->num_seqs;
  r.Hkv = p->num_kv_heads;
  r.eqG = p->query_group_size * p->query_len;
  r.G = p->query_group_size;
  r.sink = p->sink_tokens;
  r.partition_size = p->partition_size;
  r.max_partitions = p->max_partitions;
  const int64_t cap = (int64_t)p->max_blocks_per_seq * p->block_size;
  r.ctx_cap = cap > 0x7fffffff ? 0x7fffffff : (int32_t)cap;
  r.out_stride_seq = p->out_stride_seq;
  r.out_stride_head = p->out_stride_head;
  r.ws_stride_seq = p->ws_stride_seq;
  r.ws_stride_head = p->ws_stride_head;
  r.ws_stride_part = p->ws_stride_part;
  r.tmp_stride_seq = p->tmp_stride_seq;
  r.tmp_stride_head = p->tmp_stride_head;
  r.tmp_stride_part = p->tmp_stride_part;
  r.tmp_stride_row = p->tmp_stride_row;
  const int64_t rows = (int64_t)r.S * r.Hkv * r.eqG;
  if (rows == 0) return PA_OK;
  if (rows > 0x7fffffff) return PA_ERR_TOO_LARGE;   // the kernels index rows with 32 bits
  // one warp per row while a row has at most one chunk of 32 partitions (four rows per CTA); up to
  // four chunks: eight rows per CTA whose further chunks are dealt over the CTA's warps; beyond
  // that sixteen warps per row
  // (the eight-row form only where its CTAs are many: a few long rows, e.g. one GPU's share of a long
  // context split over eight GPUs, are latency-bound and want a CTA each -- 15.6 against 22.9 us per call
  // for 64 rows of 64 partitions; a thousand rows of 40 partitions: 107 us against 125 the other way round)
  DeviceInfo* dev = nullptr;
  const int rc_dev = device_info(&dev);
  if (rc_dev != PA_OK) return rc_dev;
  const bool many_rows = rows >= (int64_t)4 * dev->sm_count;   // eight-row CTAs on half of the SMs at least
  const int wpr = r.max_partitions <= 32 ? 1 : (r.max_partitions <= 32 * pa::kMidChunks && many_rows ? 4 : 16);
  const int64_t blocks = wpr == 16 ? rows : (wpr == 4 ? (rows + pa::kMidRows - 1) / pa::kMidRows : (rows + 3) / 4);
  if (blocks > 0x7fffffff) return PA_ERR_TOO_LARGE;
  // Programmatic dependent launch: the reduce grid may be scheduled while the partition kernel
  // drains; it waits (griddepcontrol.wait) before it reads anything that kernel wrote.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(wpr == 1 ? 128 : (wpr == 4 ? pa::kMidRows * 32 : 512));
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = wpr == 1   ? cudaLaunchKernelEx(&cfg, pa::pa_reduce_kernel<1>, r)
                  : wpr == 4 ? cudaLaunchKernelEx(&cfg, pa::pa_reduce_mid_kernel, r)
                             : cudaLaunchKernelEx(&cfg, pa::pa_reduce_kernel<16>, r);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}

}  // namespace

extern "C" {

int pa_partition_sm100(const PaDecodeParams* params, void* stream) {
  LaunchPlan plan;
  int rc = make_plan(params, &plan);
  if (rc != PA_OK) return rc;
  return launch_partition(plan, static_cast<cudaStream_t>(stream));
}

int pa_reduce_sm100(const PaDecodeParams* params, float* tri_m, float* tri_l, float* tri_o,
                    void* stream) {
  const bool triples = tri_m || tri_l || tri_o;
  if (triples && !(tri_m && tri_l && tri_o)) return PA_ERR_NULL_POINTER;
  int rc = validate(params, false, !triples);
  if (rc != PA_OK) return rc;
  if (triples && (!aligned16(tri_o))) return PA_ERR_ALIGNMENT;
  return launch_reduce(params, tri_m, tri_l, tri_o, static_cast<cudaStream_t>(stream));
}

int pa_decode_sm100(const PaDecodeParams* params, void* stream) {
  LaunchPlan plan;
  int rc = make_plan(params, &plan, true);
  if (rc != PA_OK) return rc;
  rc = validate(params, true, true);
  if (rc != PA_OK) return rc;
  rc = launch_partition(plan, static_cast<cudaStream_t>(stream));
  if (rc != PA_OK || plan.fused) return rc;   // the single-launch kernel has merged the partitions itself
  return launch_reduce(params, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

// ---- the entry point that allocates nothing -------------------------------------------------
// The workspaces of the split-KV pass live in this array.  In host code its name is only a
// handle: the device address is looked up once per device with cudaGetSymbolAddress.
}  // extern "C"
namespace {
static __device__ __align__(256) unsigned char g_noalloc_scratch[PA_NOALLOC_SCRATCH_BYTES];
std::mutex g_noalloc_mutex;
unsigned char* g_noalloc_ptr[kMaxDevices] = {};

int noalloc_scratch_address(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= kMaxDevices) return PA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);  // address on the current device
    if (e != cudaSuccess) return cuda_fail(e);
    if (ptr == nullptr) return PA_ERR_CUDA;
    g_noalloc_ptr[dev] = static_cast<unsigned char*>(ptr);
  }
  *out = g_noalloc_ptr[dev];
  return PA_OK;
}
}  // namespace
extern "C" {

int pa_decode_noalloc_sm100(const PaDecodeParams* params, void* stream) {
  if (!params) return PA_ERR_NULL_POINTER;
  if (params->struct_size != sizeof(PaDecodeParams) || params->abi_version != PA_ABI_VERSION) return PA_ERR_ABI;
  if (params->num_seqs < 0 || params->num_kv_heads <= 0 || params->query_group_size <= 0 ||
      params->query_len <= 0 || params->max_partitions <= 0 || params->head_size != pa::kD)
    return PA_ERR_BAD_SHAPE;
  // rows = S * Hkv * P * eqG, built up factor by factor against the array's capacity so that no
  // product of caller-supplied sizes can overflow (and wrap back under the limit)
  if (params->query_len > 4 || params->query_group_size > 64) return PA_ERR_UNSUPPORTED;
  const int64_t eqG = (int64_t)params->query_group_size * params->query_len;
  const int64_t max_rows = (int64_t)PA_NOALLOC_SCRATCH_BYTES / (8 + pa::kD * 2);
  int64_t rows = eqG;
  const int64_t factors[3] = {params->num_seqs, params->num_kv_heads, params->max_partitions};
  for (const int64_t f : factors) {
    if (f > 0 && rows > max_rows / f) return PA_ERR_TOO_LARGE;
    rows *= f;
  }
  const int64_t f32_bytes = (rows * 4 + 255) / 256 * 256;       // exp_sums, then max_logits
  const int64_t need = 2 * f32_bytes + rows * pa::kD * 2;       // then tmp_out (bf16)
  if (need > (int64_t)PA_NOALLOC_SCRATCH_BYTES) return PA_ERR_TOO_LARGE;
  unsigned char* base = nullptr;
  int rc = noalloc_scratch_address(&base);
  if (rc != PA_OK) return rc;
  PaDecodeParams q = *params;
  q.exp_sums = reinterpret_cast<float*>(base);
  q.max_logits = reinterpret_cast<float*>(base + f32_bytes);
  q.tmp_out = base + 2 * f32_bytes;
  q.ws_stride_part = eqG;
  q.ws_stride_head = eqG * params->max_partitions;
  q.ws_stride_seq = q.ws_stride_head * params->num_kv_heads;
  q.tmp_stride_row = pa::kD;
  q.tmp_stride_part = eqG * pa::kD;
  q.tmp_stride_head = q.tmp_stride_part * params->max_partitions;
  q.tmp_stride_seq = q.tmp_stride_head * params->num_kv_heads;
  return pa_decode_sm100(&q, stream);
}

namespace {
int launch_merge(void* out, int64_t out_stride_row, const float* m, const float* l, const float* o,
                 int32_t num_shards, int32_t num_rows, int32_t head_size, int64_t ml_stride,
                 int64_t o_stride, void* stream) {
  if (!out || !m || !l || !o) return PA_ERR_NULL_POINTER;
  if (num_shards <= 0 || num_rows < 0) return PA_ERR_BAD_SHAPE;
  if (head_size != pa::kD) return PA_ERR_UNSUPPORTED;
  if (!aligned16(o) || (o_stride & 3) || (reinterpret_cast<uintptr_t>(out) & 7u) || (out_stride_row & 3))
    return PA_ERR_ALIGNMENT;
  if (num_rows == 0) return PA_OK;
  const int blocks = (num_rows + 3) / 4;
  pa::pa_merge_triples_kernel<<<blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(out), out_stride_row, m, l, o, num_shards, num_rows, ml_stride, o_stride);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}
}  // namespace

int pa_merge_triples_sm100(void* out, int64_t out_stride_row, const float* m, const float* l,
                           const float* o, int32_t num_shards, int32_t num_rows, int32_t head_size,
                           void* stream) {
  return launch_merge(out, out_stride_row, m, l, o, num_shards, num_rows, head_size, num_rows,
                      (int64_t)num_rows * head_size, stream);
}

int64_t pa_packed_triple_floats(int32_t num_rows, int32_t head_size) {
  if (num_rows < 0 || head_size <= 0) return 0;
  const int64_t ml = ((int64_t)2 * num_rows + 3) & ~(int64_t)3;
  return ml + (int64_t)num_rows * head_size;
}

int pa_merge_packed_triples_sm100(void* out, int64_t out_stride_row, const float* packed,
                                  int32_t num_shards, int32_t num_rows, int32_t head_size, void* stream) {
  if (!packed) return PA_ERR_NULL_POINTER;
  if (num_rows < 0 || head_size <= 0) return PA_ERR_BAD_SHAPE;
  const int64_t stride = pa_packed_triple_floats(num_rows, head_size);
  const int64_t o_off = stride - (int64_t)num_rows * head_size;
  return launch_merge(out, out_stride_row, packed, packed + num_rows, packed + o_off, num_shards, num_rows,
                      head_size, stride, stride, stream);
}

static_assert(sizeof(cudaIpcMemHandle_t) == PA_IPC_HANDLE_BYTES, "handle size is part of the ABI");

int pa_exchange_alloc(int64_t bytes, void** ptr, uint8_t* handle) {
  if (!ptr || !handle) return PA_ERR_NULL_POINTER;
  if (bytes <= 0) return PA_ERR_BAD_SHAPE;
  void* d = nullptr;
  cudaError_t e = cudaMalloc(&d, (size_t)bytes);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaMemset(d, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();   // zeroes are in place before anybody maps it
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d);
  if (e != cudaSuccess) {
    cudaFree(d);
    return cuda_fail(e);
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = d;
  return PA_OK;
}

int pa_exchange_open(const uint8_t* handle, void** ptr) {
  if (!ptr || !handle) return PA_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* d = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&d, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e);
  // One word through a host-side copy: a mapping this device cannot use fails here with an error
  // code (a copy does not poison the context the way a faulting kernel does).
  int32_t word = 0;
  e = cudaMemcpy(&word, d, sizeof(word), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    cudaIpcCloseMemHandle(d);
    return cuda_fail(e);
  }
  *ptr = d;
  return PA_OK;
}

int pa_exchange_close(void* ptr) {
  if (!ptr) return PA_ERR_NULL_POINTER;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? PA_OK : cuda_fail(e);
}

int pa_exchange_free(void* ptr) {
  if (!ptr) return PA_ERR_NULL_POINTER;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? PA_OK : cuda_fail(e);
}

int64_t pa_exchange_bytes(int32_t world_size, int32_t num_rows, int32_t head_size) {
  if (world_size < 1 || num_rows < 0 || head_size != pa::kD) return 0;
  return 2 * (int64_t)world_size * num_rows * pa::kLinesPerRow * 16;
}

int pa_reduce_push_sm100(const PaDecodeParams* params, void* const* peer_recv, const int32_t* counters,
                         int32_t world_size, int32_t rank, int32_t step, void* stream) {
  int rc = validate(params, false, false);
  if (rc != PA_OK) return rc;
  if (!peer_recv || (step == 0 && !counters)) return PA_ERR_NULL_POINTER;
  if (world_size < 1 || world_size > pa::kMaxPeers || rank < 0 || rank >= world_size || step < 0)
    return PA_ERR_BAD_SHAPE;
  for (int g = 0; g < world_size; ++g) {
    if (!peer_recv[g]) return PA_ERR_NULL_POINTER;
    if (!aligned16(peer_recv[g])) return PA_ERR_ALIGNMENT;
  }
  PaDecodeParams q = *params;
  q.out = nullptr;   // this rank's output alone means nothing; the merge writes the result
  PushTarget t = {peer_recv, counters, world_size, rank, step};
  return launch_reduce(&q, nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream), &t);
}

int pa_merge_wait_sm100(void* out, int64_t out_stride_row, const void* recv, int32_t* counters,
                        int32_t* status, int32_t world_size, int32_t step, int32_t num_rows,
                        int32_t head_size, void* stream) {
  if (!out || !recv || (step == 0 && !counters)) return PA_ERR_NULL_POINTER;
  if (world_size < 1 || world_size > pa::kMaxPeers || step < 0 || num_rows < 0) return PA_ERR_BAD_SHAPE;
  if (head_size != pa::kD) return PA_ERR_UNSUPPORTED;
  if (!aligned16(recv) || (reinterpret_cast<uintptr_t>(out) & 7u) || (out_stride_row & 3)) return PA_ERR_ALIGNMENT;
  if (num_rows == 0) return PA_OK;
  pa::MergeWaitParams k;
  memset(&k, 0, sizeof(k));
  k.out = static_cast<uint8_t*>(out);
  k.out_stride_row = out_stride_row;
  k.recv = static_cast<const uint4*>(recv);
  k.counters = counters;
  k.status = status;
  k.world = world_size;
  k.step = step;
  k.num_rows = num_rows;
  // Programmatic dependent launch without a dependency wait in the kernel: every line it reads says
  // by its flag whether it has arrived, so the warps may start polling while the reduce kernel that
  // feeds them (all of whose CTAs are resident by then) still runs.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((num_rows + 3) / 4));
  cfg.blockDim = dim3(128);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, pa::pa_merge_wait_kernel, k);
  if (e != cudaSuccess) return cuda_fail(e);
  e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}

int pa_cache_write_sm100(const PaCacheWriteParams* p, void* stream) {
  if (!p) return PA_ERR_NULL_POINTER;
  if (p->struct_size != sizeof(PaCacheWriteParams) || p->abi_version != PA_ABI_VERSION) return PA_ERR_ABI;
  if (p->num_tokens < 0 || p->num_kv_heads <= 0 || p->block_size <= 0 || p->num_blocks <= 0) return PA_ERR_BAD_SHAPE;
  if (p->head_size != pa::kD) return PA_ERR_UNSUPPORTED;
  if (!p->key || !p->value || !p->slot_mapping || !p->key_cache || !p->value_cache) return PA_ERR_NULL_POINTER;
  const bool fp8 = p->kv_dtype == PA_DT_E4M3FN;
  if (!fp8 && p->kv_dtype != PA_DT_BF16) return PA_ERR_UNSUPPORTED;
  if (fp8 && p->kv_quant_mode != PA_QUANT_NONE && (!p->key_scale || !p->value_scale)) return PA_ERR_NULL_POINTER;
  if (!fp8 && p->kv_quant_mode != PA_QUANT_NONE) return PA_ERR_UNSUPPORTED;
  const bool v_trans = p->v_layout == PA_V_TRANSPOSED;
  if (v_trans && (!fp8 || p->block_size % 16 != 0)) return PA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(p->key) & 7u) || (reinterpret_cast<uintptr_t>(p->value) & 7u) ||
      (p->key_stride_token & 3) || (p->key_stride_head & 3) || (p->value_stride_token & 3) ||
      (p->value_stride_head & 3) || !aligned16(p->key_cache) || ((p->k_stride_block * (fp8 ? 1 : 2)) & 15) ||
      ((p->k_stride_head * (fp8 ? 1 : 2)) & 15))
    return PA_ERR_ALIGNMENT;
  if (p->num_tokens == 0) return PA_OK;
  pa::CacheWriteParams k;
  memset(&k, 0, sizeof(k));
  k.key = static_cast<const uint8_t*>(p->key);
  k.value = static_cast<const uint8_t*>(p->value);
  k.slots = p->slot_mapping;
  k.key_cache = static_cast<uint8_t*>(p->key_cache);
  k.value_cache = static_cast<uint8_t*>(p->value_cache);
  k.k_scale = p->key_scale;
  k.v_scale = p->value_scale;
  k.T = p->num_tokens;
  k.Hkv = p->num_kv_heads;
  k.block_size = p->block_size;
  k.num_blocks = p->num_blocks;
  k.kv_is_fp8 = fp8;
  k.quant_mode = p->kv_quant_mode;
  k.v_trans = v_trans;
  k.vec_ok = aligned16(p->value_cache) && !(p->v_stride_block & 15) && !(p->v_stride_head & 15) &&
             aligned16(p->key) && !(p->key_stride_token & 7) && !(p->key_stride_head & 7);
  k.key_stride_tok = p->key_stride_token;
  k.key_stride_head = p->key_stride_head;
  k.value_stride_tok = p->value_stride_token;
  k.value_stride_head = p->value_stride_head;
  k.kc_stride_block = p->k_stride_block;
  k.kc_stride_head = p->k_stride_head;
  k.vc_stride_block = p->v_stride_block;
  k.vc_stride_head = p->v_stride_head;
  k.ks_stride_block = p->kv_scale_stride_block;
  k.ks_stride_head = p->kv_scale_stride_head;
  k.status = p->status;
  const int64_t pairs = (int64_t)p->num_tokens * p->num_kv_heads;
  // e4m3 caches: a warp per window of 16 tokens and head; bf16 caches: a warp per token and head
  const int64_t warps = fp8 ? ((int64_t)p->num_tokens + 15) / 16 * p->num_kv_heads : pairs;
  const int64_t blocks = (warps + 3) / 4;
  if (blocks > 0x7fffffff) return PA_ERR_TOO_LARGE;
  if (fp8)
    pa::pa_cache_write_fp8_kernel<<<(unsigned)blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(k);
  else
    pa::pa_cache_write_kernel<<<(unsigned)blocks, 128, 0, static_cast<cudaStream_t>(stream)>>>(k);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e);
  return PA_OK;
}

int pa_stream_probe_sm100(const void* a, const void* b, int64_t bytes_each, int32_t* status, void* stream) {
  if (!a || !b) return PA_ERR_NULL_POINTER;
  if (bytes_each <= 0 || bytes_each % pa::kProbeSlotBytes != 0) return PA_ERR_BAD_SHAPE;
  if (!aligned16(a) || !aligned16(b)) return PA_ERR_ALIGNMENT;
  DeviceInfo* dev = nullptr;
  int rc = device_info(&dev);
  if (rc != PA_OK) return rc;
  cudaError_t e = cudaFuncSetAttribute(pa::pa_stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       pa::kProbeSmem);
  if (e != cudaSuccess) return cuda_fail(e);
  pa::pa_stream_probe_kernel<<<dev->sm_count, pa::kProbeWarps * 32, pa::kProbeSmem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), (long long)(bytes_each / pa::kProbeSlotBytes), status);
  e = cudaGetLastError();
  return e != cudaSuccess ? cuda_fail(e) : PA_OK;
}

int pa_query_launch_sm100(const PaDecodeParams* params, int32_t* grid_ctas, int32_t* cta_threads,
                          int32_t* smem_bytes, int32_t* ring_stages) {
  LaunchPlan plan;
  int rc = make_plan(params, &plan, true);   // what pa_decode_sm100 would launch
  if (rc != PA_OK) return rc;
  if (grid_ctas) *grid_ctas = plan.grid;
  if (cta_threads) *cta_threads = plan.warps * 32;
  if (smem_bytes) *smem_bytes = plan.smem;
  if (ring_stages) *ring_stages = plan.kp.num_stages;
  return PA_OK;
}

const char* pa_strerror(int status) {
  switch (status) {
    case PA_OK: return "ok";
    case PA_ERR_NULL_POINTER: return "a required pointer is NULL";
    case PA_ERR_BAD_SHAPE: return "a size is zero, negative or inconsistent";
    case PA_ERR_UNSUPPORTED: return "shape, dtype or layout not supported by the sm_100a kernels";
    case PA_ERR_ALIGNMENT: return "a pointer or stride is not aligned as the bulk copies require";
    case PA_ERR_CUDA: return "a CUDA runtime call failed (see pa_last_cuda_error)";
    case PA_ERR_ABI: return "PaDecodeParams.struct_size / abi_version do not match this library";
    case PA_ERR_TOO_LARGE: return "a size exceeds a fixed limit of the library";
    default: return "unknown status";
  }
}

int pa_last_cuda_error(void) { return g_last_cuda_error; }

int pa_abi_version(void) { return PA_ABI_VERSION; }

}  // extern "C"
