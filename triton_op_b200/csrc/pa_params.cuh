// Kernel-side parameter block of the partition kernels (filled by the host entry points
// from PaDecodeParams after validation).
#pragma once

#include <stdint.h>

namespace pa {

constexpr int kD = 128;  // head size, the only one the reference's test matrix uses

struct KernelParams {
  // tensors
  const uint8_t* q;            // query rows, q_dtype
  const uint8_t* k;            // key cache
  const uint8_t* v;            // value cache
  const int32_t* block_tables;
  const int32_t* context_lens;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* alibi;          // [Hkv * G] slopes or null
  float* exp_sums;
  float* max_logits;
  uint8_t* tmp_out;            // bf16
  int32_t* status;             // may be null
  unsigned long long* trace;   // tuning aid: per-role clock stamps of CTA 0; null in normal operation
  // single-launch decode (the partition kernel also merges the partitions): the final output, the
  // optional sink logits and one counter per (sequence, kv head), zero between launches
  uint8_t* out;                // bf16 [S, Hkv*eqG, D]; null unless the launch merges
  const float* sink;           // [Hkv*G] or null
  int32_t* merge_counters;     // [S*Hkv]
  int64_t out_stride_seq, out_stride_head;   // elements

  // sizes
  int32_t S, Hkv, G, L, eqG;
  int32_t block_size, num_blocks, max_blocks_per_seq;
  int32_t partition_size, max_partitions;
  int32_t pages_per_partition; // partition_size / block_size (small blocks)
  int32_t ctx_cap;             // max_blocks_per_seq * block_size

  // strides in BYTES for q / k / v, in elements for the fp32 tensors and tmp_out
  int64_t q_stride_seq, q_stride_head;
  int64_t k_stride_block, k_stride_head;
  int64_t v_stride_block, v_stride_head;
  int64_t bt_stride_seq;
  int64_t q_scale_stride_seq;
  int64_t kvs_stride_block, kvs_stride_head;
  int64_t ws_stride_seq, ws_stride_head, ws_stride_part;
  int64_t tmp_stride_seq, tmp_stride_head, tmp_stride_part, tmp_stride_row;

  int32_t q_quant_mode, kv_quant_mode;
  int32_t q_is_fp8;            // query rows are e4m3fn (1 byte per element) instead of bf16
  int32_t v_trans;             // value cache is [NB, Hkv, bs/16, D, 16]: every 16 tokens a [D][16] run of 2 KB
  float softmax_scale;

  // shared-memory carve (byte offsets from the dynamic shared base) and ring geometry
  int32_t num_stages;          // ring depth per warp
  int32_t off_seq_offsets;     // int32[S+1]: exclusive prefix sum of partitions per sequence
  int32_t off_seq_ctx;         // int32[S]: clamped context lengths
  int32_t off_q;               // query staging (ring of tiles)
  int32_t off_p;               // probability tiles (tcgen05 kernel)
  int32_t off_ring;            // stage ring (mma.sync kernel) / K ring (tcgen05 kernel)
  int32_t off_vring;           // V ring (tcgen05 kernel)
  int32_t num_vstages;         // V ring depth (tcgen05 kernel)
  int32_t num_row_blocks;      // ceil(eqG / rows per work item) (tcgen05 kernel)
  int32_t early_start;         // build the partition index before the dependency wait (checked after it)
  int32_t team_size;           // single-launch form: CTAs per team (divides Hkv and the grid)
  int32_t off_stash;           // PAIR form of the tcgen05 kernel: where a partition's first half waits for its second
};

// Fixed head of the shared-memory carve: mbarriers and the scan scratch.
constexpr int kMaxStages = 12;
constexpr int kMaxWarps = 16;
constexpr int kBarBytesPerWarp = (kMaxStages + 1) * 8;  // ring slots + query barrier
constexpr int kSmemHeadBytes = kMaxWarps * kBarBytesPerWarp + 128 /* scan scratch */;
static_assert(kSmemHeadBytes % 16 == 0, "carve must stay 16-byte aligned");

}  // namespace pa
