/*
 * pa_decode_sm100.h -- C ABI of the B200 (sm_100a) paged-attention decode operator.
 *
 * The library replaces one operator of yanguahe/triton_op: the split-KV paged-attention
 * decode ("v2") and its cross-partition log-sum-exp reduce.  Every entry point takes plain
 * device pointers, sizes and strides; nothing here knows about torch.  All pointers are
 * device pointers unless stated otherwise, are borrowed for the duration of the call only,
 * and nothing is allocated or freed by the library.  Every function returns PA_OK (0) or a
 * negative PaStatus, never throws, never prints, never exits.  Calls are asynchronous on the
 * given stream and re-entrant (the only global state is a per-device attribute cache).
 *
 * Reference interface replaced (paths inside yanguahe/triton_op):
 *   pa_decode_triton_gluon_fp8.py:1659-1897   paged_attention_decode        -> pa_decode_sm100
 *   pa_decode_triton_gluon_fp8.py:514-1002    paged_attention_decode_v2_gluon_fp8 (block 16/64)
 *   pa_decode_triton_gluon_fp8.py:27-501      ..._large_block_fp8 (block 1024) -> pa_partition_sm100
 *   pa_decode_triton_gluon_fp8.py:1187-1333   paged_attention_decode_v2_reduce_kernel -> pa_reduce_sm100
 *   pa_decode_gluon.py:655-756                bf16-KV paged_attention_decode (same entry, kv_dtype = PA_DT_BF16)
 */
#ifndef PA_DECODE_SM100_H
#define PA_DECODE_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_ABI_VERSION 3

typedef enum PaStatus {
  PA_OK = 0,
  PA_ERR_NULL_POINTER = -1,   /* a required pointer is NULL */
  PA_ERR_BAD_SHAPE = -2,      /* a size is zero/negative or sizes disagree */
  PA_ERR_UNSUPPORTED = -3,    /* shape or dtype combination the kernels do not cover */
  PA_ERR_ALIGNMENT = -4,      /* a pointer or stride breaks the 16-byte rule of the bulk copies */
  PA_ERR_CUDA = -5,           /* a CUDA runtime call failed (see pa_last_cuda_error) */
  PA_ERR_ABI = -6,            /* struct_size does not match this library */
  PA_ERR_TOO_LARGE = -7       /* a size exceeds a stated fixed limit */
} PaStatus;

typedef enum PaDType {
  PA_DT_BF16 = 0,
  PA_DT_E4M3FN = 1            /* OCP e4m3fn, max 448 */
} PaDType;

/* Quantisation mode of a scale argument; the values are the reference's own
 * (pa_decode_triton_gluon_fp8.py:1752-1790). */
typedef enum PaQuantMode {
  PA_QUANT_NONE = -1,         /* no scale */
  PA_QUANT_PER_TENSOR = 0,    /* pointer to ONE fp32 in device memory */
  PA_QUANT_PER_TOKEN = 1      /* [num_blocks, num_kv_heads, block_size] fp32, last dim contiguous */
} PaQuantMode;

/* Value-cache layouts (pa_decode_triton_gluon_fp8.py:1792-1799). */
typedef enum PaVLayout {
  PA_V_NORMAL = 0,            /* [num_blocks, num_kv_heads, head_size, block_size] */
  PA_V_TRANSPOSED = 1         /* [num_blocks, num_kv_heads, block_size/x, head_size, x] */
} PaVLayout;

/* Bits the kernels may OR into *status (device int32, optional). 0 means a clean run. */
#define PA_DEV_WAIT_TIMEOUT   1  /* a bounded wait on a bulk copy ran out; results are undefined */
#define PA_DEV_BAD_PAGE_ID    2  /* a block-table entry was outside [0, num_blocks); it was clamped */
#define PA_DEV_CTX_TOO_LONG   4  /* a context length exceeded max_blocks_per_seq*block_size; it was clamped */

/* Size, in uint64 words, of the optional trace buffer: [8 roles][item < 64][4 points]. */
#define PA_TRACE_WORDS (8 * 64 * 4)

/*
 * One decode call.  Symbols: S num_seqs, Hkv num_kv_heads, G query heads per kv head,
 * L query_len (MTP), eqG = L*G, D head_size (128), bs block_size, P max_partitions,
 * x = 16/itemsize(kv).
 *
 * Row order inside one kv head follows the reference (test_pa_mtp.py:793-822): query row
 * r = t*G + g holds new token t (0..L-1) of head g; row r attends key j iff
 * (L-1-t) + j < context_len (pa_decode_triton_gluon_fp8.py:915-920).
 */
typedef struct PaDecodeParams {
  uint32_t struct_size;        /* = sizeof(PaDecodeParams) */
  uint32_t abi_version;        /* = PA_ABI_VERSION */

  /* tensors */
  void* out;                   /* [S, Hkv*eqG, D] out_dtype; written in place */
  const void* query;           /* [S, Hkv*eqG, D] q_dtype; last dim contiguous */
  const void* key_cache;       /* [NB, Hkv, D/x, bs, x]; the last three dims contiguous */
  const void* value_cache;     /* PA_V_NORMAL: [NB, Hkv, D, bs]; the last two dims contiguous */
  const int32_t* block_tables; /* [S, max_blocks_per_seq] */
  const int32_t* context_lens; /* [S] */
  const float* query_scale;    /* per-tensor [1] / per-token [S, Hkv*eqG]; NULL when PA_QUANT_NONE */
  const float* key_scale;      /* per-tensor [1] / per-token [NB, Hkv, bs]; NULL when PA_QUANT_NONE */
  const float* value_scale;    /* same shape as key_scale */
  const float* alibi_slopes;   /* [Hkv*G] or NULL */
  const float* sink_tokens;    /* [Hkv*G] or NULL: one sink logit per query head; the reduce adds
                                * exp(sink - M) to a row's sum of weights (the reference's unused Gluon
                                * reduce, pa_decode_triton_gluon_fp8.py:1117-1123).  Not applied to triples. */

  /* workspaces, caller-owned (reference: torch.zeros at pa_decode_triton_gluon_fp8.py:1729-1733).
   * They need not be zeroed: every partition the reduce reads is written by the partition kernel. */
  float* exp_sums;             /* [S, Hkv, P, eqG] fp32 */
  float* max_logits;           /* [S, Hkv, P, eqG] fp32 */
  void* tmp_out;               /* [S, Hkv, P, eqG, D] out_dtype, already divided by exp_sums */
  int32_t* status;             /* optional device int32, OR-ed with PA_DEV_* bits */
  uint64_t* trace;             /* optional tuning aid: device buffer of PA_TRACE_WORDS uint64 that
                                * receives SM-clock stamps of CTA 0's pipeline roles; NULL normally.
                                * Only a library built with -DPA_TRACE_BUILD writes it (pages of 16 or 1024 tokens);
                                * the default build ignores it. */
  int32_t* merge_counters;     /* optional [S*Hkv] device int32, ZERO before the first call and left zero by
                                * every call that completes.  With it and tune_fuse = 1, pa_decode_sm100 runs as
                                * ONE launch where it can (e4m3fn KV, partition 256, L*G <= 8, P <= 32, no
                                * ALiBi): work items are numbered so that a CTA computes all partitions of
                                * most (sequence, kv head) row sets and merges them itself when the last one is
                                * stored; a set whose partitions are spread over several CTAs is merged by the
                                * CTA that holds its first partition, and the others add their partition counts
                                * here.  No second launch (the reference always pays that launch,
                                * pa_decode_triton_gluon_fp8.py:1862-1887).  Same bits as the two-launch form.
                                * It is not the default: the numbering that keeps a set inside one CTA reads
                                * the cache measurably slower than the round-robin numbering of the two-launch
                                * form, by more than the second launch costs.  One array serves one call at a
                                * time; after a call that reported PA_DEV_WAIT_TIMEOUT clear it again. */

  /* sizes */
  int32_t num_seqs;            /* S */
  int32_t num_kv_heads;        /* Hkv */
  int32_t query_group_size;    /* G */
  int32_t query_len;           /* L, 1..4 */
  int32_t head_size;           /* D, must be 128 */
  int32_t block_size;          /* bs: 16, 64 or 1024 */
  int32_t num_blocks;          /* NB */
  int32_t max_blocks_per_seq;  /* columns of block_tables */
  int32_t partition_size;      /* tokens per split-KV partition of the workspaces: 256 (reference constant), or 512
                                * (e4m3fn KV, L*G <= 16, no ALiBi: the tcgen05 kernel, two 256-token work items per
                                * partition merged in shared memory), or a multiple of 32 up to 512 with 16-token pages
                                * (the mma.sync kernel; also what tune_warps = 4 / 8 asks for) */
  int32_t max_partitions;      /* P, the partition extent of the workspaces */

  /* strides, in ELEMENTS of the tensor's dtype */
  int64_t out_stride_seq, out_stride_head;
  int64_t q_stride_seq, q_stride_head;
  int64_t k_stride_block, k_stride_head;
  int64_t v_stride_block, v_stride_head;
  int64_t bt_stride_seq;
  int64_t q_scale_stride_seq;              /* per-token query scale only */
  int64_t kv_scale_stride_block, kv_scale_stride_head;  /* per-token kv scales only */
  int64_t ws_stride_seq, ws_stride_head, ws_stride_part;                   /* exp_sums / max_logits */
  int64_t tmp_stride_seq, tmp_stride_head, tmp_stride_part, tmp_stride_row;/* tmp_out */

  /* dtypes and modes */
  int32_t q_dtype;             /* PaDType */
  int32_t kv_dtype;            /* PaDType */
  int32_t out_dtype;           /* PaDType; PA_DT_BF16 */
  int32_t q_quant_mode;        /* PaQuantMode */
  int32_t kv_quant_mode;       /* PaQuantMode */
  int32_t v_layout;            /* PaVLayout */
  float softmax_scale;

  /* 0 = library default.  tune_warps: consumer warps per CTA; tune_stages: ring depth per
   * warp (K ring of the tcgen05 kernel); tune_vstages: V ring depth of the tcgen05 kernel;
   * tune_ctas: grid size.  For benchmarking sweeps; results do not depend on them. */
  int32_t tune_warps, tune_stages, tune_ctas, tune_vstages;
  int32_t tune_fuse;           /* 1: run pa_decode_sm100 as ONE launch where merge_counters and the shape allow it;
                                * 1 + T: the same with teams of T CTAs sharing the kv heads of a (sequence, partition)
                                * row (T divides num_kv_heads; default: the largest T that also divides the grid);
                                * 0 (default): partition kernel, then reduce kernel (measured faster, see the field) */
  int32_t tune_early;          /* -1: the tcgen05 kernel reads nothing before its dependency wait; 0 (default): it builds
                                * its partition index from the context lengths before the wait and checks it
                                * against them after it */
} PaDecodeParams;

/* Partition kernel followed by the reduce kernel on `stream` (a cudaStream_t); one launch that
 * does both when `merge_counters` is given and the shape allows it (see the field). */
int pa_decode_sm100(const PaDecodeParams* params, void* stream);

/* The partition kernel alone: fills exp_sums / max_logits / tmp_out, leaves `out` untouched. */
int pa_partition_sm100(const PaDecodeParams* params, void* stream);

/*
 * The reduce kernel alone: merges the partitions in the workspaces into `out`.
 * When tri_m / tri_l / tri_o are all non-NULL it ALSO stores the merged (max, sum, normalised
 * output) triple of every output row in fp32 -- the unit the multi-GPU merge exchanges:
 *   tri_m, tri_l: [S*Hkv*eqG]; tri_o: [S*Hkv*eqG, D].  Row index = seq*(Hkv*eqG) + head*eqG + r.
 * `out` may be NULL in that case.
 */
int pa_reduce_sm100(const PaDecodeParams* params, float* tri_m, float* tri_l, float* tri_o,
                    void* stream);

/*
 * Cross-shard log-sum-exp merge (no counterpart in the single-GPU reference; it is the
 * reduce of pa_decode_triton_gluon_fp8.py:1187-1333 applied across GPUs instead of partitions).
 *   m, l : [num_shards, num_rows] fp32      o : [num_shards, num_rows, head_size] fp32
 *   out  : [num_rows, head_size] bf16 with row stride out_stride_row (elements)
 *   out[r] = sum_g o[g,r]*l[g,r]*exp(m[g,r]-M[r]) / sum_g l[g,r]*exp(m[g,r]-M[r]),  M = max_g m
 * Shards with l == 0 contribute nothing.
 */
int pa_merge_triples_sm100(void* out, int64_t out_stride_row, const float* m, const float* l,
                           const float* o, int32_t num_shards, int32_t num_rows, int32_t head_size,
                           void* stream);

/*
 * The same merge on triples packed for a single all-gather (no counterpart in the reference).
 * One shard's message is pa_packed_triple_floats(num_rows, head_size) floats:
 *   m[num_rows] | l[num_rows] | padding to a multiple of 4 floats | o[num_rows][head_size]
 * (point pa_reduce_sm100's tri_m / tri_l / tri_o into such a buffer); `packed` holds
 * num_shards messages back to back, as an all-gather leaves them.
 */
int64_t pa_packed_triple_floats(int32_t num_rows, int32_t head_size);
int pa_merge_packed_triples_sm100(void* out, int64_t out_stride_row, const float* packed,
                                  int32_t num_shards, int32_t num_rows, int32_t head_size, void* stream);

/*
 * The same exchange over NVLink peer stores instead of an all-gather (no counterpart in the
 * reference).  Every rank owns a receive buffer of pa_exchange_bytes(world_size, num_rows,
 * head_size) bytes, zero before the first step and mapped into its peers (pa_exchange_alloc /
 * pa_exchange_open below, or any other peer mapping); `peer_recv[g]` is rank g's buffer as this
 * process's device addresses it (entry `rank` = the local one).  It holds [2][world_size]
 * [num_rows] triples as 16-byte lines {value, step, value, step}: the step number travels inside
 * every 8-byte half, so the data needs no fence and no separate flag.  One decode step = 1, 2, ...:
 *   pa_reduce_push_sm100  pa_reduce_sm100 without the bf16 output: stores each row's (m, l, o) into
 *                         slot [step & 1][rank] of every rank's buffer;
 *   pa_merge_wait_sm100   merges the world_size triples of each row from the local buffer into
 *                         `out`, waiting, bounded (about a second, then PA_DEV_WAIT_TIMEOUT in
 *                         *status and no output for that row), for lines not yet of this step.
 * Ranks must call both once per step with the same step sequence.  step = 0 in both calls means
 * "the next step, counted on the device": `counters` is then two local device int32 words, zero
 * before the first call ([0] scratch, [1] = steps merged so far), and the arguments are the
 * same every step, so the pair can be captured in a CUDA graph.
 */
int64_t pa_exchange_bytes(int32_t world_size, int32_t num_rows, int32_t head_size);
int pa_reduce_push_sm100(const PaDecodeParams* params, void* const* peer_recv, const int32_t* counters,
                         int32_t world_size, int32_t rank, int32_t step, void* stream);
int pa_merge_wait_sm100(void* out, int64_t out_stride_row, const void* recv, int32_t* counters,
                        int32_t* status, int32_t world_size, int32_t step, int32_t num_rows,
                        int32_t head_size, void* stream);

/*
 * Exchange memory that peers can map.  Such a buffer must be an allocation of its own (a handle
 * names a whole allocation), and a peer must open the handle WITH ITS OWN DEVICE CURRENT: the
 * mapping belongs to the opening device's address space, and kernels of another device of the
 * same process cannot use it.
 *   pa_exchange_alloc  allocates `bytes` of zeroed device memory on the current device and writes
 *                      its 64-byte inter-process handle;
 *   pa_exchange_open   maps a peer process's allocation into the current device (enabling peer
 *                      access to the exporting device if needed) and reads one word of it through
 *                      a host-side copy, so an unusable mapping is an error code here, not a
 *                      fault in a kernel later;
 *   pa_exchange_close  unmaps what pa_exchange_open returned (before the owner frees it);
 *   pa_exchange_free   frees what pa_exchange_alloc returned.
 */
#define PA_IPC_HANDLE_BYTES 64
int pa_exchange_alloc(int64_t bytes, void** ptr, uint8_t* handle);
int pa_exchange_open(const uint8_t* handle, void** ptr);
int pa_exchange_close(void* ptr);
int pa_exchange_free(void* ptr);

/*
 * KV-cache write side (the step before the decode path; the reference builds its caches offline
 * with torch permutes, test_pa_mtp.py:109-172, and quantises them per token with
 * quantize_kv_cache_symmetric, :294-369): quantise T new key / value tokens and scatter them
 * into the paged layouts above.  Token t goes to slot slots[t] = block * block_size + offset;
 * negative slots are skipped.
 *   kv_quant_mode PA_QUANT_NONE       bf16 caches, bits copied
 *                 PA_QUANT_PER_TENSOR e4m3fn caches, q = x / *key_scale (read)
 *                 PA_QUANT_PER_TOKEN  e4m3fn caches, scale = max(amax(vector)/448, 1e-12) is WRITTEN to
 *                                     key_scale / value_scale [NB, Hkv, bs, 1], q = x / scale
 * Division is IEEE, conversion round-to-nearest-even, so in-range bytes equal torch's
 * (x.float() / scale).to(torch.float8_e4m3fn); values beyond +-448 (possible with a static
 * per-tensor scale) saturate, where torch's cast would store NaN.
 */
typedef struct PaCacheWriteParams {
  uint32_t struct_size;        /* = sizeof(PaCacheWriteParams) */
  uint32_t abi_version;        /* = PA_ABI_VERSION */
  const void* key;             /* [T, Hkv, D] bf16, last dim contiguous */
  const void* value;           /* [T, Hkv, D] bf16 */
  const int64_t* slot_mapping; /* [T] */
  void* key_cache;             /* [NB, Hkv, D/x, bs, x] */
  void* value_cache;           /* [NB, Hkv, D, bs] or transposed [NB, Hkv, bs/16, D, 16] */
  float* key_scale;            /* see kv_quant_mode */
  float* value_scale;
  int32_t* status;             /* optional; PA_DEV_BAD_PAGE_ID when a slot lies outside the pool */
  int32_t num_tokens;          /* T */
  int32_t num_kv_heads;
  int32_t head_size;           /* 128 */
  int32_t block_size;
  int32_t num_blocks;
  int32_t kv_dtype;            /* PaDType */
  int32_t kv_quant_mode;       /* PaQuantMode */
  int32_t v_layout;            /* PaVLayout */
  int64_t key_stride_token, key_stride_head;       /* elements */
  int64_t value_stride_token, value_stride_head;
  int64_t k_stride_block, k_stride_head;           /* caches, elements */
  int64_t v_stride_block, v_stride_head;
  int64_t kv_scale_stride_block, kv_scale_stride_head;
} PaCacheWriteParams;

int pa_cache_write_sm100(const PaCacheWriteParams* params, void* stream);

/* Bytes of dynamic shared memory and the grid the partition kernel would use for `params`
 * (host-only query, launches nothing).  Any output pointer may be NULL. */
int pa_query_launch_sm100(const PaDecodeParams* params, int32_t* grid_ctas, int32_t* cta_threads,
                          int32_t* smem_bytes, int32_t* ring_stages);

/*
 * pa_decode_sm100 for callers that must not allocate device memory.  (No counterpart in the
 * reference, which allocates its three workspaces with torch.zeros on every call.)
 *
 * Who needs it: an inference runtime that has handed the whole GPU memory to its own pool, a
 * plugin running inside somebody else's process where cudaMalloc may fail or stall behind other
 * streams, or code that may run while a stream is being captured, when allocating is not allowed.
 * Such a caller passes inputs and `out` as usual and leaves exp_sums / max_logits / tmp_out
 * NULL (they are ignored): the split-KV workspaces live in a fixed array inside the library,
 * PA_NOALLOC_SCRATCH_BYTES of device memory that every GPU holds from the moment it loads the
 * library until the process exits.
 *
 * Limits and rules:
 *  - num_seqs * num_kv_heads * max_partitions * (query_len * query_group_size) rows must fit:
 *    264 bytes per row (two fp32 + 128 bf16) plus alignment, at most PA_NOALLOC_SCRATCH_BYTES;
 *    a larger problem returns PA_ERR_TOO_LARGE and launches nothing.
 *  - The first call on each device looks up the array's device address (with that device
 *    current).  Make that first call outside any stream capture.
 *  - All calls on one device share the array and it keeps the last call's contents.  Nothing
 *    in it has to start at zero (the partition kernel writes every element the reduce reads),
 *    but two calls that overlap on the GPU -- different streams, or different host threads --
 *    race on it: serialise them.
 *  - Neither this function nor anything it calls allocates or frees memory.
 */
#define PA_NOALLOC_SCRATCH_BYTES (16u << 20)
int pa_decode_noalloc_sm100(const PaDecodeParams* params, void* stream);

/*
 * Measurement aid (no counterpart in the reference): reads `bytes_each` bytes (a multiple of
 * 8192) from each of the two device regions `a` and `b` with the partition kernels' own copy
 * mechanism (2 KB bulk copies into shared-memory rings, one persistent CTA per SM) and computes
 * nothing.  Its duration is the read-only streaming ceiling the benchmark quotes the decode
 * call against.  `status` (optional) receives PA_DEV_WAIT_TIMEOUT if a bounded wait ran out.
 */
int pa_stream_probe_sm100(const void* a, const void* b, int64_t bytes_each, int32_t* status, void* stream);

/* Static string for a PaStatus. */
const char* pa_strerror(int status);

/* cudaError_t of the last failing CUDA call made by this library on the calling thread. */
int pa_last_cuda_error(void);

/* PA_ABI_VERSION the library was built with. */
int pa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* PA_DECODE_SM100_H */
