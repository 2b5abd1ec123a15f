// Split-KV partition kernel on the tcgen05 tensor cores: e4m3fn KV cache, pages of 16, 64 or
// 1024 tokens, 256-token partitions, any query group (rows are taken 4, 8 or 16 at a time).
//
// Same contract as paged_attention_decode_v2_gluon_fp8 / ..._large_block_fp8 of
// yanguahe/triton_op (pa_decode_triton_gluon_fp8.py:514-1002, :27-501): per (sequence, kv head,
// partition) it stores m = max_j s_j, l = sum_j exp(s_j - m) and o = sum_j exp(s_j - m) v_j / l.
//
// Why this shape.  sm_100a has no native fp8 mma.sync: an e4m3 mma.sync is expanded into
// byte->half converts plus f16 tiles, and those converts (quarter-rate pipe) cap a register-level
// kernel near 65 % of HBM bandwidth.  tcgen05.mma kind::f8f6f4 multiplies e4m3 operands straight
// out of shared memory, so here no KV byte ever passes through a register:
//
//   bulk copy (contiguous runs of a page)  ->  shared memory  ->  tensor core.
//
// The tiles are transposed so that the long axis fills M = 128:
//   S^T[128 tokens, N] = K[128 tokens, 128 d] . Q^T        (4 instructions, K = 32 each)
//   O^T[128 d,      N] = V^T[128 d, 256 tokens] . P^T      (8 instructions)
// with N = 2 x (query rows of the work item): the bf16 query and the probabilities are split
// into two e4m3 numbers each (x = hi + lo/16, 8 significant bits), so the products are exact and
// the result has bf16-level precision although the tensor core only sees e4m3.
//
// The paged layouts are already what the tensor core wants (K-major "core matrices" of 8 rows
// x 16 bytes, no swizzle), so cache bytes are copied verbatim and the descriptors do the gather:
//   K cache [D/16][bs tok][16 B]: rows = tokens.
//     bs = 16: a page of one head is one 2 KB run; pages sit 2 KB apart in the slot, and one
//       M = 128 instruction takes tokens tg*8..tg*8+7 of each of the 16 pages (2048 B between
//       8-row groups, 256 B between the two 16-byte K units); tg = 0, 1 covers the partition.
//     bs >= 64: every (page, 16-dim chunk) run is copied to [chunk][256 tok][16 B], so a tile is
//       128 consecutive tokens (128 B between groups, 4096 B between K units).
//   V cache [D][bs tok]: rows = head dims, the two K units of an instruction are 32 consecutive
//     tokens: two pages of 16 (2048 B apart), or 32 bytes of a longer row.
//
// One CTA per SM, persistent over work items (an item = one partition of one kv head and one
// block of query rows), 16 warps with fixed roles joined by mbarriers:
//   warps 0-11   three softmax + epilogue groups of four warps; a thread = one TMEM lane (a
//                token of S^T, a head dim of O^T).  Group g takes the CTA's items g, g+3, ...
//                and owns its own S^T / O^T columns and P^T tile, so the per-item latency chain
//                of a group overlaps the chains of the other groups.
//   warp 12      tcgen05.mma issue (one elected lane) and TMEM allocation
//   warp 13/14   K / V producers (bulk copies; page ids prefetched an item ahead).  Issuing a bulk
//                copy costs a warp 75-90 cycles and the copies of one warp go out one after the
//                other, so the 16 + 16 copies of an item need two warps.
//   warp 15      query producer: bf16 -> hi/lo e4m3 tile in the B-operand layout, the rows' factors, and
//                what else the softmax groups need per item (the item itself; the item's per-token
//                scales by bulk copy where a page's scales are contiguous): see q_slot_bytes
// K and V have their own rings of 32 KB slots.  Every wait is bounded and reports
// PA_DEV_WAIT_TIMEOUT.
#pragma once

#include "pa_common.cuh"
#include "pa_params.cuh"
#include "pa_partition_fp8.cuh"  // build_partition_index, kPageBytes
#include "pa_reduce.cuh"         // merge_row_one_chunk
#include "pa_tcgen05.cuh"

#include <type_traits>
#include <cuda.h>  // CUtensorMap (type only; the encoder is looked up at run time by the host code)
#include "../../include/pa_decode_sm100.h"

namespace pa {
namespace tc {

constexpr int kItemTokens = 256;
constexpr int kHalfSlot = kItemTokens * kD;         // 32 KB: K (or V) of one item
constexpr int kNG = 3;                              // softmax groups
constexpr int kLag = kNG - 1;                       // P.V trails QK^T by this many items in the issue loop
constexpr int kThreads = (4 * kNG + 4) * 32;
constexpr int kMaxSlots = 4;
// The query ring has its own depth and barriers (a slot is a few KB, so the producer may run
// further ahead than the 32 KB K slots allow).
constexpr int kQSlots = 4;
constexpr int kWarpMma = 4 * kNG, kWarpK = 4 * kNG + 1, kWarpV = 4 * kNG + 2, kWarpQ = 4 * kNG + 3;
// Single-launch form (FUSE): polls of a softmax group that waits for the other partitions of a
// (sequence, kv head) before it merges them (each with a 64 ns sleep: about a second in all).
constexpr uint32_t kSetPolls = 1u << 23;

// ---- geometry that depends on the rows per work item (QR = 4, 8 or 16) ---------------------------
// Row q of the item sits in tile row / TMEM column q (hi half) and QR + q (lo half).
__host__ __device__ constexpr int mma_n(int qr) { return qr <= 8 ? 16 : 2 * qr; }
__host__ __device__ constexpr int q_tile_bytes(int qr) { return mma_n(qr) * kD; }  // [row block][8 chunks][8 rows][16 B]
// With 16 rows the hi and lo halves are tiles of their own (N = 16 each), and the tensor core
// adds the two products into the same accumulator columns: lo is then stored unscaled (x = hi +
// lo, lo down to e4m3's subnormal step, 2^-9 against a row maximum of at least 128), the
// accumulator has half the columns, and what a softmax thread loads from it is the logit (or
// the output) itself.  With 4 or 8 rows both halves share one N = 16 tile and are combined in
// registers (value = hi column + lo column / 16).
__host__ __device__ constexpr bool sums_in_tensor_core(int qr) { return qr == 16; }
__host__ __device__ constexpr int acc_n(int qr) { return sums_in_tensor_core(qr) ? qr : mma_n(qr); }
// Query slot.  Its first part belongs to a query TILE (the tile and 16 floats of per-row scales),
// the rest to a work ITEM (16-byte header: which slot holds the item's tile).  Consecutive items
// with the same query rows share a tile, so the two parts are used as two rings with their own
// counters.
constexpr int kQHdr = 64;    // offset of the item header behind the tile
constexpr int kQSlope = 80;  // offset of the tile's 16 ALiBi slopes (base-2 logit domain) behind the tile
// With per-token scales and pages of 64 tokens or more, the item part also holds the item's 256
// key scales and 256 value scales (2 KB), brought in by bulk copies of the query producer: the
// scales of a page are contiguous there.  (With 16-token pages they would be 32 copies of 64
// bytes per item; the softmax threads fetch their own tokens' scales from global memory instead.)
#ifndef PA_STAGED_SCALES
#define PA_STAGED_SCALES 1
#endif
// The item part of a slot also carries the work item itself (32 bytes: the query producer has
// decoded it anyway), so that the softmax groups need no cursor of their own -- unless they
// fetch per-token scales themselves and must know their items two ahead.
// The softmax's exponent offsets are computed once per row by one thread (1) or by every thread
// from the four warps' maxima (0).
#ifndef PA_ITEM_FROM_SLOT
#define PA_ITEM_FROM_SLOT 1
#endif
constexpr int kQItem = kQSlope + 64;        // offset of the item (8 ints) behind the tile
constexpr int kQTokScales = kQItem + 32;    // offset of the item's token scales behind the tile
__host__ __device__ constexpr bool staged_token_scales(int block_size, bool per_token) {
  return PA_STAGED_SCALES && per_token && block_size >= 64;
}
__host__ __device__ constexpr int q_slot_bytes(int qr, bool staged_scales) {
  return q_tile_bytes(qr) + kQTokScales + (staged_scales ? 2 * kItemTokens * 4 : 0);
}
// P^T tile of one item, an MN-major operand: the 16 tile rows (N) of one token are 16 consecutive bytes, the
// tokens (K) of an 8-token core matrix are 16 bytes apart and core matrices follow one another,
// so token t of the item sits at t * 16 and a softmax thread stores its token's bytes of a
// chunk of rows with one vector store.  16-row items have a tile for the hi rows and one for the lo rows.
constexpr int kPLbo = 128;                          // between 8-token core matrices (along K)
constexpr int kPSbo = 4096;                         // between 16-row blocks (there is one per tile)
__host__ __device__ constexpr int p_step_bytes(int) { return 512; }                     // a k-step: 32 tokens
__host__ __device__ constexpr int p_tile_bytes(int qr) { return qr <= 8 ? 4096 : 8192; }
// TMEM columns of group g start at 4 * N * g: S^T (tg = 0 | 1) then O^T (parity 0 | 1), N each.
__host__ __device__ constexpr int tmem_cols(int qr) { return 4 * acc_n(qr) * kNG <= 256 ? 256 : 512; }

// barrier indices inside the barrier block.
// A parity wait is only meaningful while the waiter is at most one phase ahead of the barrier,
// so every barrier below is waited on either by one role in item order, or by a role that has
// first observed an event implying the previous phase (noted at the wait).
enum : int {
  kBarKFull = 0,    // [K slot] K bytes landed (transaction count)
  kBarVFull = 4,    // [V slot] V bytes landed
  kBarQEmpty = 8,   // [query slot] the softmax group has read the slot's scales: 4 arrivals
  kBarSFull = 12,   // [group] QK^T of the group's current item is complete (commit); this also
                    //         frees the item's K slot and query tile
  kBarPFull = 16,   // [group] P^T stored, V cleared where needed, S^T consumed: 4 arrivals
  kBarOFull = 20,   // [group][parity] P.V complete (commit); this also frees the item's V slot
  kBarQFull = 28,   // [query slot] query tile (and per-token scales) written
  kNumBars = 32
};
// fixed head of the shared-memory carve (bytes).  A softmax group keeps two items in flight (the
// softmax of its next item runs before the epilogue of the previous one), so what the epilogue
// reads is double buffered by the item's parity inside the group.
constexpr int kOffBars = 0;
constexpr int kOffTmemPtr = 384;
constexpr int kOffDone = 388;                     // [3 groups] ints (single-launch form): warps of the group that have stored an item (4 per item)
constexpr int kOffScan = 400;                     // 32 ints
constexpr int kOffRowLim = 528;                   // [64] ints: L - 1 - (row / G) for every query row
constexpr int kOffSingles = 784;                  // int (PAIR form): this CTA's units that have one item only
constexpr int kOffRowOff = 800;                   // [3 groups][16] floats: exponent offset of every row of the group's current item
constexpr int kOffRedMax = 1024;                  // [4 groups][16 q][4 warps] floats
constexpr int kOffRedSum = 2048;                  // [4 groups][2 parities][16 q][4 warps] floats
constexpr int kOffMFin = 4096;                    // [4 groups][2 parities][16] floats (max, log2 domain)
constexpr int kOffVMax = 4608;                    // [4 groups][4 warps] floats (per-token V scale max)
constexpr int kOffVNorm = 4672;                   // [4 groups][2 parities] floats
constexpr int kOffFRow = 4736;                    // [4 groups][2 parities][16] floats: V scale / row sum
constexpr int kHeadBytes = 5248;

// One work item: a 256-token partition of one kv head, and one block of query rows.
struct TcItem {
  int seq, head, part, rb;
  int ctx;      // context length of the sequence (clamped)
  int tok0;     // first token of the item
  int ntok;     // tokens of the item that exist (1..256)
  int sub;      // PAIR form: which 256-token half of its 512-token partition the item is (else 0)
  bool paired;  // PAIR form: the partition has both halves
};

// Walks the work items of one role: item k = first, first + step, ...  Items are numbered
// ((sequence, partition) pair, head, row block) with the row block fastest.  Decoding an index
// needs a search in the partition prefix sum; the cursor does that once and then steps forward.
struct ItemCursor {
  int sp, head, rb, seq, step_sp, step_head, step_rb;   // (the step is kept in the same mixed radix: no divisions per item)
  __device__ __noinline__ void init(int k, int step, const KernelParams& p, const int* seq_off, const int*) {
    const int nrb = p.num_row_blocks, hr_count = p.Hkv * nrb;
    sp = k / hr_count;
    const int hr = k - sp * hr_count;
    head = hr / nrb;
    rb = hr - head * nrb;
    step_sp = step / hr_count;
    const int shr = step - step_sp * hr_count;
    step_head = shr / nrb;
    step_rb = shr - step_head * nrb;
    int lo = 0, hi = p.S;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_off[mid] <= sp) lo = mid; else hi = mid;
    }
    seq = lo;
  }
  __device__ __forceinline__ void advance(const KernelParams& p, const int* seq_off) {
    rb += step_rb;
    if (rb >= p.num_row_blocks) {
      rb -= p.num_row_blocks;
      ++head;
    }
    head += step_head;
    if (head >= p.Hkv) {
      head -= p.Hkv;
      ++sp;
    }
    sp += step_sp;
    while (seq < p.S - 1 && seq_off[seq + 1] <= sp) ++seq;
  }
  __device__ __forceinline__ TcItem item(const KernelParams& p, const int* seq_off, const int* seq_ctx) const {
    TcItem it;
    it.seq = seq;
    it.head = head;
    it.rb = rb;
    it.part = sp - seq_off[seq];
    it.ctx = seq_ctx[seq];
    it.tok0 = it.part * kItemTokens;
    it.ntok = min(kItemTokens, it.ctx - it.tok0);
    it.sub = 0;
    it.paired = false;
    return it;
  }
};

// The other numbering: (sequence, kv head, partition, row block) with the row block fastest, for
// CTAs that take a contiguous range of items.  Consecutive items of a CTA then mostly share
// their query rows, so the query tile is built once per (sequence, kv head, row block) instead of
// once per item, and the row blocks of one partition find its KV bytes in L2.  (With items
// dealt round-robin in the first numbering the eight heads of a page are read by neighbouring
// CTAs at about the same time, which DRAM likes better: 5 % on the 4-row benchmark shape.  The
// contiguous form is for 16-row items, where building the query tile is what limits a CTA.)
struct RangeCursor {
  int seq, head, part, rb, parts, step;
  __device__ __noinline__ void init(int k, int step_, const KernelParams& p, const int* seq_off, const int*) {
    step = step_;
    const int nrb = p.num_row_blocks;
    const int kk = k / nrb;                 // (sequence, head, partition) index
    rb = k - kk * nrb;
    int lo = 0, hi = p.S;                   // last sequence whose first item is <= kk
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_off[mid] * p.Hkv <= kk) lo = mid; else hi = mid;
    }
    seq = lo;
    parts = seq_off[seq + 1] - seq_off[seq];
    const int rem = kk - seq_off[seq] * p.Hkv;
    head = parts > 0 ? rem / parts : 0;
    part = rem - head * parts;
  }
  __device__ __forceinline__ void advance(const KernelParams& p, const int* seq_off) {
    for (int s = 0; s < step; ++s) {
      if (++rb < p.num_row_blocks) continue;
      rb = 0;
      if (++part < parts) continue;
      part = 0;
      if (++head < p.Hkv) continue;
      head = 0;
      do {   // next sequence that has partitions (stepping past the last item leaves a state nobody reads)
        if (seq >= p.S - 1) break;
        ++seq;
        parts = seq_off[seq + 1] - seq_off[seq];
      } while (parts == 0);
    }
  }
  __device__ __forceinline__ TcItem item(const KernelParams& p, const int* seq_off, const int* seq_ctx) const {
    TcItem it;
    it.seq = seq;
    it.head = head;
    it.rb = rb;
    it.part = part;
    it.ctx = seq_ctx[seq];
    it.tok0 = it.part * kItemTokens;
    it.ntok = min(kItemTokens, it.ctx - it.tok0);
    it.sub = 0;
    it.paired = false;
    return it;
  }
};

// The numbering of the single-launch form (one row block per item).  The grid is made of teams of
// p.team_size CTAs.  A team takes a contiguous range of (sequence, partition) rows; its member a
// takes the kv heads a * hpc .. a * hpc + hpc - 1 of every row (hpc = Hkv / team size), row by
// row.  So a CTA walks down the partitions of hpc (sequence, kv head) sets at a time and holds
// all partitions of most of its sets, which is what lets it merge them itself; the heads of a
// page are still read by the members of a team at about the same time.
struct TeamRange {
  int row0, rows, head0, hpc;
};
__device__ __forceinline__ TeamRange team_range(const KernelParams& p, int n_sp) {
  TeamRange t;
  const int team = (int)blockIdx.x / p.team_size, member = (int)blockIdx.x - team * p.team_size;
  const int n_teams = (int)gridDim.x / p.team_size;    // the host makes the grid a multiple of the team size
  const int per = n_sp / n_teams, extra = n_sp - per * n_teams;
  t.row0 = team * per + min(team, extra);
  t.rows = per + (team < extra ? 1 : 0);
  t.hpc = p.Hkv / p.team_size;
  t.head0 = member * t.hpc;
  return t;
}
struct TeamCursor {
  int row, hl, seq, head0, hpc, step_row, step_h;
  // k, step: item numbers inside the CTA
  __device__ __noinline__ void init(int k, int step, const KernelParams& p, const int* seq_off, const int*) {
    const TeamRange t = team_range(p, seq_off[p.S]);
    head0 = t.head0;
    hpc = t.hpc;
    const int kr = k / hpc;
    row = t.row0 + kr;
    hl = k - kr * hpc;
    step_row = step / hpc;
    step_h = step - step_row * hpc;
    int lo = 0, hi = p.S;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_off[mid] <= row) lo = mid; else hi = mid;
    }
    seq = lo;
  }
  __device__ __forceinline__ void advance(const KernelParams& p, const int* seq_off) {
    hl += step_h;
    if (hl >= hpc) {
      hl -= hpc;
      ++row;
    }
    row += step_row;
    while (seq < p.S - 1 && seq_off[seq + 1] <= row) ++seq;
  }
  __device__ __forceinline__ TcItem item(const KernelParams& p, const int* seq_off, const int* seq_ctx) const {
    TcItem it;
    it.seq = seq;
    it.head = head0 + hl;
    it.rb = 0;
    it.part = row - seq_off[seq];
    it.ctx = seq_ctx[seq];
    it.tok0 = it.part * kItemTokens;
    it.ntok = min(kItemTokens, it.ctx - it.tok0);
    it.sub = 0;
    it.paired = false;
    return it;
  }
};

// The numbering of the PAIR form (512-token partitions in the workspaces, one row block).  The index
// counts 512-token rows; a unit is (row, kv head) with the head fastest, units are dealt to the
// CTAs round-robin, and a unit is one work item, or two consecutive ones when the row's second
// 256 tokens exist -- so both halves of a partition run in one CTA, one right after the other.
struct PairCursor {
  int row, head, seq, sub, step_items, step_row, step_head;
  const int* ctx;
  __device__ __forceinline__ bool second(const int* seq_off) const {
    return (row - seq_off[seq]) * (2 * kItemTokens) + kItemTokens < ctx[seq];
  }
  __device__ __forceinline__ void next(const KernelParams& p, const int* seq_off) {
    if (sub == 0 && second(seq_off)) {
      sub = 1;
      return;
    }
    sub = 0;
    head += step_head;
    if (head >= p.Hkv) {
      head -= p.Hkv;
      ++row;
    }
    row += step_row;
    while (seq < p.S - 1 && seq_off[seq + 1] <= row) ++seq;
  }
  // k, step: item numbers inside the CTA
  __device__ __noinline__ void init(int k, int step, const KernelParams& p, const int* seq_off, const int* seq_ctx) {
    ctx = seq_ctx;
    step_items = step;
    row = (int)blockIdx.x / p.Hkv;
    head = (int)blockIdx.x - row * p.Hkv;
    step_row = (int)gridDim.x / p.Hkv;
    step_head = (int)gridDim.x - step_row * p.Hkv;
    sub = 0;
    int lo = 0, hi = p.S;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seq_off[mid] <= row) lo = mid; else hi = mid;
    }
    seq = lo;
    for (int j = 0; j < k; ++j) next(p, seq_off);
  }
  __device__ __forceinline__ void advance(const KernelParams& p, const int* seq_off) {
    for (int j = 0; j < step_items; ++j) next(p, seq_off);
  }
  __device__ __forceinline__ TcItem item(const KernelParams& p, const int* seq_off, const int* seq_ctx) const {
    TcItem it;
    it.seq = seq;
    it.head = head;
    it.rb = 0;
    it.part = row - seq_off[seq];
    it.ctx = seq_ctx[seq];
    it.sub = sub;
    it.paired = sub != 0 || second(seq_off);
    it.tok0 = it.part * (2 * kItemTokens) + sub * kItemTokens;
    it.ntok = min(kItemTokens, it.ctx - it.tok0);
    return it;
  }
};

// Error bits are set from rare paths only: one shared out-of-line copy of the atomic.
__device__ __noinline__ void report_status(int32_t* status, int bit) {
  if (status) atomicOr(status, bit);
}

// Monotonic float <-> int map, so a float maximum can use the single-instruction integer
// warp reduction.
__device__ __forceinline__ int float_to_ordered(float x) {
  const int i = __float_as_int(x);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) {
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

// Nine shuffles add eight values over the warp; lane ends up with the sum for q = (lane >> 2) & 7.
__device__ __forceinline__ float warp_sum8(const float (&v)[8], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float a[4], b[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float mine = b4 ? v[4 + j] : v[j];
    const float other = b4 ? v[j] : v[4 + j];
    a[j] = mine + __shfl_xor_sync(kFullMask, other, 16);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b3 ? a[2 + j] : a[j];
    const float other = b3 ? a[j] : a[2 + j];
    b[j] = mine + __shfl_xor_sync(kFullMask, other, 8);
  }
  float c = (b2 ? b[1] : b[0]) + __shfl_xor_sync(kFullMask, b2 ? b[0] : b[1], 4);
  c += __shfl_xor_sync(kFullMask, c, 2);
  c += __shfl_xor_sync(kFullMask, c, 1);
  return c;
}
// Six shuffles for four values; lane ends up with the sum for q = (lane >> 3) & 3.
__device__ __forceinline__ float warp_sum4(const float (&v)[4], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8;
  float a[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b4 ? v[2 + j] : v[j];
    const float other = b4 ? v[j] : v[2 + j];
    a[j] = mine + __shfl_xor_sync(kFullMask, other, 16);
  }
  float c = (b3 ? a[1] : a[0]) + __shfl_xor_sync(kFullMask, b3 ? a[0] : a[1], 8);
  c += __shfl_xor_sync(kFullMask, c, 4);
  c += __shfl_xor_sync(kFullMask, c, 2);
  c += __shfl_xor_sync(kFullMask, c, 1);
  return c;
}

// The same exchanges with a maximum: lane ends up with the maximum for q = (lane >> 2) & 7.
__device__ __forceinline__ float warp_max8(const float (&v)[8], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
  float a[4], b[2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float mine = b4 ? v[4 + j] : v[j];
    const float other = b4 ? v[j] : v[4 + j];
    a[j] = fmaxf(mine, __shfl_xor_sync(kFullMask, other, 16));
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b3 ? a[2 + j] : a[j];
    const float other = b3 ? a[j] : a[2 + j];
    b[j] = fmaxf(mine, __shfl_xor_sync(kFullMask, other, 8));
  }
  float c = fmaxf(b2 ? b[1] : b[0], __shfl_xor_sync(kFullMask, b2 ? b[0] : b[1], 4));
  c = fmaxf(c, __shfl_xor_sync(kFullMask, c, 2));
  c = fmaxf(c, __shfl_xor_sync(kFullMask, c, 1));
  return c;
}
// ... and for four values: lane ends up with the maximum for q = (lane >> 3) & 3.
__device__ __forceinline__ float warp_max4(const float (&v)[4], int lane) {
  const bool b4 = lane & 16, b3 = lane & 8;
  float a[2];
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const float mine = b4 ? v[2 + j] : v[j];
    const float other = b4 ? v[j] : v[2 + j];
    a[j] = fmaxf(mine, __shfl_xor_sync(kFullMask, other, 16));
  }
  float c = fmaxf(b3 ? a[1] : a[0], __shfl_xor_sync(kFullMask, b3 ? a[0] : a[1], 8));
  c = fmaxf(c, __shfl_xor_sync(kFullMask, c, 4));
  c = fmaxf(c, __shfl_xor_sync(kFullMask, c, 2));
  c = fmaxf(c, __shfl_xor_sync(kFullMask, c, 1));
  return c;
}

// ---- geometry that depends on the page size (BS = 16, 64 or 1024) -------------------------------
template <int BS>
struct Geo {
  // K operand descriptor: stride between the two 16-byte K units, between 8-token groups, and the
  // offset of the second M = 128 tile.  BS = 16 keeps whole pages in the slot; otherwise the
  // slot is [chunk][256 tokens][16 B].
  static constexpr int kKLbo = BS == 16 ? 256 : 4096;
  static constexpr int kKSbo = BS == 16 ? 2048 : 128;
  static constexpr int kKTile1 = BS == 16 ? 128 : 2048;
  // V operand.  BS = 16: a page [128 d][16 tok] is already a column of core matrices (rows 16 B
  // apart); two pages make the two K units of an instruction.  Longer pages have rows BS bytes
  // apart, which only the swizzled operand form can express: a tiled TMA copy brings boxes of
  // [128 d][kVSpan tokens] (kVSpan = 64 or 128) into the slot with the matching swizzle.
  static constexpr int kVSpan = BS == 16 ? 16 : (BS == 64 ? 64 : 128);   // bytes (= tokens) per row of a box
  static constexpr int kVBox = 128 * kVSpan;                              // bytes of one box
  static constexpr int kVSbo = 8 * kVSpan;
  // byte offset in the V slot of (head dim d, tokens [16*g, 16*g + 16) of the item)
  __host__ __device__ static constexpr int v_chunk(int d, int g) {
    if (BS == 16) return g * 2048 + d * 16;
    const int per_box = kVSpan / 16;                 // 16-token chunks per row of a box
    const int box = g / per_box, c = g % per_box;
    return box * kVBox + d * kVSpan + ((c ^ (BS == 64 ? ((d >> 1) & 3) : (d & 7))) * 16);
  }
  // start address (inside the V slot) of the operand of k-step ks (tokens [32*ks, 32*ks + 32))
  __host__ __device__ static constexpr int v_kstep(int ks) {
    if (BS == 16) return 2 * ks * 2048;
    const int per_box = kVSpan >= 32 ? kVSpan / 32 : 1;   // k-steps per box
    return (ks / per_box) * kVBox + (ks % per_box) * 32;
  }
  // token (0..255 inside the item) held by TMEM lane r of S^T tile tg
  __device__ static __forceinline__ int token(int tg, int r) {
    return BS == 16 ? (r >> 3) * 16 + tg * 8 + (r & 7) : tg * 128 + r;
  }
};

// BS: tokens per page.  QR: query rows per work item (4, 8 or 16; the host picks the smallest
// that holds eqG, or 16 with several row blocks).  PER_TOKEN: per-token-per-head K/V scales.
// TRACE: compile the clock stamps in (tuning builds).
// ALIBI: add slope[head] * (key position - (context - 1)) to the logits
// (pa_decode_triton_gluon_fp8.py:905-908).
// FUSE: the launch also does the cross-partition reduce (paged_attention_decode_v2_reduce_kernel,
// pa_decode_triton_gluon_fp8.py:1187-1333).  CTAs take their items in the TeamCursor numbering, so
// that a CTA computes all partitions of most of its (sequence, kv head) sets; the softmax group
// that stores the last of a set's partitions in the CTA merges the set right there (see the
// epilogue).  A set cut by the end of a team's range is merged by the CTA that holds its first
// partitions -- it reaches them at the very end of its range -- and the CTAs of the later teams,
// which meet their share at the start of theirs, hand it over through p.merge_counters.
// PAIR: the workspaces hold 512-token partitions (p.partition_size = 512, one row block).  The
// kernel still works on 256-token items; the two halves of a partition run as consecutive items
// of one CTA (PairCursor), the first half leaves its (max, sum, output) in shared memory and the
// second half's epilogue merges the two and stores the partition (see the epilogue).
// STAGE: per-token scales of pages of 64 tokens or more travel in the query slots (see q_slot_bytes);
// false where the host found no room for that.
template <int BS, int QR, bool PER_TOKEN, bool TRACE, bool ALIBI = false, bool FUSE = false, bool PAIR = false, bool STAGE = true>
__global__ void __launch_bounds__(kThreads, 1)
pa_partition_fp8_tc_kernel(const __grid_constant__ KernelParams p, const __grid_constant__ CUtensorMap vmap) {
  using G = Geo<BS>;
  static_assert(!FUSE || (QR <= 8 && !ALIBI && !TRACE), "the single-launch form exists for 4- and 8-row items");
  static_assert(!PAIR || (!FUSE && !ALIBI && !TRACE), "the PAIR form is plain");
  constexpr int NG = kNG;
  constexpr bool kSum = sums_in_tensor_core(QR);   // hi and lo products summed by the tensor core
  constexpr int N = acc_n(QR);                 // MMA N and TMEM columns per tile
  constexpr bool kStaged = STAGE && staged_token_scales(BS, PER_TOKEN) && !(PAIR && QR == 16);
  constexpr int kQSlotBytes = q_slot_bytes(QR, kStaged);
  constexpr bool kItemFromSlot = PA_ITEM_FROM_SLOT && (!PER_TOKEN || kStaged);
  constexpr bool kKeepInTmem = sums_in_tensor_core(QR);   // two chunks of rows, one accumulator column per row
  constexpr int kQTile = q_tile_bytes(QR);
  constexpr int kPTile = p_tile_bytes(QR);
  constexpr int kPStep = p_step_bytes(QR);
  extern __shared__ __align__(1024) uint8_t smem[];
  const long long t_entry = TRACE ? clock64() : 0;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int NSK = p.num_stages;    // K ring (and query ring) depth
  const int NSV = p.num_vstages;   // V ring depth

  const uint32_t sbase = smem_addr(smem);
  const uint32_t bars = sbase + kOffBars;
  auto bar = [&](int which, int idx) -> uint32_t { return bars + (which + idx) * 8; };
  int* seq_off = reinterpret_cast<int*>(smem + p.off_seq_offsets);
  int* seq_ctx = reinterpret_cast<int*>(smem + p.off_seq_ctx);
  int* row_lim = reinterpret_cast<int*>(smem + kOffRowLim);
  float* red_max = reinterpret_cast<float*>(smem + kOffRedMax);
  float* red_sum = reinterpret_cast<float*>(smem + kOffRedSum);
  float* m_fin = reinterpret_cast<float*>(smem + kOffMFin);
  float* v_max = reinterpret_cast<float*>(smem + kOffVMax);
  float* v_norm = reinterpret_cast<float*>(smem + kOffVNorm);
  float* f_row = reinterpret_cast<float*>(smem + kOffFRow);
  float* row_off = reinterpret_cast<float*>(smem + kOffRowOff);
  const uint32_t q_ring = sbase + p.off_q;     // kQSlots x kQSlotBytes
  const uint32_t p_tiles = sbase + p.off_p;    // NG x kPTile
  const uint32_t k_ring = sbase + p.off_ring;  // NSK x kHalfSlot
  const uint32_t v_ring = sbase + p.off_vring; // NSV x kHalfSlot

  if (tid == 0) {
    for (int s = 0; s < kMaxSlots; ++s) {
      mbar_init(bar(kBarKFull, s), 1);
      mbar_init(bar(kBarQFull, s), 1);
      mbar_init(bar(kBarVFull, s), 1);
      mbar_init(bar(kBarQEmpty, s), 4);
    }
    for (int g = 0; g < 4; ++g) {
      mbar_init(bar(kBarSFull, g), 1);
      mbar_init(bar(kBarPFull, g), 4);
      for (int b = 0; b < 2; ++b) mbar_init(bar(kBarOFull, 2 * g + b), 1);
    }
    mbar_fence_init();
    fence_proxy_async();
    if (FUSE || PAIR) {
      for (int g = 0; g < NG; ++g) *reinterpret_cast<volatile int*>(smem + kOffDone + 4 * g) = 0;
      *reinterpret_cast<volatile int*>(smem + kOffSingles) = 0;
    }
  }
  // row r = t * G + g of a kv head sees token j iff j < ctx - (L - 1 - t)
  // (padding rows of the last row block see nothing)
  for (int r = tid; r < 64; r += (int)blockDim.x) row_lim[r] = r < p.eqG ? (p.L - 1 - r / p.G) : 0x7fffffff;
  if (warp == kWarpMma) tmem_alloc(sbase + kOffTmemPtr, tmem_cols(QR));
  // Everything above touches this CTA's shared and tensor memory only and may run while the
  // kernel before this one in the stream drains.
  //
  // So may the first link of this CTA's own chain of dependent loads (lengths -> partition index
  // -> block-table entries -> pages), as long as nothing depends on what it reads early: the
  // index is built from lengths read past the L1; after the wait it is checked against the
  // lengths as they are then, and rebuilt if one changed.  In a decode loop a CTA becomes
  // resident while the call before it drains, and one of the three memory latencies before its
  // first bytes is then behind it when the wait returns (0.5-1 us of a call).  (Going further --
  // requesting the pages of the CTA's first items into L2 before the wait, from block-table
  // entries read early -- was measured and is not done: two items ahead made no difference,
  // four cost 2 us; the traffic competes with the tail of the call before.)
  int n_sp = 0;
  const bool early = p.early_start != 0;
  if (early) {
    n_sp = build_partition_index(p, seq_off, seq_ctx, reinterpret_cast<int*>(smem + kOffScan), true);
  }
  // From here on global memory is read for good, and written.
  grid_dependency_wait();
  const long long t_dep = TRACE ? clock64() : 0;
  if (!early || !partition_index_still_valid(p, seq_ctx))
    n_sp = build_partition_index(p, seq_off, seq_ctx, reinterpret_cast<int*>(smem + kOffScan));
  if (PAIR) {
    // units of this CTA whose row has no second half: the last row of a sequence that ends in its first 256 tokens
    for (int s = tid; s < p.S; s += (int)blockDim.x) {
      const int rows = seq_off[s + 1] - seq_off[s];
      if (rows == 0 || (rows - 1) * (2 * kItemTokens) + kItemTokens < seq_ctx[s]) continue;
      const int u0 = (seq_off[s + 1] - 1) * p.Hkv;     // the row's units: u0 .. u0 + Hkv - 1
      int mine = 0;
      for (int h = 0; h < p.Hkv; ++h) mine += ((u0 + h) % (int)gridDim.x == (int)blockIdx.x) ? 1 : 0;
      if (mine) atomicAdd(reinterpret_cast<int*>(smem + kOffSingles), mine);
    }
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  grid_launch_dependents();  // the reduce kernel may become resident; it waits for this grid to finish
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + kOffTmemPtr);

  const int n_items = n_sp * p.Hkv * p.num_row_blocks;
  if (FUSE) {
    // a sequence without tokens has no work item, so nobody would merge it: its output rows are zeros
    for (int s = blockIdx.x; s < p.S; s += gridDim.x) {
      if (seq_off[s + 1] != seq_off[s]) continue;
      const int words = p.Hkv * p.eqG * (kD / 4);      // 8-byte words of the sequence's rows
      for (int w = tid; w < words; w += (int)blockDim.x) {
        const int row = w / (kD / 4), c = w - row * (kD / 4);
        *reinterpret_cast<uint2*>(p.out + 2 * ((int64_t)s * p.out_stride_seq + (int64_t)row * p.out_stride_head + 4 * c)) =
            make_uint2(0u, 0u);
      }
    }
  }
  // items of this CTA: a contiguous range for 16-row items, a team's share in the single-launch
  // form (numbered inside the CTA), else every gridDim.x-th item
  constexpr bool kContiguous = QR == 16;
  using Cursor = typename std::conditional<PAIR, PairCursor, typename std::conditional<FUSE, TeamCursor,
                                           typename std::conditional<kContiguous, RangeCursor, ItemCursor>::type>::type>::type;
  // (PAIR form: n_items counts units here, and a unit is one item or two)
  const int per_cta = n_items / (int)gridDim.x, extra = n_items - per_cta * (int)gridDim.x;
  TeamRange team{};
  if (FUSE) team = team_range(p, n_sp);
  const int first = (FUSE || PAIR) ? 0 : (kContiguous ? (int)blockIdx.x * per_cta + min((int)blockIdx.x, extra) : (int)blockIdx.x);
  const int stride = (FUSE || PAIR || kContiguous) ? 1 : (int)gridDim.x;
  const int n_units = per_cta + ((int)blockIdx.x < extra ? 1 : 0);
  const int n_local = FUSE ? team.rows * team.hpc
                           : (PAIR ? 2 * n_units - *reinterpret_cast<volatile int*>(smem + kOffSingles) : n_units);
  bool dead = false;

  // Tuning aid: when p.trace is set, lane 0 of each role of CTA 0 stamps the SM clock at a few
  // points of its first 64 items: trace[(role * 64 + item) * 4 + point].
  auto stamp = [&](int role, int item, int point) {
    if (TRACE && p.trace != nullptr && blockIdx.x == 0 && lane == 0 && item < 64)
      p.trace[(role * 64 + item) * 4 + point] = (unsigned long long)clock64();
  };
  if (TRACE && p.trace != nullptr && blockIdx.x == 0 && tid == 0) {   // entry, dependency wait passed, set-up done
    p.trace[(7 * 64 + 60) * 4 + 0] = (unsigned long long)t_entry;
    p.trace[(7 * 64 + 60) * 4 + 1] = (unsigned long long)t_dep;
    p.trace[(7 * 64 + 60) * 4 + 2] = (unsigned long long)clock64();
  }
  auto fail = [&]() {
    dead = true;
    if (lane == 0) report_status(p.status, PA_DEV_WAIT_TIMEOUT);
  };
  // whole-warp bounded wait, uniform result
  auto wait = [&](uint32_t b, uint32_t parity) -> bool {
    return __all_sync(kFullMask, mbar_wait(b, parity));
  };
  // Block-table entry of page `pg` (counted inside the item) of an item, as loaded: the roles
  // fetch it an item ahead and must not touch the value before they use it (a comparison right
  // after the load would make them wait for it there), so clamping is a separate step.
  auto page_id_raw = [&](const TcItem& it, int pg) -> int {
    const int64_t col = BS >= kItemTokens ? (int64_t)(it.tok0 / BS) : (int64_t)(it.tok0 / BS + pg);
    return __ldg(p.block_tables + (int64_t)it.seq * p.bt_stride_seq + col);
  };
  auto clamp_page = [&](int id, bool report) -> int {
    if ((unsigned)id >= (unsigned)p.num_blocks) {
      id = 0;
      if (report) report_status(p.status, PA_DEV_BAD_PAGE_ID);
    }
    return id;
  };
  // pages of the item that hold at least one valid token
  auto pages_of = [&](const TcItem& it) -> int { return BS >= kItemTokens ? 1 : (it.ntok + BS - 1) / BS; };

  if (warp == kWarpK || warp == kWarpV) {
    // ------------------------------------------------------------------ K / V producer
    const bool is_v = warp == kWarpV;
    const uint8_t* cache = is_v ? p.v : p.k;
    const int64_t stride_block = is_v ? p.v_stride_block : p.k_stride_block;
    const int64_t stride_head = is_v ? p.v_stride_head : p.k_stride_head;
    const int NS = is_v ? NSV : NSK;
    const uint32_t ring = is_v ? v_ring : k_ring;
    const uint64_t pol = l2_policy_evict_first();
    // which page of the item this lane copies from
    // (transposed value layout: lane = one of the item's sixteen 16-token runs)
    const bool vt = BS != 16 && is_v && p.v_trans != 0;
    auto my_page = [&]() -> int {
      if (BS == 16) return lane;
      if (BS == 64) return is_v ? (vt ? (lane >> 2) : lane) : (lane >> 3);
      return 0;
    };
    auto load_page_id = [&](const TcItem& it) -> int {
      const int pg = my_page();
      return pg < pages_of(it) ? page_id_raw(it, pg) : 0;
    };
    Cursor cur;
    TcItem it_next{};
    int pid_next = 0;
    if (n_local > 0) {
      cur.init(first, stride, p, seq_off, seq_ctx);
      it_next = cur.item(p, seq_off, seq_ctx);
      pid_next = load_page_id(it_next);
    }
    for (int i = 0; i < n_local && !dead; ++i) {
      const TcItem it = it_next;
      const int pid = clamp_page(pid_next, true);
      const int slot = i % NS;
      stamp(is_v ? 1 : 0, i, 0);
      if (i >= NS) {
        // The slot is free once the product that read it (item i - NS) is complete: QK^T for K,
        // P.V for V.  This role has already seen the products of all earlier items, so the
        // barrier's previous phase is known to be complete.
        const int j = i - NS;
        const int g = j % NG;
        const uint32_t gu = (uint32_t)(j / NG);
        const bool ok = is_v ? wait(bar(kBarOFull, 2 * g + (int)(gu & 1)), (gu >> 1) & 1)
                             : wait(bar(kBarSFull, g), gu & 1);
        if (!ok) { fail(); break; }
      }
      stamp(is_v ? 1 : 0, i, 1);
      const uint32_t full = bar(is_v ? kBarVFull : kBarKFull, slot);
      const uint32_t dst = ring + slot * kHalfSlot;
      const int npg = pages_of(it);
      const uint8_t* src = cache + (int64_t)pid * stride_block + (int64_t)it.head * stride_head;
      if (BS == 16) {        // one 2 KB run per page, K and V alike
        if (lane == 0) mbar_arrive_expect_tx(full, npg * kPageBytes);
        __syncwarp();
        if (lane < npg) bulk_g2s(dst + lane * kPageBytes, src, kPageBytes, full, pol);
      } else if (vt) {       // transposed values: 2 KB runs [128 d][16 tok], laid out in the slot as 16-token pages
        const int runs = (it.ntok + 15) >> 4;
        const int first_run = BS == 64 ? (lane & 3) : ((it.tok0 % BS) >> 4) + lane;   // run inside the page
        if (lane == 0) mbar_arrive_expect_tx(full, runs * kPageBytes);
        __syncwarp();
        if (lane < runs) bulk_g2s(dst + lane * kPageBytes, src + (int64_t)first_run * kPageBytes, kPageBytes, full, pol);
      } else if (BS == 64) {
        if (lane == 0) mbar_arrive_expect_tx(full, npg * 8192);
        __syncwarp();
        if (is_v) {          // one swizzled box [128 d][64 tok] per page
          if (lane < npg) tma_load_4d(dst + lane * G::kVBox, &vmap, 0, 0, it.head, pid, full, pol);
        } else {             // (page, chunk) run of 64 tok x 16 B -> [chunk][256 tok][16 B]
          const int pg = lane >> 3, c = lane & 7;
          if (pg < npg) bulk_g2s(dst + c * 4096 + pg * 1024, src + c * 1024, 1024, full, pol);
        }
      } else {               // 256-token slice of one large page
        // only what holds a token of the context is fetched (the last partition of a sequence): rows
        // of the K tile past it keep older bytes, whose logits are masked, and the softmax clears the
        // V slot past the context whether it was loaded or not
        const int tin = it.tok0 % BS;
        const int boxes = it.ntok > 128 ? 2 : 1;
        const uint32_t kbytes = (uint32_t)it.ntok * 16;
        if (lane == 0) mbar_arrive_expect_tx(full, is_v ? (uint32_t)(boxes * G::kVBox) : 8 * kbytes);
        __syncwarp();
        if (is_v) {          // swizzled boxes [128 d][128 tok]
          if (lane < boxes) tma_load_4d(dst + lane * G::kVBox, &vmap, tin + 128 * lane, 0, it.head, pid, full, pol);
        } else if (lane < 8) {  // 8 chunks x (tokens x 16 B)
          bulk_g2s(dst + lane * 4096, src + (int64_t)lane * BS * 16 + tin * 16, kbytes, full, pol);
        }
      }
      stamp(is_v ? 1 : 0, i, 2);
      // the next item and its page id, after this item's copies are on their way (the load has
      // the whole wait for the next slot to land)
      if (i + 1 < n_local) {
        cur.advance(p, seq_off);
        it_next = cur.item(p, seq_off, seq_ctx);
        pid_next = load_page_id(it_next);
      }
    }
  } else
  if (warp == kWarpQ) {
    // ------------------------------------------------------------------ query (+ scales) producer
    // lane -> row n0 = lane / 4 of a pass of 8 rows, quarter qq = lane % 4 of the head dims (32 each)
    constexpr int kPasses = QR > 8 ? QR / 8 : 1;
    static_assert(kPasses <= 2, "the pass loop selects between two register sets");
    const int n0 = lane >> 2, qq = lane & 3;
    const float q_base_scale = p.softmax_scale * kLog2e *
                               ((!PER_TOKEN && p.kv_quant_mode == PA_QUANT_PER_TENSOR) ? __ldg(p.k_scale) : 1.0f);
    auto load_q = [&](const TcItem& it, uint4 (&raw)[kPasses][4]) {
#pragma unroll
      for (int ps = 0; ps < kPasses; ++ps) {
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[ps][e] = make_uint4(0u, 0u, 0u, 0u);
        const int n = ps * 8 + n0;
        const int row = it.rb * QR + n;              // row inside the kv head's query group
        if (n < QR && row < p.eqG) {
          // this lane's 32 elements of the row: 64 bytes of bf16, or 32 bytes of e4m3
          const uint8_t* row_ptr = p.q + (int64_t)it.seq * p.q_stride_seq + (int64_t)(it.head * p.eqG + row) * p.q_stride_head;
          const uint4* src = reinterpret_cast<const uint4*>(row_ptr + (p.q_is_fp8 ? qq * 32 : qq * 64));
          raw[ps][0] = __ldg(src);
          raw[ps][1] = __ldg(src + 1);
          if (!p.q_is_fp8) {
            raw[ps][2] = __ldg(src + 2);
            raw[ps][3] = __ldg(src + 3);
          }
        }
      }
    };
    Cursor cur;
    TcItem it_next{};
    uint4 q_next[kPasses][4];
    // A tile is built when an item's query rows are not among the tiles of the current
    // (sequence, kv head): one tile per row block, remembered until the head changes.  It goes
    // to tile slot (tile count) % kQSlots.  That slot's previous tile is four tiles old, and
    // usually its last user is at least four items back, whose release this loop has waited for
    // anyway.  Not always: a CTA whose range begins in the middle of a partition meets the row
    // blocks in rotated order, and with three or four row blocks the tile about to be replaced
    // may belong to an item only two or three back, whose QK^T may not even have been issued.
    // So the loop remembers the last item that uses each tile slot and, before it rebuilds a
    // slot, waits for that very item's release.
    int tile = -1;
    int last_user[kQSlots];
#pragma unroll
    for (int s = 0; s < kQSlots; ++s) last_user[s] = -1;
    int key_seq = -1, key_head = -1;
    uint32_t tile_slots = 0;     // 4 bits per row block: bit 3 = valid, bits 0-1 = slot
    auto have_tile = [&](const TcItem& it) -> bool {
      return it.seq == key_seq && it.head == key_head && ((tile_slots >> (4 * it.rb)) & 8u) != 0;
    };
    bool fresh_next = true;
    // staged token scales: lane pg copies the scales of page pg of the item (one page of 1024
    // tokens, or four of 64); its block-table entry is fetched an item ahead
    constexpr int kScalePages = BS >= kItemTokens ? 1 : kItemTokens / (BS >= 64 ? BS : 64);
    auto scale_page_id = [&](const TcItem& it) -> int {
      return (kStaged && lane < kScalePages && lane < pages_of(it)) ? page_id_raw(it, lane) : 0;
    };
    int spid_next = 0;
    if (n_local > 0) {
      cur.init(first, stride, p, seq_off, seq_ctx);
      it_next = cur.item(p, seq_off, seq_ctx);
      load_q(it_next, q_next);
      spid_next = scale_page_id(it_next);
    }
    for (int i = 0; i < n_local && !dead; ++i) {
      const TcItem it = it_next;
      uint4 qraw[kPasses][4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
#pragma unroll
        for (int ps = 0; ps < kPasses; ++ps) qraw[ps][e] = q_next[ps][e];
      }
      const bool fresh = fresh_next;
      const int spid = spid_next;
      if (it.seq != key_seq || it.head != key_head) {
        key_seq = it.seq;
        key_head = it.head;
        tile_slots = 0;
      }
      if (fresh) {
        ++tile;
        tile_slots = (tile_slots & ~(15u << (4 * it.rb))) | ((8u | (uint32_t)(tile % kQSlots)) << (4 * it.rb));
      }
      const int tslot = (int)((tile_slots >> (4 * it.rb)) & 3u);
      {
        int lu = -1;
#pragma unroll
        for (int s = 0; s < kQSlots; ++s) {
          if (s == tslot) {
            lu = last_user[s];
            last_user[s] = i;
          }
        }
        // (the release of item lu completes phase lu / kQSlots of its slot's barrier; item lu + kQSlots,
        // whose release would complete the next phase, has not been produced yet)
        if (fresh && lu >= 0 && lu > i - kQSlots && !wait(bar(kBarQEmpty, lu % kQSlots), (uint32_t)(lu / kQSlots) & 1)) {
          fail();
          break;
        }
      }
      if (i + 1 < n_local) {
        cur.advance(p, seq_off);
        it_next = cur.item(p, seq_off, seq_ctx);
        fresh_next = !have_tile(it_next);
        if (fresh_next) load_q(it_next, q_next);
        spid_next = scale_page_id(it_next);
      }
      const int slot = i % kQSlots;
      const uint32_t use = (uint32_t)(i / kQSlots);
      stamp(2, i, 0);
      if (!wait(bar(kBarQEmpty, slot), (use & 1) ^ 1)) { fail(); break; }
      stamp(2, i, 1);
      const uint32_t qt = q_ring + tslot * kQSlotBytes;
      const uint32_t aux = qt + kQTile;                                   // the tile's row scales
      const uint32_t item_aux = q_ring + slot * kQSlotBytes + kQTile;     // the item's header
      if (lane == 0) {
        sts32(item_aux + kQHdr, (uint32_t)tslot);
        if (kItemFromSlot) {
          sts128(item_aux + kQItem, make_uint4((uint32_t)it.seq, (uint32_t)it.head, (uint32_t)it.part, (uint32_t)it.rb));
          sts128(item_aux + kQItem + 16, make_uint4((uint32_t)it.ctx, (uint32_t)it.tok0, (uint32_t)it.ntok,
                                                    (uint32_t)it.sub | (it.paired ? 2u : 0u)));
        }
      }
      if (kStaged) {
        // the item's token scales, straight from the scale tensors into the slot; they complete
        // the slot's barrier together with this warp's arrival below
        constexpr int kRun = (BS >= kItemTokens ? kItemTokens : BS) * 4;          // bytes of one page's scales inside the item
        const int npg = pages_of(it);
        if (lane == 0) mbar_expect_tx(bar(kBarQFull, slot), (uint32_t)(2 * npg * kRun));
        __syncwarp();
        if (lane < kScalePages && lane < npg) {
          const int64_t idx = (int64_t)clamp_page(spid, false) * p.kvs_stride_block + (int64_t)it.head * p.kvs_stride_head +
                              (BS >= kItemTokens ? it.tok0 % BS : 0);
          const uint32_t dst = item_aux + kQTokScales + lane * kRun;
          const uint64_t pol = l2_policy_evict_first();
          bulk_g2s(dst, p.k_scale + idx, kRun, bar(kBarQFull, slot), pol);
          bulk_g2s(dst + kItemTokens * 4, p.v_scale + idx, kRun, bar(kBarQFull, slot), pol);
        }
      }
      // (rolled: the code of every role's loop should stay resident in the instruction cache)
#pragma unroll 1
      for (int ps = 0; ps < (fresh ? kPasses : 0); ++ps) {
        const int n = ps * 8 + n0;
        const int row = it.rb * QR + n;
        uint4 qv[4];   // this lane's 32 bf16 of the row
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          qv[e] = qraw[0][e];
          if (kPasses > 1 && ps == 1) qv[e] = qraw[kPasses - 1][e];
        }
        // row maximum -> power-of-two pre-scale putting it in [128, 256).  |x| of a packed bf16
        // pair is a mask, and non-negative bf16 bit patterns order like unsigned integers.
        uint32_t m2 = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          m2 = __vmaxu2(m2, __vmaxu2(__vmaxu2(qv[e].x & 0x7fff7fffu, qv[e].y & 0x7fff7fffu),
                                     __vmaxu2(qv[e].z & 0x7fff7fffu, qv[e].w & 0x7fff7fffu)));
        }
        float amax = __uint_as_float(max(m2 & 0xffffu, m2 >> 16) << 16);
        amax = quad_max(amax);
        float pre = 1.0f, inv_pre = 1.0f;
        const int be = (int)((__float_as_uint(amax) >> 23) & 0xff);
        if (p.q_is_fp8) {
          // e4m3 rows are the hi half as they are (the lo half is zero, no pre-scale)
          if (n < QR) {
            const int nl = QR + n;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const uint32_t dst = qt + (2 * qq + c) * 128;
              sts128(dst + (n >> 3) * 1024 + (n & 7) * 16, qv[c]);
              sts128(dst + (nl >> 3) * 1024 + (nl & 7) * 16, make_uint4(0u, 0u, 0u, 0u));
            }
          }
        } else {
        if (be > 30 && be < 225) {
          pre = __uint_as_float((uint32_t)(254 + 7 - be) << 23);
          inv_pre = __uint_as_float((uint32_t)(be - 7) << 23);
        }
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {  // the two 16-dim chunks of this lane's quarter (rolled: code size)
          const uint4 a = c ? qv[2] : qv[0], b = c ? qv[3] : qv[1];
          const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
          uint32_t hi4[4], lo4[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float x[4] = {bf16_lo_to_f32(w[2 * k]), bf16_hi_to_f32(w[2 * k]),
                                bf16_lo_to_f32(w[2 * k + 1]), bf16_hi_to_f32(w[2 * k + 1])};
            float hi[4], lo[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) split_parts<kSum>(x[e] * pre, hi[e], lo[e]);
            hi4[k] = pack_e4m3x4(hi[0], hi[1], hi[2], hi[3]);
            lo4[k] = pack_e4m3x4(lo[0], lo[1], lo[2], lo[3]);
          }
          if (n < QR) {  // tile row n holds the hi half, tile row QR + n the lo half
            const int nl = QR + n;
            const uint32_t dst = qt + (2 * qq + c) * 128;
            sts128(dst + (n >> 3) * 1024 + (n & 7) * 16, make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]));
            sts128(dst + (nl >> 3) * 1024 + (nl & 7) * 16, make_uint4(lo4[0], lo4[1], lo4[2], lo4[3]));
          }
        }
        }  // bf16 rows
        if (qq == 0 && n < QR) {
          float qs = 1.0f;
          if (p.q_quant_mode == PA_QUANT_PER_TENSOR) qs = __ldg(p.q_scale);
          if (p.q_quant_mode == PA_QUANT_PER_TOKEN && row < p.eqG)
            qs = __ldg(p.q_scale + (int64_t)it.seq * p.q_scale_stride_seq + it.head * p.eqG + row);
          // the row's positive factor that turns a raw product into a base-2 logit (> 0 always, so that
          // a masked -inf stays -inf and maxima commute with the factor)
          sts32(aux + n * 4, __float_as_uint(fmaxf(inv_pre * qs * q_base_scale, 1e-30f)));
          if (ALIBI)   // slope of the row's query head, in the base-2 logit domain
            sts32(aux + kQSlope + n * 4, __float_as_uint(row < p.eqG ? __ldg(p.alibi + it.head * p.G + row % p.G) * kLog2e : 0.f));
        }
      }
      fence_proxy_async();  // the tile is read by the tensor core (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarQFull, slot));
      stamp(2, i, 2);
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issue
    constexpr uint32_t kIdesc = idesc_f32acc(128, N, 0, 0);
    constexpr uint32_t kIdescPV = idesc_f32acc(128, N, 0, 0, true);   // P^T is MN-major
    const bool leader = elect_one();  // the one lane that issues every MMA and commit
    // per item i: group g = i % NG, use gu = i / NG of the group's buffers, O^T parity gu & 1.
    // P.V of an item is issued kLag items after its QK^T, so a softmax group has that long to
    // turn S^T into P^T before this in-order issue loop would have to wait for it.  The S^T
    // columns QK^T(i) overwrites were read by the softmax of item i - NG, whose P.V was issued
    // one iteration ago (kLag = NG - 1), after that group's arrival.
    for (int i = 0; i < n_local + kLag && !dead; ++i) {
      if (i < n_local) {  // S^T(i) = K . Q^T
        const int slot = i % NSK, g = i % NG;
        const uint32_t use = (uint32_t)(i / NSK);
        stamp(3, i, 0);
        const int qslot = i % kQSlots;
        if (!wait(bar(kBarKFull, slot), use & 1) ||
            !wait(bar(kBarQFull, qslot), (uint32_t)(i / kQSlots) & 1)) { fail(); break; }
        stamp(3, i, 1);
        fence_after_sync();
        const uint64_t kd = smem_desc(k_ring + slot * kHalfSlot, G::kKLbo, G::kKSbo);
        const uint32_t tslot = lds32(q_ring + qslot * kQSlotBytes + kQTile + kQHdr);  // slot of the item's tile
        const uint64_t qd = smem_desc(q_ring + tslot * kQSlotBytes, 128, 1024);
        const uint32_t d0 = tmem_base + g * 4 * N;
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t ad = kd + (uint64_t)((2 * j * G::kKLbo + tg * G::kKTile1) >> 4);
            const uint64_t bd = qd + (uint64_t)(((2 * j) * 128) >> 4);
            if (leader) mma_f8_ss(d0 + tg * N, ad, bd, kIdesc, j > 0);
            if (kSum && leader) mma_f8_ss(d0 + tg * N, ad, bd + (uint64_t)((QR / 8 * 1024) >> 4), kIdesc, true);   // the lo rows' tile
          }
        }
        if (leader) mma_commit(bar(kBarSFull, g));
        __syncwarp();
      }
      if (i >= kLag) {  // O^T(j) = V^T . P^T
        const int j = i - kLag;
        const int vslot = j % NSV, g = j % NG;
        const uint32_t vuse = (uint32_t)(j / NSV), gu = (uint32_t)(j / NG);
        const int ob = 2 * g + (int)(gu & 1);
        // The group arrives only after its epilogue of two items ago has read the O^T columns
        // this product overwrites.  This warp waits on both barriers in item order.
        if (!wait(bar(kBarPFull, g), gu & 1) || !wait(bar(kBarVFull, vslot), vuse & 1)) { fail(); break; }
        stamp(3, j, 2);
        fence_after_sync();
        const bool v16 = BS == 16 || p.v_trans != 0;   // the slot holds [128 d][16 tok] runs
        const uint64_t vd = v16 ? smem_desc(v_ring + vslot * kHalfSlot, 2048, 128)
                                : smem_desc_swizzled(v_ring + vslot * kHalfSlot, G::kVSpan);
        const uint64_t pd = smem_desc(p_tiles + g * kPTile, kPLbo, kPSbo);
        const uint32_t d0 = tmem_base + g * 4 * N + 2 * N + (int)(gu & 1) * N;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t ad = vd + (uint64_t)((v16 ? Geo<16>::v_kstep(ks) : G::v_kstep(ks)) >> 4);
          const uint64_t bd = pd + (uint64_t)((ks * kPStep) >> 4);
          if (leader) mma_f8_ss(d0, ad, bd, kIdescPV, ks > 0);
          if (kSum && leader)   // the lo rows' tile
            mma_f8_ss(d0, ad, bd + (uint64_t)(4096 >> 4), kIdescPV, true);
        }
        if (leader) mma_commit(bar(kBarOFull, ob));
        __syncwarp();
        stamp(3, j, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue groups
    constexpr int RC = QR < 8 ? QR : 8;   // rows handled at a time
    constexpr int NCH = QR / RC;          // chunks of rows per item
    const int grp = warp >> 2;            // softmax group: takes items grp, grp + NG, ...
    const int wq = warp & 3;              // TMEM lane quarter this warp may touch
    const int r = wq * 32 + lane;         // TMEM lane: S^T row (token slot) / O^T row (head dim)
    const int bar_a = 1 + grp, bar_b = 5 + grp;  // named barriers of the group
    const uint32_t tmem_grp = tmem_base + ((uint32_t)(wq * 32) << 16) + grp * 4 * N;
    // (the per-tensor key scale is part of the row factors the query producer writes)
    float v_scale_t = 1.0f;
    if (!PER_TOKEN && p.kv_quant_mode == PA_QUANT_PER_TENSOR) v_scale_t = __ldg(p.v_scale);
    float* rm = red_max + grp * 64;       // [16 rows][4 warps]
    const int tok[2] = {G::token(0, r), G::token(1, r)};  // tokens (inside the item) of this lane
    // where this lane's two tokens go in the P^T tile (row 0)
    uint32_t p_at[2];
#pragma unroll
    for (int tg = 0; tg < 2; ++tg)
      p_at[tg] = p_tiles + grp * kPTile + tok[tg] * 16;

    // One chunk of RC rows of a transposed accumulator tile: value = hi column + lo column / 16.
    auto load_rows = [&](uint32_t tile, int ch, uint32_t (&h)[8], uint32_t (&l)[8]) {
      if (kSum) {
        tmem_ld8(tile + ch * 8, h);      // the finished sums
      } else if (QR == 4) {
        tmem_ld8(tile, h);               // columns 0-3 hi, 4-7 lo
      } else {
        tmem_ld8(tile + ch * 8, h);
        tmem_ld8(tile + QR + ch * 8, l);
      }
    };
    auto row_value = [&](const uint32_t (&h)[8], const uint32_t (&l)[8], int q) -> float {
      if (kSum) return __uint_as_float(h[q]);
      return QR == 4 ? fmaf(__uint_as_float(h[4 + q]), 0.0625f, __uint_as_float(h[q]))
                     : fmaf(__uint_as_float(l[q]), 0.0625f, __uint_as_float(h[q]));
    };

    // Unless they are staged in the query slot (kStaged), per-token K / V scales of this lane's two
    // tokens come straight from global memory, fetched ahead by the group itself: the block-table
    // entry two of the group's items ahead, the four scales one item ahead (each step has a whole
    // group iteration to land).
    auto load_tok_pids = [&](const TcItem& it, int (&pid)[2]) {
      pid[0] = 0;
      pid[1] = 0;
      if (PER_TOKEN && !kStaged) {
        // tokens of one lane share a page unless pages hold 64 tokens (then they are 128 tokens apart)
        if (tok[0] < it.ntok) pid[0] = page_id_raw(it, BS == 16 ? (tok[0] >> 4) : (BS == 64 ? (tok[0] >> 6) : 0));
        if (BS == 64) {
          if (tok[1] < it.ntok) pid[1] = page_id_raw(it, tok[1] >> 6);
        } else {
          pid[1] = pid[0];
        }
      }
    };
    auto load_tok_scales = [&](const TcItem& it, const int (&pid)[2], float (&sc)[4]) {  // k0, k1, v0, v1
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[e] = 0.f;
      if (PER_TOKEN && !kStaged) {
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
          if (tok[tg] < it.ntok) {
            const int in_page = BS == 16 ? (tok[tg] & 15) : (BS == 64 ? (tok[tg] & 63) : (it.tok0 % BS) + tok[tg]);
            const int64_t idx = (int64_t)clamp_page(pid[tg], false) * p.kvs_stride_block +
                                (int64_t)it.head * p.kvs_stride_head + in_page;
            sc[tg] = __ldg(p.k_scale + idx);
            sc[2 + tg] = __ldg(p.v_scale + idx);
          }
        }
      }
    };

    auto softmax = [&](int i, TcItem& it_io, const float (&tok_scales)[4]) -> bool {
      const int slot = i % kQSlots;
      const uint32_t use = (uint32_t)(i / kQSlots), gu = (uint32_t)(i / NG);
      const int par = grp * 2 + (int)(gu & 1);  // double-buffer index of what the epilogue reads
      if (wq == 0) stamp(4, i, 0);
      if (!wait(bar(kBarSFull, grp), gu & 1)) return false;
      if (wq == 0) stamp(4, i, 1);
      // QK^T of the item is done, so its query tile was complete: this wait returns at once and
      // orders the producer's scale writes before the reads below.
      if (!wait(bar(kBarQFull, slot), use & 1)) return false;
      const uint32_t item_aux = q_ring + slot * kQSlotBytes + kQTile;   // the item's header
      const uint32_t aux = q_ring + lds32(item_aux + kQHdr) * kQSlotBytes + kQTile;   // the tile's row scales
      if (kItemFromSlot) {
        const uint4 a = lds128(item_aux + kQItem), b = lds128(item_aux + kQItem + 16);
        it_io.seq = (int)a.x, it_io.head = (int)a.y, it_io.part = (int)a.z, it_io.rb = (int)a.w;
        it_io.ctx = (int)b.x, it_io.tok0 = (int)b.y, it_io.ntok = (int)b.z;
        it_io.sub = (int)(b.w & 1u), it_io.paired = (b.w & 2u) != 0;
      }
      const TcItem& it = it_io;
      // Per-row constants of one chunk of rows (fetched again for every chunk: the chunk loops
      // are rolled): the positive factor that turns a raw product into a base-2 logit, and the
      // causal limit.  The query slot is released when pass 2 has read them for the last time.
      float row_scale[RC];
      float slope[RC];   // ALiBi only
      int lim[RC];  // row q sees token j iff (tokens from j to the end of the context) > lim[q]
      // (This loop is bound by instruction fetch for 16-row items, and every block added to it
      // counts, executed or not.  Measured against their absence on the 16-row MTP workload: a second
      // copy of the logit code without the masking, for the items that lie wholly inside every row's
      // view -- all but the last partition of a context; a seventh fewer instructions -- 7 % slower;
      // one fminf against a per-token +-inf instead of the compare and select, with the row-wise
      // limits patched up in a rarely taken block, 7 % slower; both passes through one copy of the
      // logit code, no change.)
      auto load_row_consts = [&](int ch) {
#pragma unroll
        for (int q4 = 0; q4 < RC; q4 += 4) {
          const uint4 a = lds128(aux + (ch * RC + q4) * 4);
          row_scale[q4] = __uint_as_float(a.x), row_scale[q4 + 1] = __uint_as_float(a.y);
          row_scale[q4 + 2] = __uint_as_float(a.z), row_scale[q4 + 3] = __uint_as_float(a.w);
          const uint4 b = lds128(smem_addr(row_lim) + (it.rb * QR + ch * RC + q4) * 4);
          lim[q4] = (int)b.x, lim[q4 + 1] = (int)b.y, lim[q4 + 2] = (int)b.z, lim[q4 + 3] = (int)b.w;
          if (ALIBI) {
            const uint4 c = lds128(aux + kQSlope + (ch * RC + q4) * 4);
            slope[q4] = __uint_as_float(c.x), slope[q4 + 1] = __uint_as_float(c.y);
            slope[q4 + 2] = __uint_as_float(c.z), slope[q4 + 3] = __uint_as_float(c.w);
          }
        }
      };
      if (NCH == 1) load_row_consts(0);
      float ks_tok[2] = {1.f, 1.f}, vs_tok[2] = {1.f, 1.f};
      if (kStaged) {        // the item's slot holds its tokens' scales (key scales, then value scales)
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
          ks_tok[tg] = __uint_as_float(lds32(item_aux + kQTokScales + tok[tg] * 4));
          vs_tok[tg] = __uint_as_float(lds32(item_aux + kQTokScales + (kItemTokens + tok[tg]) * 4));
        }
      } else if (PER_TOKEN) {
        ks_tok[0] = tok_scales[0], ks_tok[1] = tok_scales[1];
        vs_tok[0] = tok_scales[2], vs_tok[1] = tok_scales[3];
      }
      fence_after_sync();
      if (wq == 0) stamp(6, i, 0);

      const int room[2] = {it.ctx - (it.tok0 + tok[0]), it.ctx - (it.tok0 + tok[1])};  // > lim <=> visible
      if (PER_TOKEN) {
        if (room[0] <= 0) vs_tok[0] = 0.f;
        if (room[1] <= 0) vs_tok[1] = 0.f;
      }
      // key position relative to the last one, for ALiBi: -(room - 1)
      const float rel_pos[2] = {(float)(1 - room[0]), (float)(1 - room[1])};
      // Raw logits of one chunk of rows for this lane's two tokens: the product (times the
      // token's key scale), -inf where the row does not see the token.  The row's factor is
      // applied later, fused into the exponent's argument.  (With ALiBi the bias differs per
      // token, so the factor and the bias are applied here and the maxima are those of the
      // finished logits.)
      auto raw_logits = [&](int ch, float (&s)[2][RC]) {
        uint32_t h[2][8], l[2][8];
        load_rows(tmem_grp, ch, h[0], l[0]);
        load_rows(tmem_grp + N, ch, h[1], l[1]);
        if (NCH > 1) load_row_consts(ch);
        tmem_ld_wait();
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
          for (int q = 0; q < RC; ++q) {
            float v = row_value(h[tg], l[tg], q);
            if (PER_TOKEN) v *= ks_tok[tg];
            if (ALIBI) v = fmaf(v, row_scale[q], slope[q] * rel_pos[tg]);
            s[tg][q] = room[tg] > lim[q] ? v : -INFINITY;
          }
        }
      };

      // ---- pass 1: partition maximum of the raw logits per row (transposing shuffle reduction)
      float s_keep[2][RC];
#pragma unroll 1
      for (int ch = 0; ch < NCH; ++ch) {
        raw_logits(ch, s_keep);
        // 16-row items: both chunks do not fit in registers, so the finished (scaled, masked) logits
        // go back into the accumulator columns they came from, and pass 2 reads them as they are
        if constexpr (kKeepInTmem) {
          tmem_st8(tmem_grp + ch * 8, s_keep[0]);
          tmem_st8(tmem_grp + N + ch * 8, s_keep[1]);
        }
        float mx[RC];
#pragma unroll
        for (int q = 0; q < RC; ++q) mx[q] = fmaxf(s_keep[0][q], s_keep[1][q]);
        if constexpr (RC == 8) {
          const float wm = warp_max8(mx, lane);
          if ((lane & 3) == 0) rm[(ch * 8 + ((lane >> 2) & 7)) * 4 + wq] = wm;
        } else {
          const float wm = warp_max4(mx, lane);
          if ((lane & 7) == 0) rm[((lane >> 3) & 3) * 4 + wq] = wm;
        }
      }
      if (PER_TOKEN) {
        const int vk = __reduce_max_sync(kFullMask, float_to_ordered(fmaxf(vs_tok[0], vs_tok[1])));
        if (lane == 0) v_max[grp * 4 + wq] = ordered_to_float(vk);
      }
      if (wq == 0) stamp(6, i, 1);
      named_barrier_sync(bar_a, 128);
      // thread `row` of the group combines the four warps' maxima of its row, once for the group:
      // the exponent offset every thread applies in pass 2 (raw * factor - m * factor + 8 as one
      // multiply-add per element), and the row's maximum (base-2 logit domain) for the epilogue
      if (r < QR) {
        const float4 m4 = *reinterpret_cast<const float4*>(rm + r * 4);
        const float m = fmaxf(fmaxf(m4.x, m4.y), fmaxf(m4.z, m4.w));
        const float sc = __uint_as_float(lds32(aux + r * 4));
        row_off[grp * 16 + r] = (m == -INFINITY) ? 8.0f : (ALIBI ? 8.0f - m : fmaf(-m, sc, 8.0f));
        m_fin[par * 16 + r] = (m == -INFINITY || ALIBI) ? m : m * sc;
      }
      named_barrier_sync(bar_a, 128);
      float vinv = 1.0f, vnorm = 1.0f;
      if (PER_TOKEN) {
        const float4 vm4 = *reinterpret_cast<const float4*>(v_max + grp * 4);
        vnorm = fmaxf(fmaxf(vm4.x, vm4.y), fmaxf(vm4.z, vm4.w));
        vinv = vnorm > 0.f ? 1.0f / vnorm : 0.f;
        vs_tok[0] *= vinv;
        vs_tok[1] *= vinv;
      }
      // The group's P^T tile is still being read by P.V of the group's previous item until that
      // product's commit has arrived (normally long ago).
      if (gu > 0) {
        const uint32_t pu = gu - 1;
        if (!wait(bar(kBarOFull, 2 * grp + (int)(pu & 1)), (pu >> 1) & 1)) return false;
      }

      if constexpr (kKeepInTmem) tmem_st_wait();
      if (wq == 0) stamp(6, i, 2);
      // ---- pass 2: P = exp2(raw * factor - m) * 256, split into hi / lo e4m3, stored as P^T
      // row sums of one chunk: lane ends up with the sum of one row over the warp's 64 tokens
      auto row_sums = [&](int ch, const float (&psum)[RC]) {
        if constexpr (RC == 8) {
          const float wsum = warp_sum8(psum, lane);
          if ((lane & 3) == 0) red_sum[par * 64 + (ch * 8 + ((lane >> 2) & 7)) * 4 + wq] = wsum;
        } else {
          const float wsum = warp_sum4(psum, lane);
          if ((lane & 7) == 0) red_sum[par * 64 + ((lane >> 3) & 3) * 4 + wq] = wsum;
        }
      };
      float psum[RC];
#pragma unroll 1
      for (int ch = 0; ch < NCH; ++ch) {
        if constexpr (kKeepInTmem) {
          uint32_t a[8], b[8];
          tmem_ld8(tmem_grp + ch * 8, a);
          tmem_ld8(tmem_grp + N + ch * 8, b);
          load_row_consts(ch);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < RC; ++q) s_keep[0][q] = __uint_as_float(a[q]), s_keep[1][q] = __uint_as_float(b[q]);
        } else
        if (NCH > 1) raw_logits(ch, s_keep);  // recomputed rather than kept: registers
        uint32_t pbytes[2][2 * ((RC + 3) / 4)];  // [tg][hi words, lo words], row q = byte q % 4
        float hi[2][RC], lo[2][RC];
        float offs[RC];
#pragma unroll
        for (int q4 = 0; q4 < RC; q4 += 4) {
          const float4 o4 = *reinterpret_cast<const float4*>(row_off + grp * 16 + ch * RC + q4);
          offs[q4] = o4.x, offs[q4 + 1] = o4.y, offs[q4 + 2] = o4.z, offs[q4 + 3] = o4.w;
        }
#pragma unroll
        for (int q = 0; q < RC; ++q) {
          // exponent argument raw * factor - m * factor + 8 as one multiply-add per element
          float p0, p1;
          if (ALIBI) {   // s_keep holds finished logits
            p0 = ex2(s_keep[0][q] + offs[q]);
            p1 = ex2(s_keep[1][q] + offs[q]);
          } else {
            p0 = ex2(fmaf(s_keep[0][q], row_scale[q], offs[q]));
            p1 = ex2(fmaf(s_keep[1][q], row_scale[q], offs[q]));
          }
          psum[q] = p0 + p1;
          split_parts<kSum>(PER_TOKEN ? p0 * vs_tok[0] : p0, hi[0][q], lo[0][q]);
          split_parts<kSum>(PER_TOKEN ? p1 * vs_tok[1] : p1, hi[1][q], lo[1][q]);
        }
        constexpr int W = (RC + 3) / 4;
#pragma unroll
        for (int tg = 0; tg < 2; ++tg) {
#pragma unroll
          for (int w = 0; w < W; ++w) {
            pbytes[tg][w] = pack_e4m3x4(hi[tg][4 * w], hi[tg][4 * w + 1], hi[tg][4 * w + 2], hi[tg][4 * w + 3]);
            pbytes[tg][W + w] = pack_e4m3x4(lo[tg][4 * w], lo[tg][4 * w + 1], lo[tg][4 * w + 2], lo[tg][4 * w + 3]);
          }
          // tile row n of the token is byte n of its 16: hi rows at q, lo rows at QR + q (their own tile with 16 rows)
          if constexpr (RC == 4) {
            sts64(p_at[tg], pbytes[tg][0], pbytes[tg][1]);
          } else {
            sts64(p_at[tg] + ch * 8, pbytes[tg][0], pbytes[tg][1]);
            sts64(p_at[tg] + (QR == 16 ? 4096 + ch * 8 : 8), pbytes[tg][2], pbytes[tg][3]);
          }
        }
        if (NCH > 1) row_sums(ch, psum);
      }
      __syncwarp();   // the query slot's scales were read until here
      if (lane == 0) mbar_arrive(bar(kBarQEmpty, slot));
      if (PER_TOKEN && r == 0) v_norm[par] = vnorm;
      if (wq == 0) stamp(6, i, 3);

      // Bytes of V past the context (absent pages, tokens past the end of the last page) may
      // hold anything, NaN patterns included, and 0 * NaN would poison O^T: clear them.
      if (it.ntok < kItemTokens) {
        const int vslot = i % NSV;
        if (i >= NSV) {
          // P.V of the slot's previous item was issued before QK^T of this one and products
          // complete in order, so its barrier is at most one phase behind; its completion in
          // turn means the slot's previous fill had landed, which makes the wait below valid.
          const int j = i - NSV;
          const uint32_t ju = (uint32_t)(j / NG);
          if (!wait(bar(kBarOFull, 2 * (j % NG) + (int)(ju & 1)), (ju >> 1) & 1)) return false;
        }
        if (!wait(bar(kBarVFull, vslot), (uint32_t)(i / NSV) & 1)) return false;
        const uint32_t vrow = v_ring + vslot * kHalfSlot;                  // this lane clears row = head dim r
        const bool v16 = BS == 16 || p.v_trans != 0;  // the slot holds [128 d][16 tok] runs
        auto v_at = [&](int g16) -> int { return v16 ? Geo<16>::v_chunk(r, g16) : G::v_chunk(r, g16); };
        const int first_bad = it.ntok >> 4;           // 16-token group holding the first invalid token
        const int keep = it.ntok & 15;                // valid tokens in that group
        for (int g16 = first_bad; g16 < 16; ++g16) {
          uint4 val = make_uint4(0u, 0u, 0u, 0u);
          if (g16 == first_bad && keep > 0) {
            val = lds128(vrow + v_at(g16));
            uint32_t w[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int nk = min(max(keep - 4 * k, 0), 4);
              w[k] &= nk >= 4 ? 0xffffffffu : ((1u << (8 * nk)) - 1u);
            }
            val = make_uint4(w[0], w[1], w[2], w[3]);
          }
          sts128(vrow + v_at(g16), val);
        }
      }
      fence_proxy_async();   // P^T and the cleared V bytes are read by the tensor core
      fence_before_sync();   // the S^T loads above are complete (tmem_ld_wait)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarPFull, grp));
      if (wq == 0) stamp(4, i, 2);
      // row sums, needed only by the epilogue of this item: off the path to P.V
      if (NCH == 1) row_sums(0, psum);
      return true;
    };

    // Single-launch form.  Item j of this group was the last partition of the set (it.seq, it.head)
    // that this CTA computes; the set's partitions are the rows [set_row0, set_end) of the index.
    //  * All of the CTA's earlier items are waited for first: the other two groups count the
    //    items they have stored (release), and an item of a set precedes the set's later ones.
    //  * A set that began in an earlier team belongs to the CTA that holds its first partition:
    //    one thread fences -- which makes this CTA's partitions, ordered before the fence by the
    //    counts, visible to the whole GPU -- and adds their number to the set's counter.
    //  * Otherwise this group merges the set, warp w the rows w and w + 4 (the arithmetic of
    //    pa_reduce_kernel<1>), after the counter has reached the number of partitions that later
    //    teams compute, if any.  Those teams meet the set at the START of their ranges and this
    //    CTA at the END of its own, so normally the count is complete long before it is looked at;
    //    a set longer than a team's range ends with the chain fence - count - poll - merge.
    //    The counter is cleared for the next launch.
    // Nobody waits for a group that merges, except through the pipeline's own barriers: the rings
    // absorb the microsecond or so.  Every poll is bounded.
    auto finish_set = [&](int j, const TcItem& it, int set_row0, int set_end) -> bool {
      auto poll = [&](auto&& ready) -> bool {
        bool ok = false;
        for (uint32_t w = 0; w < kSetPolls && !ok; ++w) {
          ok = ready();
          if (!ok) __nanosleep(64);
        }
        return __all_sync(kFullMask, ok);
      };
      named_barrier_sync(bar_b, 128);   // the four warps of this group have stored the item
      for (int g2 = 0; g2 < NG; ++g2) {
        if (g2 == grp) continue;
        const uint32_t before = j > g2 ? (uint32_t)((j - g2 + NG - 1) / NG) : 0u;   // items below j of that group
        const uint32_t at = sbase + kOffDone + 4 * g2;
        if (!poll([&]() { return ld_acquire_cta_shared(at) >= 4u * before; })) return false;
      }
      const int np = set_end - set_row0;
      const int own = set_row0 + it.part + 1 - max(set_row0, team.row0);   // partitions of the set computed here
      int32_t* counter = p.merge_counters + (it.seq * p.Hkv + it.head);
      if (set_row0 < team.row0) {
        if (wq == 0 && lane == 0) {
          __threadfence();
          atomicAdd(counter, own);
        }
        return true;
      }
      if (own < np) {
        if (!poll([&]() { return ld_relaxed_gpu(counter) == np - own; })) return false;
        __threadfence();   // the partitions counted into the set are visible from here on
      }
      for (int row = wq; row < p.eqG; row += 4) {
        const int64_t ws_row = (int64_t)it.seq * p.ws_stride_seq + (int64_t)it.head * p.ws_stride_head + row;
        const int64_t tmp_row = (int64_t)it.seq * p.tmp_stride_seq + (int64_t)it.head * p.tmp_stride_head +
                                (int64_t)row * p.tmp_stride_row + 4 * lane;
        const bool has_sink = p.sink != nullptr;
        const float sink_logit = has_sink ? __ldg(p.sink + it.head * p.G + row % p.G) : 0.f;
        merge_row_one_chunk(p.max_logits, p.exp_sums, p.tmp_out, ws_row, p.ws_stride_part, tmp_row, p.tmp_stride_part,
                            np, sink_logit, has_sink,
                            p.out + 2 * ((int64_t)it.seq * p.out_stride_seq + ((int64_t)it.head * p.eqG + row) * p.out_stride_head),
                            lane);
      }
      if (own < np) {   // every warp of the group has seen the count: clear it
        named_barrier_sync(bar_b, 128);
        if (wq == 0 && lane == 0) *counter = 0;
      }
      return true;
    };

    // `tail`: no softmax of a later item of this group ran in between, so the row sums of item j
    // still need a barrier of their own to be visible to the whole group.
    // PAIR form: waits (bounded) until every item of this CTA below `limit` has been stored or
    // stashed by its group (the groups count their finished epilogues, release / acquire)
    auto items_below_done = [&](int limit) -> bool {
      for (int g2 = 0; g2 < NG; ++g2) {
        if (g2 == grp) continue;   // this group's own earlier items are behind it in program order
        const uint32_t before = limit > g2 ? (uint32_t)((limit - g2 + NG - 1) / NG) : 0u;
        const uint32_t at = sbase + kOffDone + 4 * g2;
        bool ok = false;
        for (uint32_t w = 0; w < kSetPolls && !ok; ++w) {
          ok = ld_acquire_cta_shared(at) >= 4u * before;
          if (!ok) __nanosleep(32);
        }
        if (!__all_sync(kFullMask, ok)) return false;
      }
      return true;
    };
    // PAIR form: where the first half of a partition leaves its result for the second half.  Two
    // buffers, taken by the first half's item number: [QR rows][128 dims] bf16 outputs (what the
    // partition would hold in the workspace if it ended there), then per row the maximum (base-2
    // domain) and the sum (units of 1/256) in fp32; behind the buffers, per group and parity, the
    // first half's weight per row.  (bf16: with fp32 outputs the buffers would cost 8-row items a
    // stage of the V ring.)
    constexpr int kStashBytes = QR * kD * 2 + 2 * 16 * 4;
    float* g_first = reinterpret_cast<float*>(smem + p.off_stash + 2 * kStashBytes);   // [groups][2 parities][16]

    auto epilogue = [&](int j, const TcItem& it, bool tail) -> bool {
      const uint32_t gu = (uint32_t)(j / NG);
      const int par = grp * 2 + (int)(gu & 1);
      const float* rs = red_sum + par * 64;
      // PAIR form: 0 = a partition of one item, 1 = first half (stash), 2 = second half (merge and store)
      const int half = !PAIR || !it.paired ? 0 : 1 + it.sub;
      uint8_t* st_raw = smem + p.off_stash + (((half == 2 ? j - 1 : j) >> 1) & 1) * kStashBytes;
      unsigned short* st_o = reinterpret_cast<unsigned short*>(st_raw);            // [QR][128] bf16
      float* st = reinterpret_cast<float*>(st_raw + QR * kD * 2);                  // [16] maxima, [16] sums
      if (tail) named_barrier_sync(bar_b, 128);
      if (wq == 0) stamp(5, j, 0);
      if (PAIR && half != 0) {
        // second half: the first half (item j - 1, another group's) must be stashed.  First half: the
        // buffer's previous reader is item j - 2 at the latest (see the buffer choice above).
        if (!items_below_done(half == 2 ? j : j - 1)) return false;
      }
      if (!wait(bar(kBarOFull, par), (gu >> 1) & 1)) return false;
      if (wq == 0) stamp(5, j, 1);
      fence_after_sync();
      const float vfin = PER_TOKEN ? v_norm[par] : v_scale_t;
      const int rows = min(QR, p.eqG - it.rb * QR);   // valid rows of this block
      // thread `row` of the group: the row's sum, the factor of its O^T values, and the row's
      // partition maximum and exponential sum for the workspaces
      if (r < QR) {
        const float4 l4 = *reinterpret_cast<const float4*>(rs + r * 4);
        const float lsum = (l4.x + l4.y) + (l4.z + l4.w);   // in units of 1/256
        const int64_t ws = (int64_t)it.seq * p.ws_stride_seq + (int64_t)it.head * p.ws_stride_head +
                           (int64_t)it.part * p.ws_stride_part + it.rb * QR + r;
        if (PAIR && half == 1) {
          f_row[par * 16 + r] = lsum > 0.f ? __fdividef(vfin, lsum) : 0.f;
          st[r] = m_fin[par * 16 + r];
          st[16 + r] = lsum;
        } else if (PAIR && half == 2) {
          // log-sum-exp merge of the two halves (pa_decode_triton_gluon_fp8.py:1187-1333 does the
          // same across partitions): weights relative to the common maximum
          const float m_a = st[r], l_a = st[16 + r], m_b = m_fin[par * 16 + r];
          const float m = fmaxf(m_a, m_b);
          const float e_a = (l_a > 0.f && m_a > -INFINITY) ? ex2(m_a - m) : 0.f;
          const float e_b = (lsum > 0.f && m_b > -INFINITY) ? ex2(m_b - m) : 0.f;
          const float l = l_a * e_a + lsum * e_b;
          const float inv = l > 0.f ? __fdividef(1.0f, l) : 0.f;
          g_first[par * 16 + r] = l_a * e_a * inv;   // the first half's outputs are already divided by its sum
          f_row[par * 16 + r] = vfin * e_b * inv;
          if (r < rows) {
            p.max_logits[ws] = m * kLn2;
            p.exp_sums[ws] = l * (1.0f / 256.0f);
          }
        } else {
          f_row[par * 16 + r] = lsum > 0.f ? __fdividef(vfin, lsum) : 0.f;
          if (r < rows) {
            p.max_logits[ws] = m_fin[par * 16 + r] * kLn2;
            p.exp_sums[ws] = lsum * (1.0f / 256.0f);
          }
        }
      }
      named_barrier_sync(bar_b, 128);
      // lane r holds head dim r of every row: 2-byte stores, 64 contiguous bytes per warp and row
      unsigned short* dst = reinterpret_cast<unsigned short*>(p.tmp_out) + (int64_t)it.seq * p.tmp_stride_seq +
                            (int64_t)it.head * p.tmp_stride_head + (int64_t)it.part * p.tmp_stride_part +
                            (int64_t)(it.rb * QR) * p.tmp_stride_row + r;
      const int64_t row_stride = p.tmp_stride_row;
      const uint32_t otile = tmem_grp + 2 * N + (int)(gu & 1) * N;
#pragma unroll 1
      for (int ch = 0; ch < NCH; ++ch) {
        uint32_t h[8], l[8];
        load_rows(otile, ch, h, l);
        float f[RC];
#pragma unroll
        for (int q4 = 0; q4 < RC; q4 += 4) {
          const float4 f4 = *reinterpret_cast<const float4*>(f_row + par * 16 + ch * RC + q4);
          f[q4] = f4.x, f[q4 + 1] = f4.y, f[q4 + 2] = f4.z, f[q4 + 3] = f4.w;
        }
        tmem_ld_wait();
        if (wq == 0) stamp(7, j, 2 * ch);
#pragma unroll
        for (int q = 0; q < RC; ++q) {
          float o = row_value(h, l, q) * f[q];
          if (PAIR && half == 1) {          // thread r keeps its head dim of every row for the second half
            st_o[(ch * RC + q) * kD + r] = (unsigned short)(pack_bf16x2(o, 0.f) & 0xffffu);
          } else {
            if (PAIR && half == 2)
              o = fmaf(__uint_as_float((uint32_t)st_o[(ch * RC + q) * kD + r] << 16), g_first[par * 16 + ch * RC + q], o);
            if (ch * RC + q < rows) *dst = (unsigned short)(pack_bf16x2(o, 0.f) & 0xffffu);
          }
          dst += row_stride;
        }
        if (wq == 0) stamp(7, j, 2 * ch + 1);
      }
      fence_before_sync();  // the O^T loads are ordered before this warp's next arrival on the P barrier
      if constexpr (PAIR) {
        // this warp's part of the item is stored or stashed (and what it read of the stash is read): count it
        __syncwarp();
        if (lane == 0) red_release_cta_add(sbase + kOffDone + 4 * grp, 1u);
      }
      if constexpr (FUSE) {
        // this warp's stores of the item are issued: count it (a release at CTA scope)
        __syncwarp();
        if (lane == 0) red_release_cta_add(sbase + kOffDone + 4 * grp, 1u);
        // Was this the last partition of its (sequence, kv head) that this CTA computes -- the
        // set's last partition, or the one in the last row of the team's range?
        const int set_row0 = seq_off[it.seq], set_end = seq_off[it.seq + 1];
        const int row = set_row0 + it.part;
        if ((row + 1 == set_end || row + 1 == team.row0 + team.rows) && !finish_set(j, it, set_row0, set_end)) return false;
      }
      if (wq == 0) stamp(5, j, 2);
      return true;
    };

    // group g walks the CTA's items g, g+NG, ...; the epilogue of an item runs after the softmax
    // of the group's next item, by which time its P.V product has long been issued
    // (With the item in the slot, the softmax fills it0 in and none of the cursor code below exists.)
    Cursor cur;
    if (!kItemFromSlot && grp < n_local) cur.init(first + grp * stride, NG * stride, p, seq_off, seq_ctx);
    // the group's current item and the two after it (for the scale prefetch)
    TcItem it0{}, it1{}, it2{};
    int pid1[2] = {0, 0};            // block-table entries of it1's pages, in flight
    float sc0[4] = {0.f, 0.f, 0.f, 0.f};   // token scales of it0, in flight
    if (!kItemFromSlot && grp < n_local) {
      it0 = cur.item(p, seq_off, seq_ctx);
      if (PER_TOKEN) {
        int pid0[2];
        load_tok_pids(it0, pid0);
        load_tok_scales(it0, pid0, sc0);
      }
    }
    if (!kItemFromSlot && grp + NG < n_local) {
      cur.advance(p, seq_off);
      it1 = cur.item(p, seq_off, seq_ctx);
      load_tok_pids(it1, pid1);
    }
    TcItem it_prev{};
    int prev = -1;
    // one call site each for softmax and epilogue: the code of this loop should stay small
    for (int i = grp; !dead; i += NG) {
      const bool more = i < n_local;
      if (wq == 0) stamp(4, i, 3);
      if (more) {
        float sc_use[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) sc_use[e] = sc0[e];
        if (!kItemFromSlot && PER_TOKEN && i + NG < n_local) load_tok_scales(it1, pid1, sc0);
        if (!kItemFromSlot && i + 2 * NG < n_local) {
          cur.advance(p, seq_off);
          it2 = cur.item(p, seq_off, seq_ctx);
          load_tok_pids(it2, pid1);
        }
        if (!softmax(i, it0, sc_use)) { fail(); break; }
      }
      if (prev >= 0 && !epilogue(prev, it_prev, !more)) { fail(); break; }
      if (!more) break;
      it_prev = it0;
      prev = i;
      if (!kItemFromSlot) {
        it0 = it1;
        it1 = it2;
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  __syncwarp();
  fence_before_sync();
  __syncthreads();
  if (TRACE && p.trace != nullptr && blockIdx.x == 0 && tid == 0)
    p.trace[(7 * 64 + 60) * 4 + 3] = (unsigned long long)clock64();
  if (warp == kWarpMma) {
    fence_after_sync();
    tmem_dealloc(tmem_base, tmem_cols(QR));
  }
}

}  // namespace tc
}  // namespace pa
