// Device kernels of the B200 paged-attention decode library (sm_100a).
//
// One templated attention kernel serves the four entry points:
//   MODE_LOOP   one (sequence, KV-head group) per thread-block cluster, the context
//               split over the cluster's CTAs and merged through distributed
//               shared memory; writes `out`
//               (reference paged_attention_loop_kernel, paged_attention_kernel_loop.hpp:42-637)
//   MODE_SPLIT  persistent CTAs walking (sequence, partition, KV-head group) items;
//               writes max_logits, exp_sums and the fp16 partial output
//               (reference paged_attention_kernel, paged_attention_kernel_v2.hpp:42-588)
// with the KV cache stored as fp16, e5m2 or e4m3 (FP8 dequantised in
// registers, reference paged_attention_kernel_fp8_loop.hpp:270-278,328-333,540-545).
// merge_partitions_kernel is the second kernel of the split variant
// (reference paged_attention_reduce, paged_attention_kernel_v2.hpp:594-970).
//
// Structure of the attention kernel: warp 0 walks the block table and issues
// tiled TMA copies (one box per KV block and 128-byte slab, spanning the CTA's KV
// heads where a block fills the stage) into a ring of shared-memory stages guarded
// by full/empty mbarriers; warps 1..4 each own a 16-row tile of every tile step of
// a stage (TILES = 1, 2 or 4 steps per stage: larger stages mean larger copies for
// KV blocks of 32 tokens and more).  A CTA works on `hpc` (1, 2 or 4) neighbouring
// KV heads at once: with hpc = 4 a warp owns one KV head and sees every token of
// the item, so nothing has to be merged across warps; with fewer heads the warps
// split the tokens and merge through shared memory in a fixed order.  A second
// shape of the same kernel (NWARPS = 8: warps 1..8, hpc = 8, one CTA per SM, a ring
// twice as large) serves FP8 caches in split mode; a warp does the same work on
// its head in both shapes, so they give the same bits.  The GQA query group sits
// on the N=8 extent of mma.m16n8k16 and the tokens on M, so a KV byte is read from
// HBM once for the whole group:
//   S^T[tok, g] = K[tok, d] . Q^T[d, g]          (A = K via ldmatrix)
//   O^T[d, g]  += V^T[d, tok] . P^T[tok, g]      (A = V via ldmatrix.trans)
// Softmax is online per warp in the log2 domain with warp-shuffle column
// maxima; the accumulator is rescaled only when the running maximum has grown
// by more than kRescaleThreshold.  Every wait on an mbarrier is bounded
// (pa::mbar_wait_bounded).
#pragma once

#include <atomic>

#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "paged_attention_policy_v2.hpp"
#include "paged_attention_utils.hpp"

namespace pa {

enum Mode : int { MODE_LOOP = 0, MODE_SPLIT = 1 };

// Set when a bounded wait gave up; read and cleared by pa_device_status().
// One copy per translation unit (the launchers are compiled separately).
static __device__ int g_pa_device_status = 0;

// Work counters of the split kernel's dynamic scheduler: [slot][0] hands out item numbers,
// [slot][1] counts retired CTAs; the last CTA of a launch zeroes its slot again.  The table
// exists once per translation unit and is shared by every kernel instantiation of that unit,
// so the unit also has exactly one slot allocator (next_sched_slot below): consecutive
// launches of the unit, whatever their instantiation and stream, take consecutive slots, and
// launches that overlap in time (other streams, programmatic dependent launch) never share
// one unless more than kDirectSchedSlots of them are in flight at once.  A launch recorded
// into a CUDA graph keeps its slot for every replay, so recorded launches draw from a range of
// their own (the upper half of the table) that direct launches never touch; two replays of one
// graph never overlap, and different recordings hold different slots (up to kSchedSlots -
// kDirectSchedSlots recorded launches per unit before the range wraps).
constexpr uint32_t kSchedSlots = 1024;
constexpr uint32_t kDirectSchedSlots = 512;
static __device__ unsigned int g_sched[kSchedSlots][2];
static std::atomic<uint32_t> g_next_direct_slot{0};
static std::atomic<uint32_t> g_next_captured_slot{0};

static inline uint32_t next_sched_slot(bool capturing) { // static like the counters it advances: one per unit
  if (capturing)
    return kDirectSchedSlots +
           g_next_captured_slot.fetch_add(1, std::memory_order_relaxed) % (kSchedSlots - kDirectSchedSlots);
  return g_next_direct_slot.fetch_add(1, std::memory_order_relaxed) % kDirectSchedSlots;
}

// Per-CTA time stamps (%globaltimer, ns), compiled in with -DPA_TIMELINE only: a measuring aid
// for the launch ramp and the tail of a launch.  One row per CTA of the most recent launch of
// this translation unit: [0] kernel entry, [1] after the wait for the previous kernel,
// [2] first copy issued, [3] first stage complete, [4] last stage of the last item consumed,
// [5] exit, [6] work items done, [7] loop mode: the cluster has met for the merge (else 0).
#ifdef PA_TIMELINE
constexpr uint32_t kTimelineCtas = 4096;
static __device__ unsigned long long g_timeline[kTimelineCtas][8];
#define PA_STAMP(slot)                                                                          \
  do {                                                                                          \
    if (timeline_cta < kTimelineCtas) g_timeline[timeline_cta][slot] = global_timer_ns();       \
  } while (0)
#define PA_STAMP_VALUE(slot, v)                                                                 \
  do {                                                                                          \
    if (timeline_cta < kTimelineCtas) g_timeline[timeline_cta][slot] = (v);                     \
  } while (0)
#else
#define PA_STAMP(slot) do { } while (0)
#define PA_STAMP_VALUE(slot, v) do { } while (0)
#endif

// Range-checked build (-DPA_DEBUG_BOUNDS): every index that the block tables and context
// lengths can move is checked where it is formed, and the first value found out of range is
// recorded here instead of being cut or zero-filled silently: [0] findings so far, then the
// first one as [1] kind, [2] index, [3] limit, [4] sequence, [5] token.  The access itself is
// made safe either way (index 0 / cut length), so a finding never faults.  One table per
// translation unit, read and cleared by that unit's pa_debug_bounds_* export.
enum BoundsKind : unsigned int {
  BOUNDS_TABLE_INDEX = 1,   // block-table column beyond the sequence's row
  BOUNDS_BLOCK_ID = 2,      // block id >= num_blocks
  BOUNDS_CONTEXT_LENGTH = 3 // context length beyond what the row addresses
};
#ifdef PA_DEBUG_BOUNDS
static __device__ unsigned int g_bounds_report[8];
__device__ __forceinline__ bool bounds_ok(unsigned int kind, uint64_t index, uint64_t limit, uint32_t seq,
                                          uint32_t tok) {
  if (index < limit) return true;
  if (atomicAdd(&g_bounds_report[0], 1u) == 0u) {
    g_bounds_report[1] = kind;
    g_bounds_report[2] = static_cast<unsigned int>(min(index, static_cast<uint64_t>(0xffffffffu)));
    g_bounds_report[3] = static_cast<unsigned int>(min(limit, static_cast<uint64_t>(0xffffffffu)));
    g_bounds_report[4] = seq;
    g_bounds_report[5] = tok;
  }
  return false;
}
#endif

struct AttnArgs {
  const __half *query;
  __half *out;
  float *max_logits;
  float *exp_sums;
  __half *tmp_out;
  const __half *sinks; // nullable
  const uint32_t *block_tables;
  const uint32_t *context_lens;
  uint32_t num_seqs;
  uint32_t num_heads;
  uint32_t num_kv_heads;
  uint32_t group;
  uint32_t max_blocks_per_seq;
  uint32_t num_blocks;       // blocks in the cache: the bound of every block id
  uint32_t max_num_partitions;
  uint32_t block_shift;      // log2(block_size)
  uint32_t hpc;              // KV heads per CTA: 1, 2, 4, or 8 in the wide CTA (divides num_kv_heads)
  uint32_t tokens_per_stage; // 64 / hpc
  uint32_t rows_per_box;     // min(block_size, tokens_per_stage)
  uint32_t boxes_per_stage;  // hpc * tokens_per_stage / rows_per_box: 1, 2 or 4
  uint32_t heads_per_box;    // KV heads one TMA box covers: hpc if rows_per_box == tokens_per_stage, else 1
  float scale_log2;          // sm_scale * fp8_scale * log2(e), > 0
  float out_scale;           // fp8_scale (1 for fp16)
  // optional per-KV-head dequantisation scales of an FP8 cache, [num_kv_heads] each; when
  // set they take the place of fp8_scale for K and for V
  const float *k_scale_per_head;
  const float *v_scale_per_head;
  // optional per-block dequantisation scales of an FP8 cache, [num_blocks, num_kv_heads] each
  // (both or neither): the producer stages them in shared memory beside every ring stage
  const float *k_scale_per_block;
  const float *v_scale_per_block;
  float sm_scale_log2;       // sm_scale * log2(e)
  uint32_t sched_slot;       // row of g_sched this launch uses (split mode)
  // split mode: log2 of the partition size in tokens
  uint32_t partition_shift;
  // split mode run on behalf of the loop variant (many short sequences): a work item is the whole
  // context of a (sequence, head group), its normalised result goes straight to `out`, and the
  // scratch tensors are neither read nor written (they may be null)
  uint32_t whole_context_items;
  // max_blocks_per_seq * block_size (saturated to 32 bits): a context length beyond it is cut
  // to it, so no block-table read leaves the sequence's row whatever context_lens holds
  uint32_t ctx_limit;
  // optional packed block tables: when set, block_tables is one list of block ids and the row
  // of sequence i is block_tables[table_offsets[i] .. table_offsets[i + 1]); the limit of a
  // context then is the length of its own row
  const uint32_t *table_offsets;
  // optional list of the sequences this launch covers (num_seqs entries); all tensors are
  // still indexed by the sequence ids found in the list
  const uint32_t *seq_indices;
  // loop mode: context-length hint used to launch long sequences first (0 = keep the order)
  uint32_t longest_first_hint;
  // opt-in score modifiers (off in the reference, whose call sites are commented out,
  // paged_attention_kernel_loop.hpp:329-342): soft-cap s -> cap * tanh(s / cap), then an ALiBi
  // bias slope[h] * (t - (ctx - 1)) on the score of token t
  const float *alibi_slopes; // fp32 [num_heads] or null
  float softcap;             // > 0 enables the soft-cap
};

constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLog2e = 1.4426950408889634f;
// The exponent reference of the online softmax follows the running maximum only in
// steps larger than this (log2 units), so weights stay below 2^8 and most tiles skip
// the rescaling of the accumulator.
constexpr float kRescaleThreshold = 8.0f;

template <int D, int KV, int NWARPS = 4, int TILES = 1>
struct SmemLayout {
  using policy = paged_attention_policy_v2<D, KV, NWARPS, TILES>;
  using geo = typename policy::geometry;
  static constexpr uint32_t NW = policy::consumer_warps;
  // rows of a stage: hpc heads x (64 * TILES / hpc) tokens, head-major
  static constexpr uint32_t ROWS = policy::tokens_per_stage;
  static constexpr uint32_t NSTAGES = policy::ring_stages;
  static constexpr uint32_t SLAB_TILE = ROWS * geo::slab_bytes;   // one slab of one stage
  static constexpr uint32_t KV_TILE = geo::num_slabs * SLAB_TILE; // K (or V) of one stage
  static constexpr uint32_t STAGE_BYTES = 2 * KV_TILE;
  static constexpr uint32_t RING_BYTES = NSTAGES * STAGE_BYTES;
  static_assert(NW == 4 || NW == 8, "warp <-> (head, token slice) mapping: 4 warps, or 8 with one head per warp");
  // split mode, fewer than 4 heads per CTA: two O[8][D] buffers filled in a fixed order
  static constexpr uint32_t MERGE_OFFSET = RING_BYTES;
  static constexpr uint32_t MERGE_BYTES = (NWARPS == 8) ? 0 : 2 * 8 * D * 4; // the wide CTA never merges
  // per-warp (reference max, true max, sum) of the 8 query columns, double-buffered by item parity
  static constexpr uint32_t WARP_STATS_OFFSET = MERGE_OFFSET + MERGE_BYTES;
  static constexpr uint32_t WARP_STATS_FLOATS = 3 * NW * 8;
  static constexpr uint32_t WARP_STATS_BYTES = 2 * WARP_STATS_FLOATS * 4;
  static constexpr uint32_t BAR_OFFSET = WARP_STATS_OFFSET + WARP_STATS_BYTES;
  // after the ring barriers: abort flag (16 B), then the item queue between the producer and
  // the consumers: two entries, each an item number and a full / empty mbarrier pair
  static constexpr uint32_t SCHED_OFFSET = BAR_OFFSET + 2 * NSTAGES * 8 + 16;
  // per-block FP8 scales of a stage: (K scale, V scale) for each of its at most 8 (block, head)
  // pairs -- 4 blocks of one head up to 1 block of 8 heads
  static constexpr uint32_t SCALE_SLOTS = 8;
  static constexpr uint32_t SCALES_OFFSET = SCHED_OFFSET + 4 * 8 + 16;
  static constexpr uint32_t TOTAL_BYTES = SCALES_OFFSET + NSTAGES * SCALE_SLOTS * 8;
  static constexpr uint32_t DYN_SMEM = TOTAL_BYTES + 1024; // slack for 1024-byte alignment
  // loop mode: every warp parks (O[8][D], m[8], l[8]) on the (by then idle) ring for the
  // cluster-wide merge
  static constexpr uint32_t WARP_AREA_FLOATS = 8 * D + 16;
  static_assert(NW * WARP_AREA_FLOATS * 4 <= RING_BYTES, "cluster merge scratch must fit in the ring");
};

// d index of accumulator tile `tile`, row half `h` (0: rows gid, 1: rows gid+8)
template <int KV>
__device__ __forceinline__ uint32_t acc_dim_index(uint32_t tile, uint32_t h, uint32_t gid) {
  if constexpr (KV == KV_F16) {
    return tile * 16u + h * 8u + gid;
  } else {
    // FP8: tiles come in (even, odd) byte pairs of a 32-dim group
    return (tile >> 1) * 32u + h * 16u + 2u * gid + (tile & 1u);
  }
}

// One unit of work of a CTA: tokens [tok_begin, tok_end) of KV heads
// [head_base, head_base + hpc) of one sequence.
struct WorkItem {
  uint32_t linear; // item number (split mode), see SplitCursor
  uint32_t seq, head_base, partition;
  uint32_t tok_begin, tok_end;
  uint32_t ctx; // context length of the sequence
  uint32_t table_off; // packed block tables: first entry of the sequence's row
  bool valid;
};

// Context length of sequence `seq`, cut to what its block-table row can address, and (packed
// tables) the offset of that row.
__device__ __forceinline__ uint32_t load_context(const AttnArgs &args, uint32_t seq, uint32_t &table_off) {
  const uint32_t ctx = __ldg(args.context_lens + seq);
  if (args.table_offsets == nullptr) {
    table_off = 0u;
#ifdef PA_DEBUG_BOUNDS
    bounds_ok(BOUNDS_CONTEXT_LENGTH, ctx, static_cast<uint64_t>(args.ctx_limit) + 1u, seq, ctx);
#endif
    return min(ctx, args.ctx_limit);
  }
  table_off = __ldg(args.table_offsets + seq);
  const uint64_t row_tokens = static_cast<uint64_t>(__ldg(args.table_offsets + seq + 1) - table_off) << args.block_shift;
#ifdef PA_DEBUG_BOUNDS
  bounds_ok(BOUNDS_CONTEXT_LENGTH, ctx, row_tokens + 1u, seq, ctx);
#endif
  return static_cast<uint32_t>(min(static_cast<uint64_t>(ctx), row_tokens));
}

// Split mode: the work items are the (sequence, partition, head group) triples whose partition
// starts inside the context, numbered densely with the head group fastest (CTAs that run
// together stream neighbouring rows of the same KV blocks) and the sequence slowest; CTA b
// starts with item b and draws every further number from the launch's counter.  Partitions
// past a context have no number, so their scratch rows stay untouched (reference
// paged_attention_kernel_v2.hpp:194-200,577-579) and ragged batches spread evenly.
//
// The numbering needs the running sum of items per sequence.  A warp keeps a window of 32
// sequences in registers (one per lane) and moves it forward as its item numbers grow, so the
// context lengths are read once per warp over the life of the kernel.  Every method is
// called by all 32 lanes of a warp together.
struct SplitCursor {
  uint32_t window_seq;     // first sequence of the window (multiple of 32)
  uint32_t items_before;   // items of all sequences before the window
  uint32_t lane_seq;       // id of the (window_seq + lane)-th sequence of the launch
  uint32_t lane_ctx;       // its context length (0 past the end of the launch)
  uint32_t lane_off;       // packed block tables: offset of its row
  uint32_t lane_incl;      // items of sequences window_seq .. window_seq + lane (inclusive scan)
  uint32_t window_items;   // items of the whole window

  // partitions of a context that have a number; with whole-context items every sequence of the
  // launch, an empty one included, is exactly one (its output row has to be written)
  static __device__ __forceinline__ uint32_t parts_of(const AttnArgs &args, uint32_t ctx) {
    if (args.whole_context_items != 0u) return 1u;
    const uint32_t psize = 1u << args.partition_shift;
    return min((ctx + psize - 1u) >> args.partition_shift, args.max_num_partitions);
  }

  __device__ __forceinline__ void load_window(const AttnArgs &args, uint32_t groups, uint32_t lane) {
    const uint32_t pos = window_seq + lane;
    lane_seq = (pos < args.num_seqs) ? (args.seq_indices != nullptr ? __ldg(args.seq_indices + pos) : pos) : 0u;
    lane_off = 0u;
    lane_ctx = (pos < args.num_seqs) ? load_context(args, lane_seq, lane_off) : 0u;
    const uint32_t parts = (pos < args.num_seqs) ? parts_of(args, lane_ctx) : 0u;
    uint32_t v = parts * groups;
#pragma unroll
    for (uint32_t o = 1; o < 32; o <<= 1) {
      const uint32_t up = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += up;
    }
    lane_incl = v;
    window_items = __shfl_sync(0xffffffffu, v, 31);
  }

  __device__ __forceinline__ void init(const AttnArgs &args, uint32_t groups, uint32_t lane) {
    window_seq = 0;
    items_before = 0;
    if (args.whole_context_items != 0u) return; // the numbering needs no running sums there
    load_window(args, groups, lane);
  }

  // Item number `index` (never smaller than the previous one asked for) -> work item.
  __device__ __forceinline__ WorkItem seek(uint32_t index, const AttnArgs &args, uint32_t groups,
                                           uint32_t lane) {
    WorkItem it{};
    it.valid = false;
    if (args.whole_context_items != 0u) {
      // every sequence has `groups` items: the number gives the sequence directly.  (Walking the
      // windows instead costs a CTA several dependent loads per draw when the items are small:
      // between two draws of one CTA all the others have moved the numbering on by several windows.)
      const uint32_t pos = index / groups;
      if (pos >= args.num_seqs) return it; // past the last item
      it.linear = index;
      it.seq = (args.seq_indices != nullptr) ? __ldg(args.seq_indices + pos) : pos;
      it.partition = 0u;
      it.head_base = (index - pos * groups) * args.hpc;
      it.table_off = 0u;
      it.ctx = load_context(args, it.seq, it.table_off);
      it.tok_begin = 0u;
      it.tok_end = it.ctx;
      it.valid = true;
      return it;
    }
    if (index < items_before) init(args, groups, lane); // never happens with increasing numbers
    while (index >= items_before + window_items) {
      if (window_seq + 32 >= args.num_seqs) return it; // past the last item
      items_before += window_items;
      window_seq += 32;
      load_window(args, groups, lane);
    }
    const uint32_t local = index - items_before;
    // the owning sequence is the first lane whose inclusive count exceeds `local`
    const uint32_t owner = __ffs(__ballot_sync(0xffffffffu, lane_incl > local)) - 1u;
    const uint32_t incl = __shfl_sync(0xffffffffu, lane_incl, owner);
    const uint32_t ctx = __shfl_sync(0xffffffffu, lane_ctx, owner);
    const uint32_t parts = parts_of(args, ctx);
    const uint32_t within = local - (incl - parts * groups); // item number inside the sequence
    it.linear = index;
    it.seq = __shfl_sync(0xffffffffu, lane_seq, owner);
    it.partition = within / groups;
    it.head_base = (within - it.partition * groups) * args.hpc;
    if (args.whole_context_items != 0u) {
      it.tok_begin = 0u;
      it.tok_end = ctx;
    } else {
      it.tok_begin = it.partition << args.partition_shift;
      it.tok_end = min(ctx, it.tok_begin + (1u << args.partition_shift));
    }
    it.ctx = ctx;
    it.table_off = __shfl_sync(0xffffffffu, lane_off, owner);
    it.valid = true;
    return it;
  }
};

template <int D, int KV>
__device__ __forceinline__ void load_q_fragments(uint32_t (&qf)[D / 16][2], const AttnArgs &args,
                                                 uint32_t seq, uint32_t kv_head, uint32_t gid,
                                                 uint32_t t4) {
  // B operand of S^T = K . Q^T: column n = gid is the query head inside the group
  const uint32_t G = args.group;
  const __half *qrow = args.query + (static_cast<size_t>(seq) * args.num_heads + kv_head * G + gid) * D;
#pragma unroll
  for (uint32_t ks = 0; ks < D / 16; ++ks) {
    if (gid < G) {
      if constexpr (KV == KV_F16) {
        qf[ks][0] = __ldg(reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 2 * t4));
        qf[ks][1] = __ldg(reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 8 + 2 * t4));
      } else {
        // FP8 K fragments take 4 consecutive bytes per lane, so the k slots of an MMA
        // step map to dims 16*ks + 4*t4 + {0,1} and + {2,3}
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(qrow + ks * 16 + 4 * t4));
        qf[ks][0] = v.x;
        qf[ks][1] = v.y;
      }
    } else {
      qf[ks][0] = 0u;
      qf[ks][1] = 0u;
    }
  }
}

// Loop mode: merge of the partial results that the warps of a cluster have parked in their
// shared memory (per warp: O[8][D], then m[8], then l[8], WARP_AREA floats apart), through
// distributed shared memory.
//
// A unit of the merge is one output row (KV head hh of the CTA's group, query column g) times
// one chunk of 32 dims.  Unit u belongs to CTA u mod num_ranks and, there, to warp
// (u / num_ranks) mod NW.  The sources of a row are the R = num_ranks * slices warps that hold a
// part of its tokens; lane j of the merging warp fetches source j's (m, l), so the row
// statistics take one round trip, and the partial rows of UB units from JB sources each are
// requested together before the first is used.  All sums run in a fixed order.
template <int D, uint32_t NW, uint32_t WARP_AREA, uint32_t UB, uint32_t JB>
__device__ __noinline__ void merge_cluster_rows(float *areas, __half *out, const float *v_scale_per_head,
                                                float out_scale, uint32_t G, uint32_t num_heads, uint32_t seq,
                                                uint32_t head_base, uint32_t hpc, uint32_t cta_rank,
                                                uint32_t num_ranks, uint32_t cw, uint32_t lane, bool ok) {
  const cooperative_groups::cluster_group cluster = cooperative_groups::this_cluster();
  const uint32_t slices = NW / hpc;           // 1, 2 or 4: a power of two
  const uint32_t slice_shift = 31u - __clz(slices);
  const uint32_t R = num_ranks * slices;      // <= 8 * 4 = 32
  constexpr uint32_t CHUNKS = D / 32;
  const uint32_t units = hpc * G * CHUNKS;
  // lane j < R looks at source j: warp (j mod slices) of the row's head in CTA j / slices
  const float *lane_src = cluster.map_shared_rank(areas, (lane < R) ? (lane >> slice_shift) : 0u) +
                          (lane & (slices - 1u)) * WARP_AREA;
#pragma unroll 1
  for (uint32_t k0 = cw; cta_rank + num_ranks * k0 < units; k0 += NW * UB) {
    uint32_t row_g[UB], head_area[UB], chunk[UB], kv_head[UB];
    bool valid[UB];
    float f[UB], l_all[UB], m_src[UB], l_src[UB];
#pragma unroll
    for (uint32_t q = 0; q < UB; ++q) {
      const uint32_t u = cta_rank + num_ranks * (k0 + q * NW);
      valid[q] = u < units;
      const uint32_t row = valid[q] ? u / CHUNKS : 0u;
      chunk[q] = valid[q] ? u % CHUNKS : 0u;
      const uint32_t hh = row / G;
      row_g[q] = row - hh * G;
      kv_head[q] = head_base + hh;
      head_area[q] = (hh << slice_shift) * WARP_AREA; // first warp area of the row's head
      m_src[q] = neg_infinity();
      l_src[q] = 0.f;
      if (valid[q] && lane < R) {
        const float *pa = lane_src + head_area[q] + 8 * D;
        m_src[q] = pa[row_g[q]];
        l_src[q] = pa[8 + row_g[q]];
      }
    }
#pragma unroll
    for (uint32_t q = 0; q < UB; ++q) {
      float m_all = m_src[q];
#pragma unroll
      for (uint32_t o = 16; o > 0; o >>= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
      f[q] = (m_src[q] == neg_infinity()) ? 0.f : fast_exp2(m_src[q] - m_all);
      float l_sum = f[q] * l_src[q];
#pragma unroll
      for (uint32_t o = 16; o > 0; o >>= 1) l_sum += __shfl_xor_sync(0xffffffffu, l_sum, o);
      l_all[q] = l_sum;
    }
    float o_all[UB];
#pragma unroll
    for (uint32_t q = 0; q < UB; ++q) o_all[q] = 0.f;
#pragma unroll 1
    for (uint32_t j0 = 0; j0 < R; j0 += JB) {
      float v[UB][JB];
#pragma unroll
      for (uint32_t jj = 0; jj < JB; ++jj) {
        const uint32_t j = j0 + jj;
        const float *pj = cluster.map_shared_rank(areas, (j < R) ? (j >> slice_shift) : 0u) +
                          (j & (slices - 1u)) * WARP_AREA;
#pragma unroll
        for (uint32_t q = 0; q < UB; ++q)
          v[q][jj] = (valid[q] && j < R) ? pj[head_area[q] + row_g[q] * D + chunk[q] * 32 + lane] : 0.f;
      }
#pragma unroll
      for (uint32_t jj = 0; jj < JB; ++jj) {
#pragma unroll
        for (uint32_t q = 0; q < UB; ++q) {
          const float fj = __shfl_sync(0xffffffffu, f[q], (j0 + jj) & 31u);
          if (j0 + jj < R) o_all[q] += fj * v[q][jj];
        }
      }
    }
#pragma unroll
    for (uint32_t q = 0; q < UB; ++q) {
      if (valid[q] && ok) {
        // acc * (1 / l) as the reference does (paged_attention_utils.hpp:834-835);
        // an empty context (l = 0) gives zeros
        const float inv = (l_all[q] > 0.f) ? (1.f / l_all[q]) : 0.f;
        const size_t head = static_cast<size_t>(seq) * num_heads + kv_head[q] * G + row_g[q];
        const float head_scale = (v_scale_per_head != nullptr) ? __ldg(v_scale_per_head + kv_head[q]) : out_scale;
        out[head * D + chunk[q] * 32 + lane] = __float2half_rn(o_all[q] * head_scale * inv);
      }
    }
  }
}

// Internal linkage: the kernel reads and writes the per-unit tables above (scheduler counters,
// status word, time stamps, range-check report), and two launchers may build the same
// instantiation (the loop launchers also run the persistent form).  With external linkage the
// host stubs of such twins would be merged and a launch could run the other unit's copy, with
// the other unit's tables behind this unit's slot allocator.
namespace {
template <int D, int KV, int MODE, int NWARPS = 4, int TILES = 1>
__global__ void __launch_bounds__(paged_attention_policy_v2<D, KV, NWARPS, TILES>::threads_per_cta,
                                  paged_attention_policy_v2<D, KV, NWARPS, TILES>::ctas_per_sm)
paged_attention_kernel(const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const AttnArgs args) {
  using L = SmemLayout<D, KV, NWARPS, TILES>;
  using policy = typename L::policy;
  using geo = typename L::geo;
  constexpr uint32_t NW = L::NW;
  constexpr uint32_t NSTAGES = L::NSTAGES;
  constexpr uint32_t KSTEPS = D / 16; // MMA k-steps of QK^T == accumulator tiles of PV
  constexpr uint32_t NCONS = NW * 32; // consumer threads

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment of the ring makes the TMA swizzle a function of (row, chunk).
  // The offset is identical in every CTA, so cluster-mapped addresses line up.
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t *smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  float *merge_buf = reinterpret_cast<float *>(smem + L::MERGE_OFFSET);
  float *warp_stats = reinterpret_cast<float *>(smem + L::WARP_STATS_OFFSET);
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L::BAR_OFFSET);
  uint64_t *empty_bar = full_bar + NSTAGES;
  volatile uint32_t *abort_flag =
      reinterpret_cast<volatile uint32_t *>(smem + L::BAR_OFFSET + 2 * NSTAGES * 8);
  uint64_t *sched_full = reinterpret_cast<uint64_t *>(smem + L::SCHED_OFFSET); // [2]
  uint64_t *sched_empty = sched_full + 2;                                       // [2]
  volatile uint32_t *sched_item = reinterpret_cast<volatile uint32_t *>(sched_full + 4); // [2]
  constexpr uint32_t kNoItem = 0xffffffffu;
  float2 *stage_scales = reinterpret_cast<float2 *>(smem + L::SCALES_OFFSET); // [NSTAGES][SCALE_SLOTS]
  const bool block_scales = (KV != KV_F16) && args.k_scale_per_block != nullptr;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t hpc = args.hpc;
  const uint32_t tps = args.tokens_per_stage; // tokens of a KV head in one stage
  const uint32_t tpt = tps / TILES;           // ... that the warps consume in one tile step
#ifdef PA_TIMELINE
  const uint32_t timeline_cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  if (threadIdx.x == 32) {
    PA_STAMP(0);
    PA_STAMP_VALUE(2, 0ull);
    PA_STAMP_VALUE(3, 0ull);
    PA_STAMP_VALUE(4, 0ull);
    PA_STAMP_VALUE(6, 0ull);
    PA_STAMP_VALUE(7, 0ull);
  }
#endif

  // ---- barriers first: none of this touches global memory, so in split mode it runs before
  // the wait for the previous kernel of the stream
  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < NSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);   // one arrive.expect_tx by the producer
      mbar_init(&empty_bar[s], NW); // one arrive per consumer warp
    }
    for (uint32_t s = 0; s < 2; ++s) {
      mbar_init(&sched_full[s], 1);
      mbar_init(&sched_empty[s], NW);
    }
    *abort_flag = 0u;
    mbar_fence_init();
    // the descriptors are kernel parameters, not data of an earlier kernel: fetch them now
    tma_prefetch_descriptor(&tmap_k);
    tma_prefetch_descriptor(&tmap_v);
  }
  __syncthreads();

  // ---- the first work item of this CTA (integer bookkeeping, bit-exact); every warp keeps
  // its own cursor over the item numbering and walks it in step with its own loop
  uint32_t cta_rank = 0, num_ranks = 1;
  WorkItem first{};
  SplitCursor cursor{};
  const uint32_t head_groups = args.num_kv_heads / hpc;
  if constexpr (MODE == MODE_SPLIT) {
    // let the merge kernel's CTAs be scheduled as this grid's CTAs retire (it waits for the
    // completion of this grid before it reads anything)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // this grid may itself have been scheduled while the previous kernel of the stream was
    // draining: nothing in global memory is touched before that kernel has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 32) PA_STAMP(1);
    cursor.init(args, head_groups, lane);
    first = cursor.seek(blockIdx.x, args, head_groups, lane);
  } else {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    cta_rank = cluster.block_rank();
    num_ranks = cluster.num_blocks();
    // programmatic dependent launch, as in split mode: the next kernel of the stream may be
    // scheduled while this one runs, and this one touches no global memory before the
    // previous kernel of the stream has completed (back-to-back calls on tiny batches are
    // bound by launch latency otherwise)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 32) PA_STAMP(1);
    // Clusters start in block-index order.  With ragged lengths a long sequence that starts
    // last leaves the machine idle behind it, so block index z is mapped to the z-th sequence
    // in (approximately) descending length: 16 length classes, longest class first, position
    // order inside a class.  Every CTA computes the same map from the context lengths alone.
    uint32_t position = blockIdx.z;
    if (args.longest_first_hint != 0u && args.num_seqs > 1u) {
      __shared__ uint32_t class_count[16];
      __shared__ uint32_t chosen;
      if (threadIdx.x < 16) class_count[threadIdx.x] = 0u;
      __syncthreads();
      auto length_class = [&](uint32_t pos) -> uint32_t {
        const uint32_t id = (args.seq_indices != nullptr) ? __ldg(args.seq_indices + pos) : pos;
        const uint64_t c = __ldg(args.context_lens + id);
        const uint64_t k = c * 16ull / (static_cast<uint64_t>(args.longest_first_hint) + 1ull);
        return 15u - static_cast<uint32_t>(k > 15ull ? 15ull : k); // class 0 = longest
      };
      for (uint32_t pos = threadIdx.x; pos < args.num_seqs; pos += blockDim.x)
        atomicAdd(&class_count[length_class(pos)], 1u);
      __syncthreads();
      if (warp == 0) {
        uint32_t want = blockIdx.z, cls = 0;
        while (cls < 15u && want >= class_count[cls]) want -= class_count[cls++];
        // the want-th sequence (in position order) of class cls
        uint32_t found = blockIdx.z;
        for (uint32_t base = 0; base < args.num_seqs; base += 32) {
          const uint32_t pos = base + lane;
          const bool hit = pos < args.num_seqs && length_class(pos) == cls;
          const uint32_t mask = __ballot_sync(0xffffffffu, hit);
          const uint32_t n = __popc(mask);
          if (want < n) {
            found = base + __fns(mask, 0, want + 1);
            break;
          }
          want -= n;
        }
        if (lane == 0) chosen = found;
      }
      __syncthreads();
      position = chosen;
    }
    first.seq = (args.seq_indices != nullptr) ? __ldg(args.seq_indices + position) : position;
    first.head_base = blockIdx.y * hpc;
    first.partition = 0;
    const uint32_t ctx = load_context(args, first.seq, first.table_off);
    // the context is cut into whole stages, spread evenly over the CTAs of the cluster
    const uint32_t total_stages = divide_round_up(ctx, tps);
    const uint32_t stages_per_rank = divide_round_up(total_stages, num_ranks);
    first.tok_begin = min(ctx, cta_rank * stages_per_rank * tps);
    first.tok_end = min(ctx, (cta_rank + 1) * stages_per_rank * tps);
    first.ctx = ctx;
    first.valid = true;
  }

  if (warp == 0) {
    // =========================== producer warp ===========================
    const uint64_t kv_policy = l2_evict_first_policy(); // every KV byte is read once
    const uint32_t rows = args.rows_per_box;
    const uint32_t bps = args.boxes_per_stage;
    const uint32_t chunks_per_stage = bps / hpc;      // token chunks (boxes per head) in a stage
    const uint32_t box_bytes = rows * geo::row_bytes; // K (or V) bytes of one box
    const uint32_t ring_base = smem_u32(smem);
    const uint32_t row_mask = (1u << args.block_shift) - 1u;
    // lane -> (token chunk of the batch, head inside the CTA's head group), head fastest
    const uint32_t lane_chunk = lane / hpc;
    const uint32_t lane_head = lane % hpc;
    const uint32_t chunks_per_batch = 32 / hpc;
    uint32_t slot = 0, phase = 0; // ring position, continuous across work items
    bool alive = true;
    // lane 0: stages whose full barrier it has armed, and the phase parity of the last arming
    uint32_t armed_stages = 0, armed_parity = 0;

    auto fetch_block_id = [&](const WorkItem &it, uint32_t chunk) -> uint32_t {
      const uint32_t tok = it.tok_begin + chunk * rows;
      if (!it.valid || tok >= it.tok_end) return 0u;
      const size_t row = (args.table_offsets != nullptr) ? static_cast<size_t>(it.table_off)
                                                         : static_cast<size_t>(it.seq) * args.max_blocks_per_seq;
#ifdef PA_DEBUG_BOUNDS
      const uint32_t width = (args.table_offsets != nullptr)
                                 ? __ldg(args.table_offsets + it.seq + 1) - it.table_off
                                 : args.max_blocks_per_seq;
      if (!bounds_ok(BOUNDS_TABLE_INDEX, tok >> args.block_shift, width, it.seq, tok)) return 0u;
      const uint32_t id = __ldg(args.block_tables + row + (tok >> args.block_shift));
      return bounds_ok(BOUNDS_BLOCK_ID, id, args.num_blocks, it.seq, tok) ? id : 0u;
#else
      return __ldg(args.block_tables + row + (tok >> args.block_shift));
#endif
    };

    WorkItem cur = first;
    uint32_t block_id_next = fetch_block_id(cur, lane_chunk);
    uint32_t item_no = 0;
    while (cur.valid && alive) {
      WorkItem nxt{};
      nxt.valid = false;
      // Dynamic scheduling (split mode): the CTA's first item is its block index, every further
      // one is drawn from a global counter, so CTAs that run faster take more items.  The
      // draw is issued here and its answer is only looked at after this item's first copies
      // have been issued, so the round trip of the atomic never delays a copy.  The number is
      // published to the consumer warps through a two-entry queue in shared memory.
      unsigned int ticket = 0;
      bool next_known = (MODE != MODE_SPLIT);
      if constexpr (MODE == MODE_SPLIT) {
        if (lane == 0) ticket = atomicAdd(&g_sched[args.sched_slot][0], 1u);
      }
      auto resolve_next = [&]() {
        const uint32_t next_index = gridDim.x + __shfl_sync(0xffffffffu, ticket, 0);
        nxt = cursor.seek(next_index, args, head_groups, lane);
        const uint32_t entry = item_no + 1, qs = entry & 1u, use = (entry - 1u) >> 1; // n-th use of the slot
        if (lane == 0) {
          alive = mbar_wait_bounded(&sched_empty[qs], (use & 1u) ^ 1u, abort_flag);
          if (alive) {
            sched_item[qs] = nxt.valid ? next_index : kNoItem;
            mbar_arrive(&sched_full[qs]);
          }
        }
        alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
        next_known = true;
      };
      const uint32_t total_chunks = divide_round_up(cur.tok_end - cur.tok_begin, rows);
      const int32_t head_coord = static_cast<int32_t>(cur.head_base + lane_head);
      // The number is needed when the item's last batch of copies has been issued: the next
      // item's context length and first table entries are then fetched while those copies fly
      // (a short item would otherwise wait for them before its only copies).  The consumers ask
      // for the number when they have consumed this item's last stage.
      for (uint32_t chunk0 = 0; chunk0 < total_chunks && alive; chunk0 += chunks_per_batch) {
        const bool last_batch = chunk0 + chunks_per_batch >= total_chunks;
        const uint32_t chunk = chunk0 + lane_chunk;
        const uint32_t block_id = block_id_next;
        // prefetch the table entries of this item's next batch
        if (!last_batch) block_id_next = fetch_block_id(cur, chunk + chunks_per_batch);
        const bool valid = chunk < total_chunks;
        const uint32_t tok = cur.tok_begin + chunk * rows;
        const int32_t y = static_cast<int32_t>((block_id << args.block_shift) + (tok & row_mask));
        const uint32_t chunks_in_batch = min(chunks_per_batch, total_chunks - chunk0);
        const uint32_t stages_in_batch = divide_round_up(chunks_in_batch, chunks_per_stage);
        // per-block scales of this lane's (block, head): requested now, written beside the stage
        // before it is armed; in steady state the wait for a free stage hides the latency
        float2 lane_scales = make_float2(1.f, 1.f);
        if (block_scales && valid) {
          // a block id beyond the cache reads zeros through the descriptor; its scales come from the last block
          const size_t si = static_cast<size_t>(min(block_id, args.num_blocks - 1u)) * args.num_kv_heads +
                            cur.head_base + lane_head;
          lane_scales = make_float2(__ldg(args.k_scale_per_block + si), __ldg(args.v_scale_per_block + si));
        }
        for (uint32_t sb = 0; sb < stages_in_batch; ++sb) {
          if (lane == 0) alive = mbar_wait_bounded(&empty_bar[slot], phase ^ 1u, abort_flag);
          alive = __shfl_sync(0xffffffffu, alive ? 1 : 0, 0) != 0;
          if (!alive) break;
          if (block_scales) {
            // the stage is free: its scale slots may be overwritten; the arming below releases them
            if (valid && lane_chunk / chunks_per_stage == sb)
              stage_scales[slot * L::SCALE_SLOTS + (lane_chunk % chunks_per_stage) * hpc + lane_head] = lane_scales;
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t chunks_here = min(chunks_per_stage, chunks_in_batch - sb * chunks_per_stage);
            mbar_arrive_expect_tx(&full_bar[slot], chunks_here * hpc * box_bytes * 2u);
            armed_stages |= 1u << slot;
            armed_parity = (armed_parity & ~(1u << slot)) | (phase << slot);
          }
          if (valid && lane_chunk / chunks_per_stage == sb && lane_head % args.heads_per_box == 0) {
            // rows of a stage: head-major, tokens_per_stage rows per head; a box that spans
            // several heads lands as [head][row][slab], which is this very layout
            const uint32_t row0 = lane_head * tps + (lane_chunk % chunks_per_stage) * rows;
            const uint32_t stage_base = ring_base + slot * L::STAGE_BYTES;
#ifdef PA_TIMELINE
            if (lane == 0 && item_no == 0 && chunk0 == 0 && sb == 0) PA_STAMP(2);
#endif
#pragma unroll
            for (uint32_t sl = 0; sl < geo::num_slabs; ++sl) {
              const uint32_t dst = stage_base + sl * L::SLAB_TILE + row0 * geo::slab_bytes;
              const int32_t x = static_cast<int32_t>(sl * geo::slab_elems);
              tma_load_3d(dst, &tmap_k, &full_bar[slot], x, y, head_coord, kv_policy);
              tma_load_3d(dst + L::KV_TILE, &tmap_v, &full_bar[slot], x, y, head_coord, kv_policy);
            }
          }
          if (++slot == NSTAGES) {
            slot = 0;
            phase ^= 1u;
          }
        }
      }
      // (also reached by an item without tokens: an empty context as a whole-context item)
      if (!next_known && alive) resolve_next();
      block_id_next = fetch_block_id(nxt, lane_chunk);
      cur = nxt;
      ++item_no;
    }
    if (*abort_flag != 0u && lane == 0) {
      // A wait gave up.  Copies already issued into the ring still complete some time and
      // would land in shared memory that belongs to the next CTA of this SM if this one left
      // now: wait (again with a limit) until every armed stage has received its bytes.
      for (uint32_t s = 0; s < NSTAGES; ++s)
        if ((armed_stages >> s) & 1u) mbar_wait_limited(&full_bar[s], (armed_parity >> s) & 1u, 20000000ull);
    }
  } else {
    // =========================== consumer warps ==========================
    const uint32_t cw = warp - 1; // 0..NW-1
    const uint32_t gid = lane >> 2;
    const uint32_t t4 = lane & 3u;
    const uint32_t G = args.group;
    const uint32_t ctid = threadIdx.x - 32; // 0 .. NCONS-1
    // warp -> (head inside the group, 16-token slice inside a tile step)
    const uint32_t slices = NW / hpc; // token slices per head: 4, 2 or 1
    const uint32_t my_head = cw / slices;
    const uint32_t my_slice = cw % slices;
    // first row of this warp's tile in tile step 0 of a stage; step k lies k * tpt rows further
    const uint32_t warp_row = my_head * tps + my_slice * 16;

    // lane-dependent, stage-independent parts of the ldmatrix addresses; the chunk pair
    // 2k, 2k+1 of a slab is reached by XOR-ing (k << 5) into the address
    const uint32_t ring_base = smem_u32(smem);
    const uint32_t lm_row_a = warp_row + (lane & 7u) + ((lane >> 3) & 1u) * 8u;
    const uint32_t lm_off_a = swizzled_offset<geo::slab_bytes>(lm_row_a, lane >> 4); // K, FP8 V
    const uint32_t lm_row_b = warp_row + (lane & 7u) + (lane >> 4) * 8u;
    const uint32_t lm_off_b = swizzled_offset<geo::slab_bytes>(lm_row_b, (lane >> 3) & 1u); // fp16 V
    constexpr uint32_t PAIRS_PER_SLAB = geo::chunks_per_slab / 2;

    // S^T tile of 16 tokens: K (A operand) from shared memory at k_addr, Q from registers;
    // two accumulation chains shorten the dependency
    auto score_tile = [&](uint32_t k_addr, const uint32_t (&q)[KSTEPS][2], float (&c)[4]) {
      float s_a[4] = {0.f, 0.f, 0.f, 0.f};
      float s_b[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (KV == KV_F16) {
#pragma unroll
        for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
          uint32_t a[4];
          ldmatrix_x4(a, (k_addr ^ ((ks % PAIRS_PER_SLAB) << 5)) + (ks / PAIRS_PER_SLAB) * L::SLAB_TILE);
          if (ks & 1u) mma_m16n8k16(s_b, a, q[ks][0], q[ks][1]);
          else mma_m16n8k16(s_a, a, q[ks][0], q[ks][1]);
        }
      } else {
#pragma unroll
        for (uint32_t qq = 0; qq < KSTEPS / 2; ++qq) {
          // r[0]/r[1]: rows gid / gid+8 of chunk 2qq, r[2]/r[3]: the same of chunk 2qq+1
          uint32_t r[4];
          ldmatrix_x4(r, k_addr ^ (qq << 5));
          uint32_t a[4];
          fp8x4_to_half2x2<KV>(r[0], a[0], a[2]);
          fp8x4_to_half2x2<KV>(r[1], a[1], a[3]);
          mma_m16n8k16(s_a, a, q[2 * qq][0], q[2 * qq][1]);
          fp8x4_to_half2x2<KV>(r[2], a[0], a[2]);
          fp8x4_to_half2x2<KV>(r[3], a[1], a[3]);
          mma_m16n8k16(s_b, a, q[2 * qq + 1][0], q[2 * qq + 1][1]);
        }
      }
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) c[j] = s_a[j] + s_b[j];
    };
    // The same for the tiles of two stages at once, as one straight-line instruction stream:
    // the two tiles' loads, conversions and MMA chains are independent, so they can be
    // scheduled into each other's latencies.  Per tile the operations and their order are
    // those of score_tile, hence the same bits.
    auto score_tile_pair = [&](uint32_t ka_addr, uint32_t kb_addr, const uint32_t (&q)[KSTEPS][2],
                               float (&ca)[4], float (&cb)[4]) {
      float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
      float b0[4] = {0.f, 0.f, 0.f, 0.f}, b1[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (KV == KV_F16) {
#pragma unroll
        for (uint32_t ks = 0; ks < KSTEPS; ++ks) {
          const uint32_t off = (ks / PAIRS_PER_SLAB) * L::SLAB_TILE;
          uint32_t fa[4], fb[4];
          ldmatrix_x4(fa, (ka_addr ^ ((ks % PAIRS_PER_SLAB) << 5)) + off);
          ldmatrix_x4(fb, (kb_addr ^ ((ks % PAIRS_PER_SLAB) << 5)) + off);
          if (ks & 1u) {
            mma_m16n8k16(a1, fa, q[ks][0], q[ks][1]);
            mma_m16n8k16(b1, fb, q[ks][0], q[ks][1]);
          } else {
            mma_m16n8k16(a0, fa, q[ks][0], q[ks][1]);
            mma_m16n8k16(b0, fb, q[ks][0], q[ks][1]);
          }
        }
      } else {
#pragma unroll
        for (uint32_t qq = 0; qq < KSTEPS / 2; ++qq) {
          uint32_t ra[4], rb[4], fa[4], fb[4];
          ldmatrix_x4(ra, ka_addr ^ (qq << 5));
          ldmatrix_x4(rb, kb_addr ^ (qq << 5));
          fp8x4_to_half2x2<KV>(ra[0], fa[0], fa[2]);
          fp8x4_to_half2x2<KV>(ra[1], fa[1], fa[3]);
          mma_m16n8k16(a0, fa, q[2 * qq][0], q[2 * qq][1]);
          fp8x4_to_half2x2<KV>(rb[0], fb[0], fb[2]);
          fp8x4_to_half2x2<KV>(rb[1], fb[1], fb[3]);
          mma_m16n8k16(b0, fb, q[2 * qq][0], q[2 * qq][1]);
          fp8x4_to_half2x2<KV>(ra[2], fa[0], fa[2]);
          fp8x4_to_half2x2<KV>(ra[3], fa[1], fa[3]);
          mma_m16n8k16(a1, fa, q[2 * qq + 1][0], q[2 * qq + 1][1]);
          fp8x4_to_half2x2<KV>(rb[2], fb[0], fb[2]);
          fp8x4_to_half2x2<KV>(rb[3], fb[1], fb[3]);
          mma_m16n8k16(b1, fb, q[2 * qq + 1][0], q[2 * qq + 1][1]);
        }
      }
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        ca[j] = a0[j] + a1[j];
        cb[j] = b0[j] + b1[j];
      }
    };
    // O^T += V^T . P^T for 16 tokens: V (A operand, transposed load) from shared memory
    auto value_tile = [&](uint32_t v_base, uint32_t p_lo, uint32_t p_hi, float (&o)[KSTEPS][4]) {
      if constexpr (KV == KV_F16) {
        const uint32_t v_addr = v_base + lm_off_b;
#pragma unroll
        for (uint32_t i = 0; i < KSTEPS; ++i) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, (v_addr ^ ((i % PAIRS_PER_SLAB) << 5)) + (i / PAIRS_PER_SLAB) * L::SLAB_TILE);
          mma_m16n8k16(o[i], a, p_lo, p_hi);
        }
      } else {
        const uint32_t v_addr = v_base + lm_off_a;
#pragma unroll
        for (uint32_t qq = 0; qq < KSTEPS / 2; ++qq) {
          // 16 tokens x 32 dims of bytes, read as transposed 16-bit units:
          // r[0]: tokens 0-7 / dims 0-15, r[1]: tokens 8-15 / dims 0-15,
          // r[2]: tokens 0-7 / dims 16-31, r[3]: tokens 8-15 / dims 16-31.
          // Each register = {V[2t][2g], V[2t][2g+1], V[2t+1][2g], V[2t+1][2g+1]}.
          uint32_t r[4];
          ldmatrix_x4_trans(r, v_addr ^ (qq << 5));
          uint32_t ae[4], ao[4];
          fp8x4_to_even_odd_half2<KV>(r[0], ae[0], ao[0]);
          fp8x4_to_even_odd_half2<KV>(r[2], ae[1], ao[1]);
          fp8x4_to_even_odd_half2<KV>(r[1], ae[2], ao[2]);
          fp8x4_to_even_odd_half2<KV>(r[3], ae[3], ao[3]);
          mma_m16n8k16(o[2 * qq], ae, p_lo, p_hi);
          mma_m16n8k16(o[2 * qq + 1], ao, p_lo, p_hi);
        }
      }
    };
    // Last tile of a context: clear the V rows past it (unused tail of the last block, or rows
    // no copy of this stage wrote), so that 0 * garbage stays 0.
    auto zero_value_rows = [&](uint32_t v_base, uint32_t first_row, uint32_t num_rows, uint32_t ln) {
      constexpr uint32_t CPR = geo::slab_bytes / 16; // 16-byte chunks per row
      for (uint32_t sl = 0; sl < geo::num_slabs; ++sl) {
        for (uint32_t c = ln; c < num_rows * CPR; c += 32) {
          const uint32_t addr = v_base + sl * L::SLAB_TILE + (first_row + c / CPR) * geo::slab_bytes + (c % CPR) * 16;
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
        }
      }
      // order these generic-proxy writes before the TMA (async proxy) refill of the slot
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    };

    uint32_t slot = 0, phase = 0, item_parity = 0;
    bool alive = true;
#ifdef PA_TIMELINE
    bool timeline_first = true;
    unsigned long long timeline_items = 0;
#endif
    uint32_t qf[KSTEPS][2];
    WorkItem cur = first;
    if (cur.valid) load_q_fragments<D, KV>(qf, args, cur.seq, cur.head_base + my_head, gid, t4);

    // state of query columns g = 2*t4 and 2*t4+1, log2 domain: m_ref is the exponent
    // reference the weights are taken against, m_true the running maximum
    float m_ref[2], m_true[2], l_run[2];
    float acc[KSTEPS][4];

    uint32_t item_no = 0;
    while (cur.valid) {
      WorkItem nxt{};
      nxt.valid = false;
      const uint32_t kv_head = cur.head_base + my_head;
      // softmax scale (log2 domain) and output scale of this warp's KV head
      const float scale = (args.k_scale_per_head != nullptr)
                              ? args.sm_scale_log2 * __ldg(args.k_scale_per_head + kv_head)
                              : args.scale_log2;
      const float out_scale = (args.v_scale_per_head != nullptr) ? __ldg(args.v_scale_per_head + kv_head)
                                                                 : args.out_scale;
      // score modifiers and per-block scales take the general path below; the straight-line
      // path for pairs of full tiles is for the plain case only
      const bool modifiers = (args.alibi_slopes != nullptr) || (args.softcap > 0.f) || block_scales;
      float slope[2] = {0.f, 0.f}; // ALiBi slopes of query columns 2*t4, 2*t4+1
      if (args.alibi_slopes != nullptr) {
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
          if (2 * t4 + j < G) slope[j] = __ldg(args.alibi_slopes + kv_head * G + 2 * t4 + j);
      }

      m_ref[0] = m_ref[1] = m_true[0] = m_true[1] = neg_infinity();
      l_run[0] = l_run[1] = 0.f; // per-lane partial sums; reduced over gid at the end
#pragma unroll
      for (uint32_t i = 0; i < KSTEPS; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
      // The sink is one extra logit with a zero value vector, attached to the first tokens
      // of the context only (reference paged_attention_kernel_loop.hpp:387-401).
      if (args.sinks != nullptr && my_slice == 0 && cur.tok_begin == 0) {
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j) {
          const uint32_t g = 2 * t4 + j;
          if (g < G) {
            m_ref[j] = m_true[j] = __half2float(args.sinks[kv_head * G + g]) * kLog2e;
            l_run[j] = (gid == 0) ? 1.f : 0.f;
          }
        }
      }

      const uint32_t my_tokens = cur.tok_end - cur.tok_begin;
      const uint32_t my_steps = divide_round_up(my_tokens, tpt); // tile steps of the item
      // Two tile steps per iteration: their score tiles are independent instruction streams
      // (more work in flight per warp) and share one softmax step.  With one tile per stage the
      // two steps are two stages; with 2 or 4 they lie in the same stage, TILES / 2 pairs of it.
      for (uint32_t st = 0; st < my_steps; st += 2) {
        const bool has_b = st + 1 < my_steps;
        uint32_t slot_a, phase_a, slot_b, phase_b, sub_a = 0, sub_b = 0;
        bool first_touch = true, last_touch = true; // of the stage that holds both steps (TILES > 1)
        if constexpr (TILES == 1) {
          slot_a = slot, phase_a = phase;
          if (++slot == NSTAGES) {
            slot = 0;
            phase ^= 1u;
          }
          slot_b = slot, phase_b = phase;
          if (has_b && ++slot == NSTAGES) {
            slot = 0;
            phase ^= 1u;
          }
        } else {
          sub_a = st % TILES;
          sub_b = sub_a + 1;
          slot_a = slot_b = slot;
          phase_a = phase_b = phase;
          first_touch = sub_a == 0;
          last_touch = sub_b + 1 == TILES || st + 2 >= my_steps;
          if (last_touch && ++slot == NSTAGES) {
            slot = 0;
            phase ^= 1u;
          }
        }
        // after an abort the loops keep their shape (the named barriers below need every
        // consumer warp) but no longer wait or compute
        if (alive && first_touch) alive = mbar_wait_bounded(&full_bar[slot_a], phase_a, abort_flag);
#ifdef PA_TIMELINE
        if (ctid == 0 && timeline_first) {
          PA_STAMP(3);
          timeline_first = false;
        }
#endif
        if (TILES == 1 && alive && has_b) alive = mbar_wait_bounded(&full_bar[slot_b], phase_b, abort_flag);
        const uint32_t tok_a = st * tpt + my_slice * 16; // first token of this warp's tile A
        const uint32_t tok_b = tok_a + tpt;
        // stage bases, moved to the tile step inside the stage
        const uint32_t base_a = ring_base + slot_a * L::STAGE_BYTES + sub_a * tpt * geo::slab_bytes;
        const uint32_t base_b = ring_base + slot_b * L::STAGE_BYTES + sub_b * tpt * geo::slab_bytes;
        bool released_a = false;
        if (alive && has_b && !modifiers && tok_b + 16u <= my_tokens) {
          // ---- the common case, two full tiles and no score modifiers, free of branches up
          // to the rescale test; every value is computed as in the general case below
          float ca[4], cb[4];
          score_tile_pair(base_a + lm_off_a, base_b + lm_off_a, qf, ca, cb);
          m_true[0] = fmaxf(m_true[0], quad_column_max(fmaxf(fmaxf(ca[0], ca[2]), fmaxf(cb[0], cb[2]))) * scale);
          m_true[1] = fmaxf(m_true[1], quad_column_max(fmaxf(fmaxf(ca[1], ca[3]), fmaxf(cb[1], cb[3]))) * scale);
          const bool stale = (m_true[0] > m_ref[0] + kRescaleThreshold) ||
                             (m_true[1] > m_ref[1] + kRescaleThreshold);
          if (__any_sync(0xffffffffu, stale)) {
            const float r0 = (m_ref[0] == neg_infinity()) ? 0.f : fast_exp2(m_ref[0] - m_true[0]);
            const float r1 = (m_ref[1] == neg_infinity()) ? 0.f : fast_exp2(m_ref[1] - m_true[1]);
            l_run[0] *= r0;
            l_run[1] *= r1;
#pragma unroll
            for (uint32_t i = 0; i < KSTEPS; ++i) {
              acc[i][0] *= r0;
              acc[i][1] *= r1;
              acc[i][2] *= r0;
              acc[i][3] *= r1;
            }
            m_ref[0] = m_true[0];
            m_ref[1] = m_true[1];
          }
          float pa[4], pb[4];
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            pa[j] = fast_exp2(fmaf(ca[j], scale, -m_ref[j & 1u]));
            pb[j] = fast_exp2(fmaf(cb[j], scale, -m_ref[j & 1u]));
          }
          l_run[0] += (pa[0] + pa[2]) + (pb[0] + pb[2]);
          l_run[1] += (pa[1] + pa[3]) + (pb[1] + pb[3]);
          const uint32_t pa_lo = movmatrix_trans(pack_half2(pa[0], pa[1]));
          const uint32_t pa_hi = movmatrix_trans(pack_half2(pa[2], pa[3]));
          const uint32_t pb_lo = movmatrix_trans(pack_half2(pb[0], pb[1]));
          const uint32_t pb_hi = movmatrix_trans(pack_half2(pb[2], pb[3]));
          value_tile(base_a + L::KV_TILE, pa_lo, pa_hi, acc);
          if constexpr (TILES == 1) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot_a]); // stage A goes back before stage B is used
            released_a = true;
          }
          value_tile(base_b + L::KV_TILE, pb_lo, pb_hi, acc);
        } else if (alive && tok_a < my_tokens) {
          const bool act_b = has_b && tok_b < my_tokens;
          const uint32_t n_a = min(16u, my_tokens - tok_a);
          const uint32_t n_b = act_b ? min(16u, my_tokens - tok_b) : 0u;
          if (n_a < 16u) zero_value_rows(base_a + L::KV_TILE, warp_row + n_a, 16u - n_a, lane);
          if (act_b && n_b < 16u) zero_value_rows(base_b + L::KV_TILE, warp_row + n_b, 16u - n_b, lane);

          // ---- S^T = K . Q^T ; lane holds S[tok gid][g 2t4, 2t4+1] in [0],[1] and
          // S[tok gid+8][..] in [2],[3]
          float ca[4], cb[4];
          score_tile(base_a + lm_off_a, qf, ca);
          if (act_b) {
            score_tile(base_b + lm_off_a, qf, cb);
          } else {
            cb[0] = cb[1] = cb[2] = cb[3] = neg_infinity();
          }
          float eff_scale = scale;
          float v_scale_a = 1.f, v_scale_b = 1.f; // per-block V scales of the two tiles
          float k_nat_a = scale * kLn2, k_nat_b = scale * kLn2; // sm_scale * k scale of the two tiles
          if (block_scales) {
            // tile A / B lie in one KV block each: the stage's slot for (that block, this head)
            const uint32_t chunk_a = (sub_a * tpt + my_slice * 16u) / args.rows_per_box;
            const uint32_t chunk_b = (sub_b * tpt + my_slice * 16u) / args.rows_per_box;
            const float2 sa = stage_scales[slot_a * L::SCALE_SLOTS + chunk_a * hpc + my_head];
            const float2 sb2 = act_b ? stage_scales[slot_b * L::SCALE_SLOTS + chunk_b * hpc + my_head] : make_float2(1.f, 1.f);
            k_nat_a = args.sm_scale_log2 * kLn2 * sa.x;
            k_nat_b = args.sm_scale_log2 * kLn2 * sb2.x;
            v_scale_a = sa.y;
            v_scale_b = sb2.y;
          }
          if (modifiers) {
            // soft-cap / ALiBi / per-block scales: turn the raw dot products into log2-domain
            // logits here; the softmax below then runs with a unit scale
            const int32_t last = static_cast<int32_t>(cur.ctx) - 1;
            const int32_t t_a = static_cast<int32_t>(cur.tok_begin + tok_a + gid);
            const int32_t t_b = t_a + static_cast<int32_t>(tpt);
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              const int32_t row = (j >> 1) * 8; // [2],[3] belong to token gid + 8
              float xa = ca[j] * k_nat_a, xb = cb[j] * k_nat_b;
              if (args.softcap > 0.f) {
                xa = args.softcap * tanhf(xa / args.softcap);
                xb = args.softcap * tanhf(xb / args.softcap);
              }
              xa += slope[j & 1u] * static_cast<float>(t_a + row - last);
              xb += slope[j & 1u] * static_cast<float>(t_b + row - last);
              ca[j] = xa * kLog2e;
              cb[j] = act_b ? xb * kLog2e : neg_infinity();
            }
            eff_scale = 1.f;
          }
          if (modifiers || n_a < 16u || (act_b && n_b < 16u)) {
            // tokens past the context never count, whatever the cache holds there
            // (reference paged_attention_kernel_loop.hpp:323-327)
            if (gid >= n_a) ca[0] = ca[1] = neg_infinity();
            if (gid + 8 >= n_a) ca[2] = ca[3] = neg_infinity();
            if (gid >= n_b) cb[0] = cb[1] = neg_infinity();
            if (gid + 8 >= n_b) cb[2] = cb[3] = neg_infinity();
          }
          // ---- online softmax (reference paged_attention_kernel_loop.hpp:382-419);
          // scale > 0, so the maximum commutes with the scaling
          m_true[0] = fmaxf(m_true[0], quad_column_max(fmaxf(fmaxf(ca[0], ca[2]), fmaxf(cb[0], cb[2]))) * eff_scale);
          m_true[1] = fmaxf(m_true[1], quad_column_max(fmaxf(fmaxf(ca[1], ca[3]), fmaxf(cb[1], cb[3]))) * eff_scale);
          const bool stale = (m_true[0] > m_ref[0] + kRescaleThreshold) ||
                             (m_true[1] > m_ref[1] + kRescaleThreshold);
          if (__any_sync(0xffffffffu, stale)) {
            const float r0 = (m_ref[0] == neg_infinity()) ? 0.f : fast_exp2(m_ref[0] - m_true[0]);
            const float r1 = (m_ref[1] == neg_infinity()) ? 0.f : fast_exp2(m_ref[1] - m_true[1]);
            l_run[0] *= r0;
            l_run[1] *= r1;
#pragma unroll
            for (uint32_t i = 0; i < KSTEPS; ++i) {
              acc[i][0] *= r0;
              acc[i][1] *= r1;
              acc[i][2] *= r0;
              acc[i][3] *= r1;
            }
            m_ref[0] = m_true[0];
            m_ref[1] = m_true[1];
          }
          float pa[4], pb[4];
#pragma unroll
          for (uint32_t j = 0; j < 4; ++j) {
            pa[j] = fast_exp2(fmaf(ca[j], eff_scale, -m_ref[j & 1u]));
            pb[j] = fast_exp2(fmaf(cb[j], eff_scale, -m_ref[j & 1u]));
          }
          l_run[0] += (pa[0] + pa[2]) + (pb[0] + pb[2]); // fp32 sum of the unrounded weights
          l_run[1] += (pa[1] + pa[3]) + (pb[1] + pb[3]);
          if (block_scales) {
            // V of a block dequantises as code * scale: fold the scale into the weights
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
              pa[j] *= v_scale_a;
              pb[j] *= v_scale_b;
            }
          }
          // P rounded to fp16 for the MMA, transposed into the B-operand layout;
          // ---- O^T += V^T . P^T
          {
            const uint32_t p_lo = movmatrix_trans(pack_half2(pa[0], pa[1])); // tokens 0..7
            const uint32_t p_hi = movmatrix_trans(pack_half2(pa[2], pa[3])); // tokens 8..15
            value_tile(base_a + L::KV_TILE, p_lo, p_hi, acc);
          }
          if (TILES == 1 && has_b) {
            // stage A is no longer needed: hand it back before working on stage B
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[slot_a]);
            released_a = true;
          }
          if (act_b) {
            const uint32_t p_lo = movmatrix_trans(pack_half2(pb[0], pb[1]));
            const uint32_t p_hi = movmatrix_trans(pack_half2(pb[2], pb[3]));
            value_tile(base_b + L::KV_TILE, p_lo, p_hi, acc);
          }
        }
        // this warp is done with the stages: let the producer refill them
        __syncwarp();
        if (alive && lane == 0) {
          if constexpr (TILES == 1) {
            if (!released_a) mbar_arrive(&empty_bar[slot_a]);
            if (has_b) mbar_arrive(&empty_bar[slot_b]);
          } else {
            if (last_touch) mbar_arrive(&empty_bar[slot_a]);
          }
        }
      }

#ifdef PA_TIMELINE
      if (ctid == 0) {
        PA_STAMP(4);
        PA_STAMP_VALUE(6, ++timeline_items);
      }
#endif
      if constexpr (MODE == MODE_SPLIT) {
        // the producer publishes the number of the next item (or "none") while it loads this
        // one, at the latest with the item's last batch of copies
        const uint32_t entry = item_no + 1, qs = entry & 1u, use = (entry - 1u) >> 1; // n-th use of the slot
        if (*abort_flag != 0u) alive = false;
        uint32_t next_index = kNoItem;
        if (alive) alive = mbar_wait_bounded(&sched_full[qs], use & 1u, abort_flag);
        if (alive) next_index = sched_item[qs];
        __syncwarp();
        if (alive && lane == 0) mbar_arrive(&sched_empty[qs]);
        if (next_index != kNoItem) nxt = cursor.seek(next_index, args, head_groups, lane);
        ++item_no;
      }
      // Q of the next item: issued now so that the loads fly during the epilogue below
      if (nxt.valid) load_q_fragments<D, KV>(qf, args, nxt.seq, nxt.head_base + my_head, gid, t4);

      l_run[0] = quad_column_sum(l_run[0]);
      l_run[1] = quad_column_sum(l_run[1]);
      const bool ok = (*abort_flag == 0u);

      if constexpr (MODE == MODE_SPLIT) {
        if (hpc == NW) {
          // ---- one warp per KV head: the warp holds the whole partition, write it out
          // (max_logits / exp_sums / tmp_out, reference paged_attention_kernel_v2.hpp:425-442,532-546)
          const size_t head0 = static_cast<size_t>(cur.seq) * args.num_heads + kv_head * G;
          const bool whole = args.whole_context_items != 0u;
#pragma unroll
          for (uint32_t j = 0; j < 2; ++j) {
            const uint32_t g = 2 * t4 + j;
            if (g < G && ok) {
              const size_t pidx = (head0 + g) * args.max_num_partitions + cur.partition;
              // report the true maximum; the sum is re-expressed relative to it
              const float l_true = l_run[j] * fast_exp2(m_ref[j] - m_true[j]);
              // normalised inside the partition (reference paged_attention_kernel_v2.hpp:386);
              // a whole-context item is the final result and goes to its row of `out`
              const float inv = (l_run[j] > 0.f) ? (out_scale / l_run[j]) : 0.f;
              __half *dst = whole ? args.out + (head0 + g) * D : args.tmp_out + pidx * D;
              if constexpr (KV == KV_F16) {
#pragma unroll
                for (uint32_t i = 0; i < KSTEPS; ++i) {
                  dst[i * 16 + gid] = __float2half_rn(acc[i][j] * inv);
                  dst[i * 16 + 8 + gid] = __float2half_rn(acc[i][2 + j] * inv);
                }
              } else {
#pragma unroll
                for (uint32_t q = 0; q < KSTEPS / 2; ++q) {
                  // even/odd tiles hold neighbouring dims: one 4-byte store per pair
                  *reinterpret_cast<uint32_t *>(dst + q * 32 + 2 * gid) =
                      pack_half2(acc[2 * q][j] * inv, acc[2 * q + 1][j] * inv);
                  *reinterpret_cast<uint32_t *>(dst + q * 32 + 16 + 2 * gid) =
                      pack_half2(acc[2 * q][2 + j] * inv, acc[2 * q + 1][2 + j] * inv);
                }
              }
              if (gid == 0 && !whole) {
                args.max_logits[pidx] = m_true[j] * kLn2;
                args.exp_sums[pidx] = l_true;
              }
            }
          }
        } else {
          // ---- the warps of a head split the tokens: merge them through shared memory in
          // a fixed order.  The stats slots alternate between items: a warp may publish the
          // next item's values while a slower warp still reads this item's.
          float *st_ref = warp_stats + item_parity * L::WARP_STATS_FLOATS;
          float *st_true = st_ref + NW * 8;
          float *st_sum = st_true + NW * 8;
          item_parity ^= 1u;
          if (gid == 0) {
#pragma unroll
            for (uint32_t j = 0; j < 2; ++j) {
              st_ref[cw * 8 + 2 * t4 + j] = m_ref[j];
              st_true[cw * 8 + 2 * t4 + j] = m_true[j];
              st_sum[cw * 8 + 2 * t4 + j] = l_run[j];
            }
          }
          named_barrier_sync(1, NCONS);
          const uint32_t w0 = my_head * slices; // first warp of this warp's head
          float f[2];
#pragma unroll
          for (uint32_t j = 0; j < 2; ++j) {
            float m_all = neg_infinity();
            for (uint32_t w = w0; w < w0 + slices; ++w) m_all = fmaxf(m_all, st_ref[w * 8 + 2 * t4 + j]);
            f[j] = (m_ref[j] == neg_infinity()) ? 0.f : fast_exp2(m_ref[j] - m_all);
          }
          // hpc = 1: slices 0,1 store into buffers 0,1 and slices 2,3 add to them;
          // hpc = 2: buffer = head, slice 0 stores and slice 1 adds
          const uint32_t buf_id = (hpc == 1) ? (my_slice & 1u) : my_head;
          const uint32_t round = (hpc == 1) ? (my_slice >> 1) : my_slice;
          float *buf = merge_buf + buf_id * (8 * D);
          if (round == 0) {
#pragma unroll
            for (uint32_t i = 0; i < KSTEPS; ++i) {
#pragma unroll
              for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t d = acc_dim_index<KV>(i, h, gid);
                buf[(2 * t4) * D + d] = acc[i][2 * h] * f[0];
                buf[(2 * t4 + 1) * D + d] = acc[i][2 * h + 1] * f[1];
              }
            }
          }
          named_barrier_sync(1, NCONS);
          if (round == 1) {
#pragma unroll
            for (uint32_t i = 0; i < KSTEPS; ++i) {
#pragma unroll
              for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t d = acc_dim_index<KV>(i, h, gid);
                buf[(2 * t4) * D + d] += acc[i][2 * h] * f[0];
                buf[(2 * t4 + 1) * D + d] += acc[i][2 * h + 1] * f[1];
              }
            }
          }
          named_barrier_sync(1, NCONS);
          // write out: thread -> (head, query column g, 8 consecutive dims)
          constexpr uint32_t THREADS_PER_ROW = D / 8;
          for (uint32_t idx = ctid; idx < hpc * 8 * THREADS_PER_ROW; idx += NCONS) {
            const uint32_t hh = idx / (8 * THREADS_PER_ROW);
            const uint32_t g = (idx / THREADS_PER_ROW) % 8;
            const uint32_t d0 = (idx % THREADS_PER_ROW) * 8;
            const uint32_t wb = hh * slices;
            float mr_all = neg_infinity(), mt_all = neg_infinity();
            for (uint32_t w = wb; w < wb + slices; ++w) {
              mr_all = fmaxf(mr_all, st_ref[w * 8 + g]);
              mt_all = fmaxf(mt_all, st_true[w * 8 + g]);
            }
            float l_all = 0.f;
            for (uint32_t w = wb; w < wb + slices; ++w) {
              const float mw = st_ref[w * 8 + g];
              l_all += (mw == neg_infinity()) ? 0.f : fast_exp2(mw - mr_all) * st_sum[w * 8 + g];
            }
            const float *b0 = merge_buf + ((hpc == 1) ? 0u : hh) * (8 * D) + g * D + d0;
            float4 lo = *reinterpret_cast<const float4 *>(b0);
            float4 hi = *reinterpret_cast<const float4 *>(b0 + 4);
            if (hpc == 1) {
              const float4 lo1 = *reinterpret_cast<const float4 *>(b0 + 8 * D);
              const float4 hi1 = *reinterpret_cast<const float4 *>(b0 + 8 * D + 4);
              lo.x += lo1.x; lo.y += lo1.y; lo.z += lo1.z; lo.w += lo1.w;
              hi.x += hi1.x; hi.y += hi1.y; hi.z += hi1.z; hi.w += hi1.w;
            }
            if (g < G && ok) {
              const size_t head = static_cast<size_t>(cur.seq) * args.num_heads + (cur.head_base + hh) * G + g;
              const size_t pidx = head * args.max_num_partitions + cur.partition;
              const float head_scale = (args.v_scale_per_head != nullptr)
                                           ? __ldg(args.v_scale_per_head + cur.head_base + hh)
                                           : args.out_scale;
              const float inv = (l_all > 0.f) ? (head_scale / l_all) : 0.f;
              uint4 packed;
              packed.x = pack_half2(lo.x * inv, lo.y * inv);
              packed.y = pack_half2(lo.z * inv, lo.w * inv);
              packed.z = pack_half2(hi.x * inv, hi.y * inv);
              packed.w = pack_half2(hi.z * inv, hi.w * inv);
              const bool whole = args.whole_context_items != 0u;
              __half *dst = whole ? args.out + head * D : args.tmp_out + pidx * D;
              *reinterpret_cast<uint4 *>(dst + d0) = packed;
              if (d0 == 0 && !whole) {
                args.max_logits[pidx] = mt_all * kLn2;
                args.exp_sums[pidx] = l_all * fast_exp2(mr_all - mt_all);
              }
            }
          }
        }
      } else {
        // ---- loop mode: park (O, m_ref, l) of this warp on the idle ring for the cluster merge
        named_barrier_sync(1, NCONS); // every consumer warp has finished reading the ring
        float *area = reinterpret_cast<float *>(smem) + cw * L::WARP_AREA_FLOATS;
        if (gid == 0) {
#pragma unroll
          for (uint32_t j = 0; j < 2; ++j) {
            area[8 * D + 2 * t4 + j] = m_ref[j];
            area[8 * D + 8 + 2 * t4 + j] = l_run[j];
          }
        }
#pragma unroll
        for (uint32_t i = 0; i < KSTEPS; ++i) {
#pragma unroll
          for (uint32_t h = 0; h < 2; ++h) {
            const uint32_t d = acc_dim_index<KV>(i, h, gid);
            area[(2 * t4) * D + d] = acc[i][2 * h];
            area[(2 * t4 + 1) * D + d] = acc[i][2 * h + 1];
          }
        }
      }
      cur = nxt;
    }
  }

  if constexpr (MODE == MODE_LOOP) {
    // ---- merge over the warps that share a head and over the CTAs of the cluster, through
    // distributed shared memory, in a fixed order.  Every thread of every CTA reaches both
    // cluster barriers, also after an abort.
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    if (num_ranks == 1) __syncthreads(); // a lone CTA has no peer to wait for
    else cluster.sync();
    if (threadIdx.x == 32) PA_STAMP(7);
    if (warp != 0) {
      // with few sources per row, more rows are merged per pass (16 partial rows in flight per
      // lane either way)
      const uint32_t sources = num_ranks * (NW / hpc);
      const bool ok = (*abort_flag == 0u);
      float *areas = reinterpret_cast<float *>(smem);
      if (sources <= 2)
        merge_cluster_rows<D, NW, L::WARP_AREA_FLOATS, 8, 2>(areas, args.out, args.v_scale_per_head, args.out_scale, args.group,
                                                                   args.num_heads, first.seq, first.head_base, hpc, cta_rank,
                                                                   num_ranks, warp - 1, lane, ok);
      else if (sources <= 4)
        merge_cluster_rows<D, NW, L::WARP_AREA_FLOATS, 4, 4>(areas, args.out, args.v_scale_per_head, args.out_scale, args.group,
                                                                   args.num_heads, first.seq, first.head_base, hpc, cta_rank,
                                                                   num_ranks, warp - 1, lane, ok);
      else
        merge_cluster_rows<D, NW, L::WARP_AREA_FLOATS, 2, 8>(areas, args.out, args.v_scale_per_head, args.out_scale, args.group,
                                                                   args.num_heads, first.seq, first.head_base, hpc, cta_rank,
                                                                   num_ranks, warp - 1, lane, ok);
    }
    if (num_ranks > 1) cluster.sync(); // peers may still be reading this CTA's shared memory
  }
  if constexpr (MODE == MODE_SPLIT) {
    if (threadIdx.x == 0) {
      // retire: the last CTA of the launch hands the counters back zeroed
      __threadfence();
      const unsigned int done = atomicAdd(&g_sched[args.sched_slot][1], 1u);
      if (done == gridDim.x - 1) {
        g_sched[args.sched_slot][0] = 0u;
        g_sched[args.sched_slot][1] = 0u;
        __threadfence();
      }
    }
  }
  if (threadIdx.x == 32) PA_STAMP(5);
  // after a give-up the CTA's shared memory stays allocated until its last thread has left,
  // which is the producer lane once the copies in flight have landed (see above)
  if (*abort_flag != 0u && threadIdx.x == 32) atomicExch(&g_pa_device_status, 4);
}
} // namespace

// Context length as the attention kernel cut it (load_context): the merge reads exactly the
// partitions that kernel wrote.
__device__ __forceinline__ uint32_t merge_context(const uint32_t *context_lens, uint32_t seq, uint32_t ctx_limit,
                                                  const uint32_t *table_offsets, uint32_t block_shift) {
  const uint32_t ctx = context_lens[seq];
  if (table_offsets == nullptr) return min(ctx, ctx_limit);
  const uint64_t row_tokens = static_cast<uint64_t>(table_offsets[seq + 1] - table_offsets[seq]) << block_shift;
  return static_cast<uint32_t>(min(static_cast<uint64_t>(ctx), row_tokens));
}

// Second kernel of the split-context variant: one CTA per (sequence, head).
//   M = max_p m_p ; w_p = l_p * exp(m_p - M) ; W = sum w_p
//   out[d] = sum_p (w_p / W) * tmp_out[p, d]
// over the partitions p < ceil(ctx / partition_size) only
// (reference paged_attention_kernel_v2.hpp:679,736-764,813-863,924-932).
// Latency-bound: a thread owns 4 dims (one 8-byte load) of kMergeUnroll partial rows, which
// are requested together with the statistics, before the weights are known; up to
// kMergeUnroll * ROWS partitions (64 for head size 128: a context of 32768 tokens) cost one
// memory round trip after the context length has arrived.
constexpr uint32_t kMergeUnroll = 16; // partial rows in flight per thread

template <int D>
struct MergeShape {
  static constexpr uint32_t LANES_PER_ROW = D / 4;        // each lane owns 4 dims (8 bytes)
  static constexpr uint32_t ROWS = 128 / LANES_PER_ROW;   // partitions handled in parallel: 4 or 8
};

template <int D>
__global__ void __launch_bounds__(128, 8) // 64 registers: 1 184 CTAs resident, config 4's 1 024 pairs in one wave
merge_partitions_kernel(__half *__restrict__ out, const __half *__restrict__ tmp_out,
                        const float *__restrict__ max_logits, const float *__restrict__ exp_sums,
                        const uint32_t *__restrict__ context_lens, const uint32_t *__restrict__ seq_indices,
                        uint32_t num_heads, uint32_t max_num_partitions, uint32_t partition_size,
                        uint32_t ctx_limit, const uint32_t *__restrict__ table_offsets, uint32_t block_shift) {
  constexpr uint32_t LANES_PER_ROW = MergeShape<D>::LANES_PER_ROW;
  constexpr uint32_t ROWS = MergeShape<D>::ROWS;
  constexpr uint32_t UNROLL = kMergeUnroll;
  constexpr uint32_t WEIGHT_CACHE = 1024;           // weights kept in shared memory
  const uint32_t head = blockIdx.x;
  const uint32_t seq = (seq_indices != nullptr) ? __ldg(seq_indices + blockIdx.y) : blockIdx.y;
  const uint32_t tid = threadIdx.x;
  // Launched with programmatic stream serialization, this grid may start while the attention
  // kernel drains; nothing is read before that kernel has completed and its writes are visible.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const size_t base = (static_cast<size_t>(seq) * num_heads + head) * max_num_partitions;
  __half *orow = out + (static_cast<size_t>(seq) * num_heads + head) * D;

  __shared__ float red[4];
  __shared__ float weights[WEIGHT_CACHE];
  __shared__ float part[ROWS][D];

  const uint32_t row = tid / LANES_PER_ROW;
  const uint32_t col = (tid % LANES_PER_ROW) * 4;
  // The first UNROLL rows of this thread and the first 128 partitions' statistics are requested
  // together with the context length, for every partition the scratch has room for: rows past
  // the context hold whatever the caller left there and are masked once the length is known.
  // One memory round trip instead of two.
  uint2 raw[UNROLL];
#pragma unroll
  for (uint32_t u = 0; u < UNROLL; ++u) {
    const uint32_t p = row + u * ROWS;
    raw[u] = (p < max_num_partitions) ? __ldg(reinterpret_cast<const uint2 *>(tmp_out + (base + p) * D + col))
                                      : make_uint2(0u, 0u);
  }
  float ml_own = (tid < max_num_partitions) ? max_logits[base + tid] : neg_infinity();
  float es_own = (tid < max_num_partitions) ? exp_sums[base + tid] : 0.f;
  const uint32_t ctx = merge_context(context_lens, seq, ctx_limit, table_offsets, block_shift);
  const uint32_t np = min(num_partitions_of(ctx, partition_size), max_num_partitions);
  if (tid >= np) {
    ml_own = neg_infinity();
    es_own = 0.f;
  }

  // global max over partitions; the first 128 partitions' statistics stay in registers, so
  // the weights below need no second trip to memory
  float m = ml_own;
  for (uint32_t p = tid + 128; p < np; p += 128) m = fmaxf(m, max_logits[base + p]);
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31u) == 0) red[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  // rescaled weights and their total
  float wsum = 0.f;
  if (tid < np) {
    const float w = es_own * __expf(ml_own - m);
    weights[tid] = w;
    wsum = w;
  }
  for (uint32_t p = tid + 128; p < np; p += 128) {
    const float w = exp_sums[base + p] * __expf(max_logits[base + p] - m);
    if (p < WEIGHT_CACHE) weights[p] = w;
    wsum += w;
  }
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
  if ((tid & 31u) == 0) red[tid >> 5] = wsum;
  __syncthreads();
  wsum = red[0] + red[1] + red[2] + red[3];
  const float inv_w = (wsum > 0.f) ? 1.f / wsum : 0.f;
  auto weight_of = [&](uint32_t p) -> float {
    return (p < WEIGHT_CACHE) ? weights[p] : exp_sums[base + p] * __expf(max_logits[base + p] - m);
  };

  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  auto accumulate = [&](uint2 v, float w) {
    const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    a0 += w * v01.x;
    a1 += w * v01.y;
    a2 += w * v23.x;
    a3 += w * v23.y;
  };
  // partitions are taken in increasing order per thread: the sum has a fixed order
#pragma unroll
  for (uint32_t u = 0; u < UNROLL; ++u) {
    const uint32_t p = row + u * ROWS;
    if (p < np) accumulate(raw[u], weight_of(p) * inv_w);
  }
  for (uint32_t p0 = row + UNROLL * ROWS; p0 < np; p0 += UNROLL * ROWS) {
#pragma unroll
    for (uint32_t u = 0; u < UNROLL; ++u) {
      const uint32_t p = p0 + u * ROWS;
      raw[u] = (p < np) ? __ldg(reinterpret_cast<const uint2 *>(tmp_out + (base + p) * D + col)) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (uint32_t u = 0; u < UNROLL; ++u) {
      const uint32_t p = p0 + u * ROWS;
      if (p < np) accumulate(raw[u], weight_of(p) * inv_w);
    }
  }
  part[row][col] = a0;
  part[row][col + 1] = a1;
  part[row][col + 2] = a2;
  part[row][col + 3] = a3;
  __syncthreads();
  if (tid < D / 2) {
    // one accumulator per residue class p mod ROWS, classes added in increasing order
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < ROWS; ++r) {
      s0 += part[r][2 * tid];
      s1 += part[r][2 * tid + 1];
    }
    *reinterpret_cast<uint32_t *>(orow + 2 * tid) = pack_half2(s0, s1);
  }
}

// Variant of merge_partitions_kernel for batches with many (sequence, head) pairs: one WARP
// per pair (four pairs per CTA), no shared memory and no block barrier.  Each lane owns
// D / 32 dims of the row.  Every sum is taken in the order merge_partitions_kernel uses
// (weights: four 32-wide shuffle trees added left to right; rows: one accumulator per
// residue class p mod ROWS, classes added in increasing order), so both kernels produce the
// same bits and the launcher may pick either.
template <int D>
__global__ void __launch_bounds__(128)
merge_partitions_warp_kernel(__half *__restrict__ out, const __half *__restrict__ tmp_out,
                             const float *__restrict__ max_logits, const float *__restrict__ exp_sums,
                             const uint32_t *__restrict__ context_lens,
                             const uint32_t *__restrict__ seq_indices, uint32_t num_heads,
                             uint32_t num_pairs, uint32_t max_num_partitions, uint32_t partition_size,
                             uint32_t ctx_limit, const uint32_t *__restrict__ table_offsets,
                             uint32_t block_shift) {
  constexpr uint32_t DPL = D / 32;                 // dims per lane: 4 or 2
  constexpr uint32_t ROWS = MergeShape<D>::ROWS;   // residue classes of the CTA-per-pair kernel
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t work = blockIdx.x * 4 + (threadIdx.x >> 5); // (position in the launch) * num_heads + head
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (work >= num_pairs) return;
  const uint32_t pos = work / num_heads;
  const uint32_t seq = (seq_indices != nullptr) ? __ldg(seq_indices + pos) : pos;
  const uint32_t pair = seq * num_heads + (work - pos * num_heads); // seq * num_heads + head
  const uint32_t ctx = merge_context(context_lens, seq, ctx_limit, table_offsets, block_shift);
  const uint32_t np = min(num_partitions_of(ctx, partition_size), max_num_partitions);
  const size_t base = static_cast<size_t>(pair) * max_num_partitions;
  const __half *rows = tmp_out + base * D + lane * DPL;

  // the first 32 partitions' statistics live in registers, one partition per lane; their
  // rows are requested right away, before the weights are known
  const bool mine = lane < np;
  const float ml_lane = mine ? __ldg(max_logits + base + lane) : neg_infinity();
  const float es_lane = mine ? __ldg(exp_sums + base + lane) : 0.f;
  constexpr uint32_t PREFETCH = 2 * ROWS;
  uint2 pre[PREFETCH];
#pragma unroll
  for (uint32_t u = 0; u < PREFETCH; ++u) {
    pre[u] = make_uint2(0u, 0u);
    if (u < np) {
      if constexpr (DPL == 4) pre[u] = __ldg(reinterpret_cast<const uint2 *>(rows + static_cast<size_t>(u) * D));
      else pre[u].x = __ldg(reinterpret_cast<const uint32_t *>(rows + static_cast<size_t>(u) * D));
    }
  }
  float m = ml_lane;
  for (uint32_t p = lane + 32; p < np; p += 32) m = fmaxf(m, max_logits[base + p]);
#pragma unroll
  for (uint32_t o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  // total weight: chunk c plays warp c of the CTA-per-pair kernel (threads 32c .. 32c+31)
  const float w_lane = mine ? es_lane * __expf(ml_lane - m) : 0.f;
  float wsum = 0.f;
#pragma unroll
  for (uint32_t c = 0; c < 4; ++c) {
    float part = (c == 0) ? w_lane : 0.f;
    for (uint32_t p = 32 * c + lane + (c == 0 ? 128u : 0u); p < np; p += 128)
      part += exp_sums[base + p] * __expf(max_logits[base + p] - m);
#pragma unroll
    for (uint32_t o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    wsum = (c == 0) ? part : wsum + part;
  }
  const float inv_w = (wsum > 0.f) ? 1.f / wsum : 0.f;

  float acc[ROWS][DPL];
#pragma unroll
  for (uint32_t r = 0; r < ROWS; ++r)
#pragma unroll
    for (uint32_t i = 0; i < DPL; ++i) acc[r][i] = 0.f;
  auto add_row = [&](uint32_t r, uint2 raw, float w) {
    const float2 v01 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    acc[r][0] += w * v01.x;
    acc[r][1] += w * v01.y;
    if constexpr (DPL == 4) {
      const float2 v23 = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
      acc[r][2] += w * v23.x;
      acc[r][3] += w * v23.y;
    }
  };
  // partitions 0 .. PREFETCH-1 from the prefetched rows (weights come from the owning lane)
#pragma unroll
  for (uint32_t u = 0; u < PREFETCH; ++u) {
    const float w = __shfl_sync(0xffffffffu, w_lane, u) * inv_w;
    if (u < np) add_row(u % ROWS, pre[u], w);
  }
  // the rest in groups of PREFETCH partitions: all rows and statistics of a group are requested
  // before the first is used (a long sequence is a chain of such groups, so the depth of a
  // group sets its latency); within a residue class the partitions still add in increasing order
  for (uint32_t p0 = PREFETCH; p0 < np; p0 += PREFETCH) {
    float ml[PREFETCH], es[PREFETCH];
#pragma unroll
    for (uint32_t u = 0; u < PREFETCH; ++u) {
      const uint32_t p = p0 + u;
      pre[u] = make_uint2(0u, 0u);
      ml[u] = neg_infinity();
      es[u] = 0.f;
      if (p < np) {
        if constexpr (DPL == 4) pre[u] = __ldg(reinterpret_cast<const uint2 *>(rows + static_cast<size_t>(p) * D));
        else pre[u].x = __ldg(reinterpret_cast<const uint32_t *>(rows + static_cast<size_t>(p) * D));
        ml[u] = max_logits[base + p];
        es[u] = exp_sums[base + p];
      }
    }
#pragma unroll
    for (uint32_t u = 0; u < PREFETCH; ++u)
      if (p0 + u < np) add_row(u % ROWS, pre[u], es[u] * __expf(ml[u] - m) * inv_w);
  }
  float total[DPL];
#pragma unroll
  for (uint32_t i = 0; i < DPL; ++i) {
    float s = 0.f;
#pragma unroll
    for (uint32_t r = 0; r < ROWS; ++r) s += acc[r][i];
    total[i] = s;
  }
  __half *orow = out + static_cast<size_t>(pair) * D + lane * DPL;
  if constexpr (DPL == 4) {
    *reinterpret_cast<uint2 *>(orow) = make_uint2(pack_half2(total[0], total[1]), pack_half2(total[2], total[3]));
  } else {
    *reinterpret_cast<uint32_t *>(orow) = pack_half2(total[0], total[1]);
  }
}

} // namespace pa
