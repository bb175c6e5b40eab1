// Host side shared by the four launchers: argument validation, TMA descriptor
// encoding, the run-time -> compile-time dispatch on (head_size, kv type), the
// launch geometry and the optional blocking timing.  Mirrors what the
// reference's dispatch_* / launch_* pairs do on the host
// (reference paged_attention_loop/launch_kernels_loop.h:16-54,56-173 and
// paged_attention_reduce/launch_kernels_reduce.h:18-78,80-197).
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "paged_attention_b200.h"
#include "paged_attention_kernels.cuh"

namespace pa {

// ------------------------------------------------------------------ errors
void set_last_error(const char *fmt, ...); // defined in host_common.cu
int fail(int code, const char *fmt, ...);  // sets the message, returns code
const char *last_error();                  // message of the last failure on this thread

#define PA_CUDA_TRY(expr)                                                               \
  do {                                                                                  \
    cudaError_t err__ = (expr);                                                         \
    if (err__ != cudaSuccess)                                                           \
      return ::pa::fail(PA_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
  } while (0)

// ------------------------------------------------------- TMA descriptor setup
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled(); // defined in host_common.cu; nullptr if the driver lacks it

// Describes one cache tensor to the TMA unit as (head dim, token row, KV head): extents
// (head_size, num_blocks*block_size, num_kv_heads), strides (1 elem, num_kv_heads*head_size
// elems, head_size elems).  A box is (one 128-byte slab, rows_per_box rows, heads_per_box
// heads) and lands in shared memory as [head][row][slab]; rows past the cache read as zero.
template <int D, int KV>
int encode_cache_map(CUtensorMap *map, const void *cache, const pa_params *p, uint32_t rows_per_box,
                     uint32_t heads_per_box) {
  using geo = kv_tile_geometry<D, KV>;
  // A decode loop calls with the same cache pointer and shape step after step: the last few
  // descriptors of this thread are kept and reused (encoding one costs about a microsecond of
  // host time, which a call on a tiny batch notices).
  struct Entry {
    const void *cache;
    uint64_t num_blocks;
    uint32_t block_size, num_kv_heads, rows_per_box, heads_per_box;
    bool valid;
    CUtensorMap map;
  };
  constexpr uint32_t kEntries = 8;
  static thread_local Entry recent[kEntries] = {};
  static thread_local uint32_t next_victim = 0;
  for (const Entry &e : recent)
    if (e.valid && e.cache == cache && e.num_blocks == p->num_blocks && e.block_size == p->block_size &&
        e.num_kv_heads == p->num_kv_heads && e.rows_per_box == rows_per_box && e.heads_per_box == heads_per_box) {
      *map = e.map;
      return PA_OK;
    }
  EncodeTiledFn encode = get_encode_tiled();
  if (encode == nullptr) return fail(PA_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(p->num_blocks) * p->block_size,
                              static_cast<cuuint64_t>(p->num_kv_heads)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(p->num_kv_heads) * D * geo::elt_bytes,
                                 static_cast<cuuint64_t>(D) * geo::elt_bytes};
  const cuuint32_t box[3] = {geo::slab_elems, rows_per_box, heads_per_box};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      (KV == KV_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapSwizzle sw =
      (geo::slab_bytes == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  // 256-byte L2 promotion measured best; a -DPA_TUNING_KNOBS build reads
  // PA_TMA_L2_PROMOTION=0..3 (none, 64 B, 128 B, 256 B) instead
#ifdef PA_TUNING_KNOBS
  static const int promo = [] {
    const char *e = std::getenv("PA_TMA_L2_PROMOTION");
    return (e != nullptr && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 3;
  }();
#else
  constexpr int promo = 3;
#endif
  const CUtensorMapL2promotion l2 = promo == 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                    : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                    : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  const CUresult r = encode(map, dt, 3, const_cast<void *>(cache), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, l2, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PA_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  Entry &slot = recent[next_victim];
  next_victim = (next_victim + 1) % kEntries;
  slot.cache = cache;
  slot.num_blocks = p->num_blocks;
  slot.block_size = p->block_size;
  slot.num_kv_heads = p->num_kv_heads;
  slot.rows_per_box = rows_per_box;
  slot.heads_per_box = heads_per_box;
  slot.map = *map;
  slot.valid = true;
  return PA_OK;
}

// ----------------------------------------------------------------- validation
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Checks shared by all entry points.  `fp8_entry` selects which kv_dtype values
// the entry point accepts; `needs_scratch` is true for the split variant.
inline int validate_params(const pa_params *p, bool fp8_entry, bool needs_scratch) {
  if (p == nullptr) return fail(PA_ERR_BAD_ARG, "params is null");
  // the two checks the reference makes, with its messages
  // (launch_kernels_loop.h:114-115,170-172)
  const bool head_ok = p->head_size == 128 || p->head_size == 64;
  const bool block_ok = p->block_size == 16 || p->block_size == 32 || p->block_size == 64 ||
                        p->block_size == 128;
  if (!head_ok || !block_ok) return fail(PA_ERR_UNSUPPORTED, "Unsupported head size or block size");
  if (p->num_queries_per_tokens < 1 || p->num_queries_per_tokens > 8)
    return fail(PA_ERR_UNSUPPORTED, "Unsupported number of queries per token");
  if (fp8_entry) {
    if (p->kv_dtype != PA_KV_FP8_E5M2 && p->kv_dtype != PA_KV_FP8_E4M3)
      return fail(PA_ERR_BAD_ARG, "FP8 entry point needs kv_dtype e5m2 or e4m3, got %d", p->kv_dtype);
  } else if (p->kv_dtype != PA_KV_F16) {
    return fail(PA_ERR_BAD_ARG, "fp16 entry point needs kv_dtype f16, got %d", p->kv_dtype);
  }
  if (!(p->sm_scale > 0.f) || (fp8_entry && !(p->fp8_scale > 0.f)))
    return fail(PA_ERR_BAD_ARG, "sm_scale and fp8_scale must be positive and finite");
  if (!fp8_entry && (p->k_scale_per_head != nullptr || p->v_scale_per_head != nullptr ||
                     p->k_scale_per_block != nullptr || p->v_scale_per_block != nullptr))
    return fail(PA_ERR_BAD_ARG, "per-head and per-block scales belong to the FP8 entry points");
  if ((p->k_scale_per_block != nullptr) != (p->v_scale_per_block != nullptr))
    return fail(PA_ERR_BAD_ARG, "k_scale_per_block and v_scale_per_block must be set together");
  if (p->k_scale_per_block != nullptr && (p->k_scale_per_head != nullptr || p->v_scale_per_head != nullptr))
    return fail(PA_ERR_BAD_ARG, "per-block and per-head scales exclude each other");
  if (p->num_seqs == 0) return PA_OK; // nothing to do; the launcher returns early
  if (!p->out || !p->query || !p->key_cache || !p->value_cache || !p->block_tables || !p->context_lens)
    return fail(PA_ERR_BAD_ARG, "a required pointer is null");
  if (p->num_kv_heads == 0 || p->num_heads != p->num_kv_heads * p->num_queries_per_tokens)
    return fail(PA_ERR_BAD_ARG, "num_heads (%u) != num_kv_heads (%u) * num_queries_per_tokens (%u)",
                p->num_heads, p->num_kv_heads, p->num_queries_per_tokens);
  if (p->num_blocks == 0 || (p->max_blocks_per_seq == 0 && p->block_table_offsets == nullptr))
    return fail(PA_ERR_BAD_ARG, "num_blocks and max_blocks_per_seq must be positive");
  if (p->num_blocks * p->block_size >= (1ull << 31))
    return fail(PA_ERR_BAD_ARG, "cache has too many token rows for a 32-bit TMA coordinate");
  if (p->num_seqs > 65535u || p->num_kv_heads > 65535u)
    return fail(PA_ERR_BAD_ARG, "num_seqs and num_kv_heads are limited to 65535");
  if (!aligned16(p->key_cache) || !aligned16(p->value_cache))
    return fail(PA_ERR_BAD_ARG, "key_cache / value_cache must be 16-byte aligned");
  if (!aligned16(p->query) || !aligned16(p->out))
    return fail(PA_ERR_BAD_ARG, "query / out must be 16-byte aligned");
  if (static_cast<uint64_t>(p->num_seqs) * p->num_kv_heads * (needs_scratch ? p->max_num_partitions : 1u) >=
      (1ull << 32))
    return fail(PA_ERR_BAD_ARG, "too many work items for a 32-bit index");
  if (needs_scratch) {
    if (!p->max_logits || !p->exp_sums || !p->tmp_out)
      return fail(PA_ERR_BAD_ARG, "the reduce variant needs max_logits, exp_sums and tmp_out");
    if (p->max_num_partitions == 0 || p->max_num_partitions > 65535u)
      return fail(PA_ERR_BAD_ARG, "max_num_partitions must be in 1..65535");
    if (!aligned16(p->tmp_out))
      return fail(PA_ERR_BAD_ARG, "tmp_out must be 16-byte aligned");
  }
  return PA_OK;
}

// ------------------------------------------------------------------ geometry
struct DeviceInfo {
  int sm_count;
  int cc_major;
};
int get_device_info(DeviceInfo *info); // cached per device; defined in host_common.cu

// Longest context a sequence's block-table row can address, saturated to 32 bits.
inline uint32_t context_limit(const pa_params *p) {
  if (p->block_table_offsets != nullptr) return 0xffffffffu; // per sequence, known on the device only
  const uint64_t tokens = static_cast<uint64_t>(p->max_blocks_per_seq) * p->block_size;
  return tokens > 0xffffffffull ? 0xffffffffu : static_cast<uint32_t>(tokens);
}

// The caller's context-length hint, cut to what the block tables can address (0 = unknown).
inline uint32_t context_hint(const pa_params *p) { return std::min(p->max_context_len, context_limit(p)); }

// Cluster size of the loop variant: enough CTAs to give every SM two, using
// only what the host knows (num_seqs, num_kv_heads and the context-length hint).
inline uint32_t choose_cluster_size(const pa_params *p, uint32_t hpc, int sm_count, uint32_t tokens_per_stage,
                                    uint32_t bytes_per_element) {
#ifdef PA_TUNING_KNOBS
  // tuning build only: PA_LOOP_CLUSTER=1..8 forces the cluster size
  static const int forced = [] {
    const char *e = std::getenv("PA_LOOP_CLUSTER");
    const int v = e ? std::atoi(e) : 0;
    return (v >= 1 && v <= 8) ? v : 0;
  }();
  if (forced != 0) return static_cast<uint32_t>(forced);
#endif
  // Any size up to 8 is portable, not only powers of two.  With fewer units than CTA slots the
  // cluster is as large as still lets every cluster be resident at once (one wave, no slot
  // left empty that a whole cluster could fill).  With more units than that the CTAs run in
  // waves and every further CTA costs a launch ramp and a merge (measured on 1024 ragged
  // sequences: clusters of 2 are 6 % faster than single CTAs, clusters of 3 already 5 % slower),
  // so clusters of 2 are used, which halve the time a CTA spends on the longest sequence, unless
  // the contexts are known to be short.
  const uint64_t units = static_cast<uint64_t>(p->num_seqs) * (p->num_kv_heads / hpc);
  const uint64_t slots = 2ull * static_cast<uint64_t>(sm_count);
  uint32_t cs = units >= slots ? 1u : static_cast<uint32_t>(std::min<uint64_t>(8ull, slots / units));
  if (cs == 1 && (units < 2 * slots || context_hint(p) == 0 || context_hint(p) >= 2048u)) cs = 2;
  // With few units one long sequence can outlast all the others together: a CTA streams about
  // 25-45 GB/s, so a unit of 32 MB on two CTAs takes 500 us whatever else the launch holds.  Up to
  // two waves of units, the cluster grows until a CTA's share of the longest possible unit is at
  // most 4 MiB (128 log-normal contexts up to 32768 tokens, 8 KV heads, e5m2: 174 us with 8 CTAs per
  // unit, 509 us with 2; uniform batches of 8192-token contexts keep their 2, where 4 are 5 %
  // and 8 are 20 % slower).
  if (context_hint(p) != 0 && units < 2 * slots) {
    const uint64_t longest_unit =
        static_cast<uint64_t>(context_hint(p)) * hpc * p->head_size * 2ull * bytes_per_element;
    const uint64_t wanted = (longest_unit + (4ull << 20) - 1) / (4ull << 20);
    cs = static_cast<uint32_t>(std::min<uint64_t>(8ull, std::max<uint64_t>(cs, wanted)));
  }
  if (context_hint(p) != 0) {
    // a CTA should own at least kMinStagesPerCta stages of the longest context: below that the
    // cluster merge and the extra CTAs cost more than the split saves
    constexpr uint32_t kMinStagesPerCta = 2;
    const uint32_t stages = divide_round_up(context_hint(p), tokens_per_stage);
    while (cs > 1 && stages / cs < kMinStagesPerCta) --cs;
  }
  return cs;
}

// KV heads per CTA: with 4 (8 in the wide CTA) a warp owns a head and nothing is merged across
// warps; fewer when the head count does not divide.
inline uint32_t choose_heads_per_cta(const pa_params *p, bool wide, bool loop_mode, int sm_count) {
  if (wide) return 8u; // the wide CTA is only chosen for num_kv_heads % 8 == 0: a warp per head
  uint32_t hpc = (p->num_kv_heads % 4 == 0) ? 4u : ((p->num_kv_heads % 2 == 0) ? 2u : 1u);
#ifdef PA_TUNING_KNOBS
  {
    // tuning build only: PA_FORCE_HPC=1|2 lowers the number of KV heads per CTA
    static const int forced = [] {
      const char *e = std::getenv("PA_FORCE_HPC");
      return e ? std::atoi(e) : 0;
    }();
    if ((forced == 1 || forced == 2) && static_cast<uint32_t>(forced) < hpc) hpc = forced;
  }
#endif
  // The loop variant has one cluster of at most 8 CTAs per (sequence, head group): with very
  // few sequences, fewer heads per CTA (warps then split the tokens of a head) is the only
  // way to put a CTA on every SM
  if (loop_mode)
    while (hpc > 1 && static_cast<uint64_t>(p->num_seqs) * (p->num_kv_heads / hpc) * 8ull <
                          static_cast<uint64_t>(sm_count))
      hpc /= 2;
  return hpc;
}

// Largest number of tiles per warp and stage for which the kernel is built, per (head size, KV
// type): the stage must stay at 32 KB or less so that the ring keeps three of them.
template <int D, int KV>
constexpr uint32_t max_stage_tiles() {
  return (KV == KV_F16) ? (D == 128 ? 1u : 2u) : (D == 128 ? 2u : 4u);
}

// Tiles per warp and stage for one launch: as many as let one TMA box still fill a head's rows
// of the stage, i.e. 16 * slices * tiles <= block_size (slices = warps per head).  KV blocks of 16
// tokens keep one tile; blocks of 32 and more get boxes of up to 16 KB.
template <int D, int KV>
uint32_t choose_stage_tiles(const pa_params *p, uint32_t hpc, uint32_t consumer_warps) {
  const uint32_t step_tokens = 16u * (consumer_warps / hpc);
  uint32_t tiles = max_stage_tiles<D, KV>();
  while (tiles > 1u && step_tokens * tiles > p->block_size) tiles /= 2u;
  return tiles;
}

template <int D, int KV, int NWARPS = 4, int TILES = 1>
AttnArgs make_attn_args(const pa_params *p, uint32_t hpc) {
  using policy = paged_attention_policy_v2<D, KV, NWARPS, TILES>;
  AttnArgs a{};
  a.query = static_cast<const __half *>(p->query);
  a.out = static_cast<__half *>(p->out);
  a.max_logits = p->max_logits;
  a.exp_sums = p->exp_sums;
  a.tmp_out = static_cast<__half *>(p->tmp_out);
  a.sinks = static_cast<const __half *>(p->sinks);
  a.block_tables = p->block_tables;
  a.context_lens = p->context_lens;
  a.num_seqs = p->num_seqs;
  a.num_heads = p->num_heads;
  a.num_kv_heads = p->num_kv_heads;
  a.group = p->num_queries_per_tokens;
  a.max_blocks_per_seq = p->max_blocks_per_seq;
  a.num_blocks = static_cast<uint32_t>(p->num_blocks); // validated: num_blocks * block_size < 2^31
  a.max_num_partitions = p->max_num_partitions;
  a.block_shift = log2_pow2(p->block_size);
  a.ctx_limit = context_limit(p);
  a.partition_shift = log2_pow2(policy::partition_size);
  a.whole_context_items = 0u;
  a.table_offsets = p->block_table_offsets;
  a.hpc = hpc;
  a.tokens_per_stage = policy::tokens_per_stage / a.hpc;
  a.rows_per_box = p->block_size < a.tokens_per_stage ? p->block_size : a.tokens_per_stage;
  a.boxes_per_stage = a.hpc * (a.tokens_per_stage / a.rows_per_box);
  // one TMA box spans all of the CTA's heads when a box fills the stage's rows of a head
  a.heads_per_box = (a.rows_per_box == a.tokens_per_stage) ? a.hpc : 1u;
  // with per-block scales every tile brings its own K and V scale and fp8_scale is not used
  const bool per_block = (KV != KV_F16) && p->k_scale_per_block != nullptr;
  const float kv_scale = (KV == KV_F16 || per_block) ? 1.f : p->fp8_scale;
  // the FP8 scale is applied once, hoisted out of the dot products
  // (reference paged_attention_kernel_fp8_loop.hpp:333,545)
  a.scale_log2 = p->sm_scale * kv_scale * kLog2e;
  a.out_scale = kv_scale;
  a.sm_scale_log2 = p->sm_scale * kLog2e;
  a.k_scale_per_head = (KV == KV_F16) ? nullptr : p->k_scale_per_head;
  a.v_scale_per_head = (KV == KV_F16) ? nullptr : p->v_scale_per_head;
  a.k_scale_per_block = per_block ? p->k_scale_per_block : nullptr;
  a.v_scale_per_block = per_block ? p->v_scale_per_block : nullptr;
  a.seq_indices = p->seq_indices;
  a.alibi_slopes = p->alibi_slopes;
  a.softcap = (p->softcap > 0.f) ? p->softcap : 0.f;
  return a;
}

// Enqueues the attention kernel of one (D, KV, MODE, CTA shape, stage size) instantiation.
// `whole_context_items` (split mode only): the persistent kernel on behalf of the loop variant,
// one work item per (sequence, head group), results straight into `out`, no scratch, no merge.
// (internal linkage, like everything below that launches the unit's own kernel copies or touches its tables:
// two launchers may hold the same instantiation, and merged definitions would launch the other unit's kernels)
template <int D, int KV, int MODE, int NWARPS = 4, int TILES = 1>
static int enqueue_attention(const pa_params *p, cudaStream_t stream, uint32_t hpc, bool whole_context_items = false) {
  static_assert(NWARPS == 4 || MODE == MODE_SPLIT, "the wide CTA exists for the split variant only");
  static_assert(NWARPS == 4 || TILES == 1, "the wide CTA is built with one tile per stage");
  using L = SmemLayout<D, KV, NWARPS, TILES>;
  using policy = typename L::policy;
  DeviceInfo dev{};
  if (int rc = get_device_info(&dev)) return rc;
  if (dev.cc_major < 10) return fail(PA_ERR_CUDA, "this library needs an sm_100a device");

  AttnArgs args = make_attn_args<D, KV, NWARPS, TILES>(p, hpc);
  if (MODE == MODE_SPLIT && whole_context_items) {
    args.whole_context_items = 1u;
    args.max_num_partitions = 1u;
    args.max_logits = nullptr;
    args.exp_sums = nullptr;
    args.tmp_out = nullptr;
  }
  if (MODE == MODE_SPLIT) {
    // one allocator per translation unit, like the counter table it indexes
    // (the legacy default stream cannot be captured, and asking about it while another stream
    // captures in global mode would invalidate that capture)
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (stream != nullptr && stream != cudaStreamLegacy) PA_CUDA_TRY(cudaStreamIsCapturing(stream, &capture));
    args.sched_slot = next_sched_slot(capture != cudaStreamCaptureStatusNone);
  }
  CUtensorMap map_k, map_v;
  if (int rc = encode_cache_map<D, KV>(&map_k, p->key_cache, p, args.rows_per_box, args.heads_per_box)) return rc;
  if (int rc = encode_cache_map<D, KV>(&map_v, p->value_cache, p, args.rows_per_box, args.heads_per_box)) return rc;

  auto kernel = paged_attention_kernel<D, KV, MODE, NWARPS, TILES>;
  static thread_local int configured_device = -1;
  int device = 0;
  PA_CUDA_TRY(cudaGetDevice(&device));
  if (configured_device != device) {
    PA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_SMEM));
    configured_device = device;
  }

  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  cfg.blockDim = dim3(policy::threads_per_cta, 1, 1);
  cfg.dynamicSmemBytes = L::DYN_SMEM;
  cfg.stream = stream;
  if (MODE == MODE_SPLIT) {
    // persistent CTAs, as many as fit on the device, each walking the (seq, partition, kv head) items with
    // stride gridDim.x; the TMA ring keeps streaming across item boundaries
    const uint64_t items = static_cast<uint64_t>(p->num_kv_heads / args.hpc) * args.max_num_partitions * p->num_seqs;
    const uint64_t resident = static_cast<uint64_t>(policy::ctas_per_sm) * static_cast<uint64_t>(dev.sm_count);
    cfg.gridDim = dim3(static_cast<unsigned>(items < resident ? items : resident), 1, 1);
    // programmatic dependent launch: back-to-back calls overlap this grid's start-up with the
    // previous kernel's tail (the kernel blocks in griddepcontrol.wait before its first read)
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else {
    // portable cluster sizes only: 9..16 CTAs per cluster measured 30-40 % slower on B200
    // (fewer clusters fit a GPC at once)
    const uint32_t cs = choose_cluster_size(p, args.hpc, dev.sm_count, args.tokens_per_stage, KV == KV_F16 ? 2u : 1u);
    // the order in which clusters start only matters when they do not all fit at once
    const uint64_t ctas = static_cast<uint64_t>(cs) * (p->num_kv_heads / args.hpc) * p->num_seqs;
    args.longest_first_hint = (ctas > 2ull * static_cast<uint64_t>(dev.sm_count)) ? context_hint(p) : 0u;
    cfg.gridDim = dim3(cs, p->num_kv_heads / args.hpc, p->num_seqs);
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
  }
  PA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map_k, map_v, args));
  return PA_OK;
}

template <int D>
static int enqueue_merge(const pa_params *p, cudaStream_t stream) {
  const uint32_t psize = (D == 64) ? 256u : 512u;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(p->num_heads, p->num_seqs, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  // programmatic dependent launch: the CTAs are scheduled while the attention kernel drains
  // and block in griddepcontrol.wait until that kernel has completed
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // Many (sequence, head) pairs: a warp per pair runs them in fewer waves than a CTA per pair.
  // Both kernels add in the same order and give the same bits (tested), so the choice is free.
  // Debugging knob: PA_MERGE_KERNEL=cta|warp forces one of them.
  static const int forced = [] {
    const char *e = std::getenv("PA_MERGE_KERNEL");
    return e == nullptr ? 0 : (e[0] == 'c' ? 1 : (e[0] == 'w' ? 2 : 0));
  }();
  const uint64_t pairs = static_cast<uint64_t>(p->num_seqs) * p->num_heads;
  // Measured on B200: from 2048 pairs on the warps win (4096 pairs of up to 6 partitions: 39.0
  // against 43.9 us per call; 2048 pairs of 8: 601 against 604); 1024 pairs of 64 partitions are
  // faster with a CTA each (174 against 181), whose threads fetch all 64 rows at once, so long
  // contexts need twice the pairs.
  uint32_t parts = p->max_num_partitions;
  if (context_hint(p) != 0u) parts = std::min(parts, divide_round_up(context_hint(p), psize));
  const bool many_pairs = pairs >= (parts > 32u ? 4096u : 2048u);
  if (forced == 2 || (forced == 0 && many_pairs)) {
    cfg.gridDim = dim3(static_cast<unsigned>((pairs + 3) / 4), 1, 1);
    PA_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partitions_warp_kernel<D>, static_cast<__half *>(p->out),
                                   static_cast<const __half *>(p->tmp_out),
                                   static_cast<const float *>(p->max_logits),
                                   static_cast<const float *>(p->exp_sums), p->context_lens, p->seq_indices,
                                   p->num_heads, static_cast<uint32_t>(pairs), p->max_num_partitions, psize,
                                   context_limit(p), p->block_table_offsets, log2_pow2(p->block_size)));
    return PA_OK;
  }
  PA_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partitions_kernel<D>, static_cast<__half *>(p->out),
                                 static_cast<const __half *>(p->tmp_out),
                                 static_cast<const float *>(p->max_logits),
                                 static_cast<const float *>(p->exp_sums), p->context_lens, p->seq_indices,
                                 p->num_heads, p->max_num_partitions, psize, context_limit(p),
                                 p->block_table_offsets, log2_pow2(p->block_size)));
  return PA_OK;
}

// Runs `first` and (if non-null) `second` on `stream`.  With us_out the call
// records events around each step, blocks, and reports device microseconds.
template <typename F1, typename F2>
int run_timed(cudaStream_t stream, float *us_out, F1 first, F2 second, bool has_second) {
  if (us_out == nullptr) {
    if (int rc = first()) return rc;
    if (has_second) return second();
    return PA_OK;
  }
  cudaEvent_t ev[3];
  for (auto &e : ev) PA_CUDA_TRY(cudaEventCreate(&e));
  int rc = PA_OK;
  cudaError_t err = cudaEventRecord(ev[0], stream);
  if (err == cudaSuccess) rc = first();
  if (rc == PA_OK && err == cudaSuccess) err = cudaEventRecord(ev[1], stream);
  if (rc == PA_OK && err == cudaSuccess && has_second) {
    rc = second();
    if (rc == PA_OK) err = cudaEventRecord(ev[2], stream);
  }
  if (rc == PA_OK && err == cudaSuccess) err = cudaEventSynchronize(has_second ? ev[2] : ev[1]);
  if (rc == PA_OK && err == cudaSuccess) {
    float ms = 0.f;
    err = cudaEventElapsedTime(&ms, ev[0], ev[1]);
    us_out[0] = ms * 1000.f;
    if (has_second && err == cudaSuccess) {
      err = cudaEventElapsedTime(&ms, ev[1], ev[2]);
      us_out[1] = ms * 1000.f;
    }
  }
  for (auto &e : ev) cudaEventDestroy(e);
  if (rc != PA_OK) return rc;
  if (err != cudaSuccess) return fail(PA_ERR_CUDA, "CUDA error while timing: %s", cudaGetErrorString(err));
  return PA_OK;
}

// Wide CTA (8 MMA warps, 8 KV heads per work item, one CTA per SM) or the default?  Wide for
// FP8 caches in the split variant when the KV heads come in eights and the launch has work
// for at least two rounds of one CTA per SM; everything else, small launches included, runs
// the default shape, whose work items are half as large.  Both shapes give the same bits.
template <int KV, int MODE>
bool wants_wide_cta(const pa_params *p) {
  if (KV == KV_F16 || MODE != MODE_SPLIT || p->num_kv_heads % 8u != 0u) return false;
  // debugging knob: PA_WIDE_CTA=0 never, 1 whenever the head count allows
  static const int knob = [] {
    const char *e = std::getenv("PA_WIDE_CTA");
    return e ? std::atoi(e) : -1;
  }();
  if (knob == 0) return false;
  if (knob == 1) return true;
  DeviceInfo dev{};
  if (get_device_info(&dev) != PA_OK) return false;
  // partitions per sequence: the scratch extent, cut down by the context-length hint if given
  uint32_t parts = p->max_num_partitions;
  if (context_hint(p) != 0u) {
    const uint32_t psize = (p->head_size == 64u) ? 256u : 512u;
    parts = std::min(parts, divide_round_up(context_hint(p), psize));
  }
  const uint64_t items = static_cast<uint64_t>(p->num_kv_heads / 8u) * parts * p->num_seqs;
  return items >= 2ull * static_cast<uint64_t>(dev.sm_count);
}

// Loop variant on a batch of many short sequences.  One cluster per (sequence, head group) then
// means thousands of CTAs that stream a few hundred KB each, and every one of them pays the
// start-up of a CTA (descriptor, barriers, first table entries, first copies) in the open.  The
// persistent kernel of the split variant runs the same items from its queue instead, a whole
// context per item, with the ring streaming across item boundaries; a CTA that holds a whole
// context holds the final result, so it writes `out` itself and there is still one launch and
// no scratch.  Taken when there are at least four units per SM and the longest possible item
// (the context-length hint times the bytes of a token of the CTA's heads) is at most 2 MiB, which
// bounds what one CTA can still be streaming after the queue has run dry (about 85 us).
// Measured on B200, 8 KV heads, group 4: 4096 sequences of 64..512 tokens 382 us instead of
// 1251 us (e5m2) and 732 instead of 1432 us (fp16); 1024 sequences of 512..2048 tokens (e5m2)
// 436 instead of 544 us (the wide CTA brings nothing here).  Longer or fewer items stay with
// the clusters: 128 sequences of 1024..8192 tokens 286 us instead of 203 us, 1024 log-normal
// lengths up to 32768 tokens 1777 instead of 1036 us.
inline bool wants_persistent_loop(const pa_params *p, uint32_t hpc, uint32_t bytes_per_element, int sm_count) {
  // debugging knob: PA_PERSISTENT_LOOP=0 never, 1 whenever the context-length hint is given
  static const int knob = [] {
    const char *e = std::getenv("PA_PERSISTENT_LOOP");
    return e ? std::atoi(e) : -1;
  }();
  const uint32_t hint = context_hint(p);
  if (knob == 0 || hint == 0u) return false;
  if (knob == 1) return true;
  const uint64_t units = static_cast<uint64_t>(p->num_seqs) * (p->num_kv_heads / hpc);
  const uint64_t longest_item = static_cast<uint64_t>(hint) * hpc * p->head_size * 2ull * bytes_per_element;
  return units >= 4ull * static_cast<uint64_t>(sm_count) && longest_item <= (2ull << 20);
}

// stage-size dispatch for one head size, KV type and mode (default CTA shape)
template <int D, int KV, int MODE>
static int dispatch_stage_tiles(const pa_params *p, cudaStream_t stream) {
  DeviceInfo dev{};
  if (int rc = get_device_info(&dev)) return rc;
  if constexpr (MODE == MODE_LOOP) {
    const uint32_t hpc_items = choose_heads_per_cta(p, /*wide=*/false, /*loop_mode=*/false, dev.sm_count);
    if (wants_persistent_loop(p, hpc_items, KV == KV_F16 ? 2u : 1u, dev.sm_count)) {
      const uint32_t tiles = choose_stage_tiles<D, KV>(p, hpc_items, 4u);
      if constexpr (max_stage_tiles<D, KV>() >= 4u) {
        if (tiles == 4u) return enqueue_attention<D, KV, MODE_SPLIT, 4, 4>(p, stream, hpc_items, true);
      }
      if constexpr (max_stage_tiles<D, KV>() >= 2u) {
        if (tiles >= 2u) return enqueue_attention<D, KV, MODE_SPLIT, 4, 2>(p, stream, hpc_items, true);
      }
      return enqueue_attention<D, KV, MODE_SPLIT, 4, 1>(p, stream, hpc_items, true);
    }
  }
  const uint32_t hpc = choose_heads_per_cta(p, /*wide=*/false, MODE == MODE_LOOP, dev.sm_count);
  const uint32_t tiles = choose_stage_tiles<D, KV>(p, hpc, 4u);
  if constexpr (max_stage_tiles<D, KV>() >= 4u) {
    if (tiles == 4u) return enqueue_attention<D, KV, MODE, 4, 4>(p, stream, hpc);
  }
  if constexpr (max_stage_tiles<D, KV>() >= 2u) {
    if (tiles >= 2u) return enqueue_attention<D, KV, MODE, 4, 2>(p, stream, hpc);
  }
  return enqueue_attention<D, KV, MODE, 4, 1>(p, stream, hpc);
}

// head-size dispatch for one KV type and mode
template <int KV, int MODE>
static int dispatch_head_size(const pa_params *p, cudaStream_t stream) {
  if constexpr (KV != KV_F16 && MODE == MODE_SPLIT) {
    if (wants_wide_cta<KV, MODE>(p)) {
      if (p->head_size == 128) return enqueue_attention<128, KV, MODE, 8>(p, stream, 8u);
      return enqueue_attention<64, KV, MODE, 8>(p, stream, 8u);
    }
  }
  if (p->head_size == 128) return dispatch_stage_tiles<128, KV, MODE>(p, stream);
  return dispatch_stage_tiles<64, KV, MODE>(p, stream);
}

static inline int dispatch_merge(const pa_params *p, cudaStream_t stream) {
  if (p->head_size == 128) return enqueue_merge<128>(p, stream);
  return enqueue_merge<64>(p, stream);
}

// A -DPA_TIMELINE build exports, per launcher, a reader of its unit's time-stamp table
// (`ctas` rows of 8 values; see g_timeline).  Synchronises the device.
#ifdef PA_TIMELINE
#define PA_TIMELINE_ACCESSOR(name)                                                                    \
  extern "C" PA_API int name(unsigned long long *dst, uint32_t ctas) {                                \
    if (dst == nullptr || ctas > ::pa::kTimelineCtas) return ::pa::fail(PA_ERR_BAD_ARG, "timeline: bad arguments"); \
    PA_CUDA_TRY(cudaDeviceSynchronize());                                                             \
    PA_CUDA_TRY(cudaMemcpyFromSymbol(dst, ::pa::g_timeline, sizeof(unsigned long long) * 8 * ctas));  \
    return PA_OK;                                                                                     \
  }
#else
#define PA_TIMELINE_ACCESSOR(name)
#endif

// A -DPA_DEBUG_BOUNDS build exports, per launcher, a reader of its unit's range-check report
// (8 values; see g_bounds_report) that also clears it.  Synchronises the device.
#ifdef PA_DEBUG_BOUNDS
#define PA_BOUNDS_ACCESSOR(name)                                                                      \
  extern "C" PA_API int name(uint32_t *dst) {                                                         \
    if (dst == nullptr) return ::pa::fail(PA_ERR_BAD_ARG, "bounds report: bad arguments");            \
    const unsigned int zeros[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};                                   \
    PA_CUDA_TRY(cudaDeviceSynchronize());                                                             \
    PA_CUDA_TRY(cudaMemcpyFromSymbol(dst, ::pa::g_bounds_report, sizeof(zeros)));                     \
    PA_CUDA_TRY(cudaMemcpyToSymbol(::pa::g_bounds_report, zeros, sizeof(zeros)));                     \
    return PA_OK;                                                                                     \
  }
#else
#define PA_BOUNDS_ACCESSOR(name)
#endif

// reads and clears this translation unit's copy of the device status word
static inline int read_and_clear_device_status(int *value) {
  int v = 0, zero = 0;
  PA_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_pa_device_status, sizeof(int)));
  if (v != 0) PA_CUDA_TRY(cudaMemcpyToSymbol(g_pa_device_status, &zero, sizeof(int)));
  *value = v;
  return PA_OK;
}

} // namespace pa
