// Compile-time tiling policy of the B200 paged-attention kernels.
//
// Keeps the knob names callers of the reference can observe
// (reference include/paged_attention_policy_v2.hpp:5-100): partition_size is
// what sizes max_logits / exp_sums / tmp_out, stages / head_size_stride /
// partition_stride / max_partitions_per_sg are reported unchanged through
// pa_query_policy().  The CUDA geometry (ring of TMA stages, warps per CTA) is
// derived here for sm_100a and has no counterpart in the reference's
// work-group / sub-group numbers, which were written for Xe.
#pragma once

#include <cstdint>

namespace pa {

enum KvType : int { KV_F16 = 0, KV_E5M2 = 1, KV_E4M3 = 2 };

struct paged_attention_base_policy {
  static constexpr uint32_t stages = 3;            // reference base policy (:6)
  static constexpr uint32_t head_size_stride = 16; // reference base policy (:7); also the MMA k extent
};

// Shared geometry of the attention kernels for one (head size, KV element type).
template <uint32_t max_head_size_, int kv_type_>
struct kv_tile_geometry {
  static constexpr uint32_t max_head_size = max_head_size_;
  static constexpr uint32_t elt_bytes = (kv_type_ == KV_F16) ? 2u : 1u;
  static constexpr uint32_t row_bytes = max_head_size_ * elt_bytes;
  // A token row of one KV head is cut into slabs of at most 128 B, the span of
  // one TMA swizzle atom, so that ldmatrix reads of 8 rows x 16 B never collide.
  static constexpr uint32_t slab_bytes = row_bytes < 128u ? row_bytes : 128u;
  static constexpr uint32_t num_slabs = row_bytes / slab_bytes;
  static constexpr uint32_t slab_elems = slab_bytes / elt_bytes;
  static constexpr uint32_t chunks_per_slab = slab_bytes / 16u;
  static_assert(slab_bytes == 64u || slab_bytes == 128u, "slab must match a TMA swizzle span");
};

// One policy serves the loop and the reduce variants; query_group_size is a
// run-time value (1..8) because the group occupies the N=8 extent of the MMA.
//
// consumer_warps_ selects the CTA shape: 4 MMA warps and two CTAs per SM (default), or 8 MMA
// warps and one CTA per SM with a ring twice as large.  The wide shape lets a CTA take eight KV
// heads at once, which doubles the size of every TMA box; a warp does the same work on its
// head in both shapes, so the results are the same bit for bit.
//
// stage_tiles_ is the number of 16-token tiles of a KV head that one ring stage holds per MMA
// warp (1, 2 or 4).  KV blocks of 32 tokens and more can be fetched with one TMA box of up to
// 16 * stage_tiles_ rows per head, so a larger stage means larger copies (the memory system
// streams 8-16 KB copies best) where the rows are short (FP8, head size 64); the ring keeps its
// size and holds fewer, larger stages.  The order of operations on a token does not depend on it.
template <uint32_t max_head_size_, int kv_type_, uint32_t consumer_warps_ = 4, uint32_t stage_tiles_ = 1>
struct paged_attention_policy_v2 : paged_attention_base_policy {
  using geometry = kv_tile_geometry<max_head_size_, kv_type_>;
  static constexpr uint32_t max_head_size = max_head_size_;
  // reference: 512 for the primary template (:28), 256 for the head-64 one (:50)
  static constexpr uint32_t partition_size = max_head_size_ == 64 ? 256u : 512u;
  static constexpr uint32_t max_query_group_size = 8;
  // merge kernel knobs, reported only (reference :35-36,57-58)
  static constexpr uint32_t partition_stride = 8;
  static constexpr uint32_t max_partitions_per_sg = max_head_size_ == 64 ? 16u : 4u;

  // ---- sm_100a geometry ----
  static_assert(consumer_warps_ == 4 || consumer_warps_ == 8, "4 or 8 MMA warps");
  static constexpr uint32_t consumer_warps = consumer_warps_;       // MMA warps
  static_assert(stage_tiles_ == 1 || stage_tiles_ == 2 || stage_tiles_ == 4, "1, 2 or 4 tiles per warp and stage");
  static constexpr uint32_t stage_tiles = stage_tiles_;
  static constexpr uint32_t tokens_per_warp = 16;                   // M extent of m16n8k16
  static constexpr uint32_t rows_per_tile_step = consumer_warps * tokens_per_warp; // rows all warps consume at once: 64
  static constexpr uint32_t tokens_per_stage = rows_per_tile_step * stage_tiles_;  // rows of a stage: 64, 128 or 256
  static constexpr uint32_t threads_per_cta = (consumer_warps + 1) * 32; // + 1 TMA warp
  static constexpr uint32_t stage_bytes = 2u * tokens_per_stage * geometry::row_bytes; // K + V
  // Two CTAs per SM, each with a ring of about 96 KB (3 stages of 32 KB for fp16 / head 128,
  // 6 stages of 16 KB for FP8).  Measured on B200: three CTAs with 64 KB rings were no faster
  // for FP8 (the kernel is bound by HBM and by the depth of the ring, not by issue slots) and
  // left the loop variant with too shallow a ring per CTA.
  // Eight MMA warps: one CTA per SM with the whole 192 KB; measured 1-2 % faster than two
  // narrow CTAs on FP8 caches with 8 KV heads (16 KB boxes instead of 8 KB), 5 % slower
  // when its ring is cut to 128 KB and no faster with 224 KB; on fp16 caches (3 stages of 64 KB) it was
  // 2 % slower than the default shape and is not used there.
  static constexpr uint32_t ctas_per_sm = consumer_warps_ == 8 ? 1u : 2u;
  static constexpr uint32_t ring_budget = (consumer_warps_ == 8 ? 192u : 96u) * 1024u;
  static constexpr uint32_t ring_stages_raw = ring_budget / stage_bytes;
  static constexpr uint32_t ring_stages = ring_stages_raw > 8u ? 8u : ring_stages_raw;
  static_assert(ring_stages >= 2, "ring too shallow");
  static_assert(partition_size % tokens_per_stage == 0, "partition must be whole stages");
  static_assert(ring_stages_raw >= 2, "stage too large for the ring");
};

// The loop variant uses the same knobs (reference :64-100).
template <uint32_t max_head_size_, int kv_type_>
using paged_attention_policy_loop = paged_attention_policy_v2<max_head_size_, kv_type_>;

} // namespace pa
