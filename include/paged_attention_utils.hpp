// Helpers shared by host and device code of the B200 paged-attention library.
//
// Host part: the integer bookkeeping of the path (partition / block counts,
// element addresses), written once so that launchers, tests and kernels agree
// bit for bit.  Device part (only under nvcc): mbarrier / TMA / ldmatrix / mma
// wrappers, the swizzled shared-memory addressing that matches the TMA swizzle
// modes, FP8 -> fp16 converters and warp reductions.  These stand where the
// reference keeps tile loads, masks and work-group reductions
// (reference include/paged_attention_utils.hpp:28-960).
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define PA_HD __host__ __device__ __forceinline__
#define PA_DEV __device__ __forceinline__
#else
#define PA_HD inline
#endif

namespace pa {

// ---------------------------------------------------------------- bookkeeping
PA_HD uint32_t divide_round_up(uint32_t a, uint32_t b) { return (a + b - 1u) / b; }

// Number of partitions the reduce variant writes for one sequence
// (reference paged_attention_kernel_v2.hpp:679).
PA_HD uint32_t num_partitions_of(uint32_t context_len, uint32_t partition_size) {
  return divide_round_up(context_len, partition_size);
}

// Element offset of K/V[token t, kv head k, dim d] given the physical block id
// (reference paged_attention_kernel_loop.hpp:288-297).
PA_HD uint64_t kv_element_offset(uint32_t block_id, uint32_t row_in_block, uint32_t kv_head,
                                 uint32_t d, uint32_t block_size, uint32_t num_kv_heads,
                                 uint32_t head_size) {
  return ((static_cast<uint64_t>(block_id) * block_size + row_in_block) * num_kv_heads + kv_head) *
             head_size + d;
}

PA_HD bool is_pow2(uint32_t v) { return v != 0u && (v & (v - 1u)) == 0u; }
PA_HD uint32_t log2_pow2(uint32_t v) {
  uint32_t s = 0;
  while ((1u << s) < v) ++s;
  return s;
}

#if defined(__CUDACC__)
// ------------------------------------------------------------------- numerics
PA_DEV float neg_infinity() { return -__int_as_float(0x7f800000); }

PA_DEV float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

PA_DEV uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// max over the 8 lanes that share (lane & 3): lanes differ in bits 2..4
PA_DEV float quad_column_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
  return v;
}
PA_DEV float quad_column_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  v += __shfl_xor_sync(0xffffffffu, v, 8);
  v += __shfl_xor_sync(0xffffffffu, v, 16);
  return v;
}

// ------------------------------------------------------- shared memory access
PA_DEV uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a slab tile that a
// TMA tiled copy wrote with SWIZZLE_128B (128-byte rows) or SWIZZLE_64B
// (64-byte rows).  The tile base must be 1024-byte aligned.
template <uint32_t SLAB_BYTES>
PA_DEV uint32_t swizzled_offset(uint32_t row, uint32_t chunk) {
  if constexpr (SLAB_BYTES == 128u) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
  } else {
    return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4);
  }
}

PA_DEV void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
PA_DEV void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// transpose an 8x8 matrix of 16-bit elements held one register per lane
PA_DEV uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}

// D = A(16x16 fp16, row) * B(16x8 fp16, col) + D, fp32 accumulate
PA_DEV void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- FP8 -> fp16
// Both formats convert exactly: every finite e5m2 and e4m3 value is representable in fp16.
// A register holds four FP8 codes (bytes 0..3); results are fp16x2 registers with the first
// named byte in the low half.
PA_DEV uint32_t e4m3x2_to_half2(uint16_t pair) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(pair));
  return r;
}

// bytes (0,1) -> lo01, bytes (2,3) -> hi23   (K fragments: consecutive dims per lane)
template <int KV>
PA_DEV void fp8x4_to_half2x2(uint32_t v, uint32_t &lo01, uint32_t &hi23) {
  static_assert(KV == 1 || KV == 2, "FP8 formats only");
  if constexpr (KV == 1) {
    // e5m2 is the high byte of an fp16: move each code into the high byte of a half
    lo01 = __byte_perm(v, 0u, 0x1404);
    hi23 = __byte_perm(v, 0u, 0x3424);
  } else {
    lo01 = e4m3x2_to_half2(static_cast<uint16_t>(v & 0xffffu));
    hi23 = e4m3x2_to_half2(static_cast<uint16_t>(v >> 16));
  }
}

// bytes (0,2) -> even, bytes (1,3) -> odd   (V fragments after a 16-bit transposing load)
template <int KV>
PA_DEV void fp8x4_to_even_odd_half2(uint32_t v, uint32_t &even, uint32_t &odd) {
  static_assert(KV == 1 || KV == 2, "FP8 formats only");
  if constexpr (KV == 1) {
    even = __byte_perm(v, 0u, 0x2404);
    odd = v & 0xff00ff00u; // bytes 1 and 3 already sit in the high byte of each half
  } else {
    const uint32_t t = __byte_perm(v, 0u, 0x3120); // [b0, b2, b1, b3]
    even = e4m3x2_to_half2(static_cast<uint16_t>(t & 0xffffu));
    odd = e4m3x2_to_half2(static_cast<uint16_t>(t >> 16));
  }
}

// ------------------------------------------------------------------- mbarrier
PA_DEV void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
PA_DEV void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
PA_DEV void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
PA_DEV void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
PA_DEV bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0u;
}
PA_DEV uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Waits for a phase of `bar` with a time limit.  Returns false if the limit
// (about one second) passed or another warp of the CTA already gave up
// (*abort_flag != 0); the caller then leaves its loop instead of spinning on.
PA_DEV bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag,
                              uint64_t limit_ns = 1000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0x3ffu) == 0u) {
      if (*abort_flag != 0u) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1u;
        return false;
      }
    }
  }
  return true;
}

// Waits for a phase of `bar` for at most `limit_ns`, whatever the abort flag says: used after
// a give-up to let copies that are already in flight land before the CTA leaves.
PA_DEV bool mbar_wait_limited(uint64_t *bar, uint32_t parity, uint64_t limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 0xffu) == 0u && global_timer_ns() - t0 > limit_ns) return false;
  }
  return true;
}

// ------------------------------------------------------------------------ TMA
// L2 policy for data that is read exactly once (the KV stream): evict it first
PA_DEV uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// Tiled 3-D copy global -> this CTA's shared memory, completion on `bar`.
PA_DEV void tma_load_3d(uint32_t dst_smem, const void *tensor_map, uint64_t *bar, int32_t x,
                        int32_t y, int32_t z, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst_smem),
      "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "l"(l2_policy)
      : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, size
// a multiple of 16 bytes), completion on `bar`.
PA_DEV void bulk_load_1d(uint32_t dst_smem, const void *src, uint32_t bytes, uint64_t *bar, uint64_t l2_policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(l2_policy)
      : "memory");
}

PA_DEV void tma_prefetch_descriptor(const void *tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

// named barrier among `count` threads (id 1..15; 0 is __syncthreads)
PA_DEV void named_barrier_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
#endif // __CUDACC__

} // namespace pa
