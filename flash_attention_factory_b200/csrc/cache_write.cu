// pa_reshape_and_cache: appends new K/V tokens to the paged cache, quantising to FP8 on the way.
//
// The step that precedes the attention path in a decode loop.  The reference has no such
// kernel: its tests build caches on the host with torch casts (test_paged_fp8cache.py:180-203)
// in the layout the attention kernels read, [num_blocks, block_size, num_kv_heads, head_size]
// (paged_attention_kernel_loop.hpp:50-51).  This kernel defines the same contract on the
// device: value stored = round-to-nearest-even(x / scale) in e5m2 or e4m3 (saturating to
// the largest finite code), or x itself for an fp16 cache.  The scale is fp8_scale, or the
// entry of the token's KV head (and block) in the per-head / per-block scale arrays that the
// attention entry points read back under the same names.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cmath>

#include "launch_common.cuh"

namespace pa {

// 8 fp16 values (one 16-byte load) -> 8 cache elements
// `exact_rcp` != 0 means 1 / scale is a power of two, so multiplying by it is exact and
// equals the division bit for bit; otherwise an IEEE division keeps the torch arithmetic.
template <int KV>
__device__ __forceinline__ void store_converted(void *dst_row, uint32_t elem, uint4 v, float scale,
                                                float exact_rcp) {
  if constexpr (KV == KV_F16) {
    *reinterpret_cast<uint4 *>(static_cast<__half *>(dst_row) + elem) = v;
  } else {
    const __half2 *h = reinterpret_cast<const __half2 *>(&v);
    uint32_t packed[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      // IEEE division in fp32, then one rounding to FP8: the arithmetic of
      // (x.float() / scale).to(float8) for every value inside the format's range
      float2 a = __half22float2(h[2 * i]);
      float2 b = __half22float2(h[2 * i + 1]);
      constexpr __nv_fp8_interpretation_t fmt = (KV == KV_E5M2) ? __NV_E5M2 : __NV_E4M3;
      if (exact_rcp != 0.f) {
        a.x *= exact_rcp; a.y *= exact_rcp; b.x *= exact_rcp; b.y *= exact_rcp;
      } else {
        a.x = __fdiv_rn(a.x, scale); a.y = __fdiv_rn(a.y, scale);
        b.x = __fdiv_rn(b.x, scale); b.y = __fdiv_rn(b.y, scale);
      }
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(a, __NV_SATFINITE, fmt);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(b, __NV_SATFINITE, fmt);
      packed[i] = lo | (hi << 16);
    }
    *reinterpret_cast<uint2 *>(static_cast<uint8_t *>(dst_row) + elem) = make_uint2(packed[0], packed[1]);
  }
}

// Where the scale of an element comes from.
enum ScaleKind : int { SCALE_SCALAR = 0, SCALE_PER_HEAD = 1, SCALE_PER_BLOCK = 2 };

struct ScaleArrays {
  const float *k; // [num_kv_heads] or [num_blocks, num_kv_heads]; unused for SCALE_SCALAR
  const float *v;
  uint32_t head_size;
  uint32_t num_kv_heads;
  uint32_t block_size;
};

// One CTA per new token; a thread moves 8 elements of K and 8 of V per step.
template <int KV, bool CHAINED, int SCALES>
__global__ void __launch_bounds__(128)
reshape_and_cache_kernel(const __half *__restrict__ key, const __half *__restrict__ value,
                         void *__restrict__ key_cache, void *__restrict__ value_cache,
                         const int64_t *__restrict__ slot_mapping, uint32_t row_elems, uint64_t num_slots,
                         float scale, float exact_rcp, ScaleArrays arrays) {
  // CHAINED (decode-sized appends): programmatic dependent launch.  The attention kernel that
  // follows in a decode step may be scheduled while this grid runs (it waits for this grid's
  // completion before its first read), and this grid reads nothing before its own predecessor
  // in the stream has completed.  Prefill-sized appends, tens of thousands of CTAs of about a
  // microsecond each, run the plain form: the two instructions per CTA measured 6 % slower on
  // the FP8 caches there.
  if constexpr (CHAINED) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  const uint32_t token = blockIdx.x;
  const int64_t slot = slot_mapping[token];
  if (slot < 0 || static_cast<uint64_t>(slot) >= num_slots) return; // padding token / out of range
  constexpr uint32_t ELT = (KV == KV_F16) ? 2u : 1u;
  const __half *ksrc = key + static_cast<size_t>(token) * row_elems;
  const __half *vsrc = value + static_cast<size_t>(token) * row_elems;
  uint8_t *kdst = static_cast<uint8_t *>(key_cache) + static_cast<size_t>(slot) * row_elems * ELT;
  uint8_t *vdst = static_cast<uint8_t *>(value_cache) + static_cast<size_t>(slot) * row_elems * ELT;
  for (uint32_t e = threadIdx.x * 8; e < row_elems; e += blockDim.x * 8) {
    const uint4 kv = __ldg(reinterpret_cast<const uint4 *>(ksrc + e));
    const uint4 vv = __ldg(reinterpret_cast<const uint4 *>(vsrc + e));
    if constexpr (SCALES == SCALE_SCALAR || KV == KV_F16) {
      store_converted<KV>(kdst, e, kv, scale, exact_rcp);
      store_converted<KV>(vdst, e, vv, scale, exact_rcp);
    } else {
      // 8 elements never straddle a head (head_size is a multiple of 8); always the IEEE division
      const uint32_t head = e / arrays.head_size;
      const size_t si = (SCALES == SCALE_PER_HEAD)
                            ? head
                            : static_cast<size_t>(slot / arrays.block_size) * arrays.num_kv_heads + head;
      store_converted<KV>(kdst, e, kv, __ldg(arrays.k + si), 0.f);
      store_converted<KV>(vdst, e, vv, __ldg(arrays.v + si), 0.f);
    }
  }
}

} // namespace pa

extern "C" PA_API int pa_reshape_and_cache(const pa_cache_write_params *p, void *stream) {
  using namespace pa;
  if (p == nullptr) return fail(PA_ERR_BAD_ARG, "params is null");
  if (p->kv_dtype != PA_KV_F16 && p->kv_dtype != PA_KV_FP8_E5M2 && p->kv_dtype != PA_KV_FP8_E4M3)
    return fail(PA_ERR_BAD_ARG, "unknown kv_dtype %d", p->kv_dtype);
  if (p->num_tokens == 0) return PA_OK;
  if (!p->key || !p->value || !p->key_cache || !p->value_cache || !p->slot_mapping)
    return fail(PA_ERR_BAD_ARG, "a required pointer is null");
  const uint64_t row_elems = static_cast<uint64_t>(p->num_kv_heads) * p->head_size;
  if (row_elems == 0 || row_elems % 8 != 0 || row_elems > (1u << 20))
    return fail(PA_ERR_BAD_ARG, "num_kv_heads * head_size must be a positive multiple of 8");
  if (p->block_size == 0 || p->num_blocks == 0) return fail(PA_ERR_BAD_ARG, "empty cache");
  const bool per_head = p->k_scale_per_head != nullptr || p->v_scale_per_head != nullptr;
  const bool per_block = p->k_scale_per_block != nullptr || p->v_scale_per_block != nullptr;
  if (per_head && (p->k_scale_per_head == nullptr || p->v_scale_per_head == nullptr))
    return fail(PA_ERR_BAD_ARG, "k_scale_per_head and v_scale_per_head must be given together");
  if (per_block && (p->k_scale_per_block == nullptr || p->v_scale_per_block == nullptr))
    return fail(PA_ERR_BAD_ARG, "k_scale_per_block and v_scale_per_block must be given together");
  if (per_head && per_block) return fail(PA_ERR_BAD_ARG, "per-head and per-block scales exclude each other");
  if ((per_head || per_block) && p->kv_dtype == PA_KV_F16)
    return fail(PA_ERR_BAD_ARG, "scale arrays need an FP8 cache");
  if ((per_head || per_block) && (p->head_size == 0 || p->head_size % 8 != 0))
    return fail(PA_ERR_BAD_ARG, "scale arrays need a head_size that is a multiple of 8");
  if (p->kv_dtype != PA_KV_F16 && !per_head && !per_block && !(p->fp8_scale > 0.f))
    return fail(PA_ERR_BAD_ARG, "fp8_scale must be positive and finite");
  if (!aligned16(p->key) || !aligned16(p->value) || !aligned16(p->key_cache) || !aligned16(p->value_cache))
    return fail(PA_ERR_BAD_ARG, "key / value / caches must be 16-byte aligned");
  const uint64_t num_slots = p->num_blocks * p->block_size;
  // a power-of-two scale (1.0 included) has an exact reciprocal: no division needed
  float exact_rcp = 0.f;
  {
    int exponent = 0;
    if (p->kv_dtype != PA_KV_F16 && !per_head && !per_block && std::frexp(p->fp8_scale, &exponent) == 0.5f &&
        exponent > -100 && exponent < 100)
      exact_rcp = 1.f / p->fp8_scale;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t re = static_cast<uint32_t>(row_elems);
  const __half *k = static_cast<const __half *>(p->key);
  const __half *v = static_cast<const __half *>(p->value);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[1];
  cfg.gridDim = dim3(p->num_tokens, 1, 1);
  cfg.blockDim = dim3(128, 1, 1);
  cfg.stream = s;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const bool chained = p->num_tokens <= 4096u;
  cfg.numAttrs = chained ? 1 : 0;
  const float scale = (p->kv_dtype == PA_KV_F16) ? 1.f : p->fp8_scale;
  const float rcp = (p->kv_dtype == PA_KV_F16) ? 1.f : exact_rcp;
  ScaleArrays arrays{};
  arrays.k = per_head ? p->k_scale_per_head : p->k_scale_per_block;
  arrays.v = per_head ? p->v_scale_per_head : p->v_scale_per_block;
  arrays.head_size = p->head_size;
  arrays.num_kv_heads = p->num_kv_heads;
  arrays.block_size = p->block_size;
  using kernel_fn = void (*)(const __half *, const __half *, void *, void *, const int64_t *, uint32_t, uint64_t,
                             float, float, ScaleArrays);
  // [cache type][chained][scale kind]; an fp16 cache has no scales
  static const kernel_fn table[3][2][3] = {
      {{reshape_and_cache_kernel<KV_F16, false, SCALE_SCALAR>, nullptr, nullptr},
       {reshape_and_cache_kernel<KV_F16, true, SCALE_SCALAR>, nullptr, nullptr}},
      {{reshape_and_cache_kernel<KV_E5M2, false, SCALE_SCALAR>, reshape_and_cache_kernel<KV_E5M2, false, SCALE_PER_HEAD>,
        reshape_and_cache_kernel<KV_E5M2, false, SCALE_PER_BLOCK>},
       {reshape_and_cache_kernel<KV_E5M2, true, SCALE_SCALAR>, reshape_and_cache_kernel<KV_E5M2, true, SCALE_PER_HEAD>,
        reshape_and_cache_kernel<KV_E5M2, true, SCALE_PER_BLOCK>}},
      {{reshape_and_cache_kernel<KV_E4M3, false, SCALE_SCALAR>, reshape_and_cache_kernel<KV_E4M3, false, SCALE_PER_HEAD>,
        reshape_and_cache_kernel<KV_E4M3, false, SCALE_PER_BLOCK>},
       {reshape_and_cache_kernel<KV_E4M3, true, SCALE_SCALAR>, reshape_and_cache_kernel<KV_E4M3, true, SCALE_PER_HEAD>,
        reshape_and_cache_kernel<KV_E4M3, true, SCALE_PER_BLOCK>}}};
  const int type_index = (p->kv_dtype == PA_KV_F16) ? 0 : (p->kv_dtype == PA_KV_FP8_E5M2) ? 1 : 2;
  const int scale_kind = per_head ? SCALE_PER_HEAD : per_block ? SCALE_PER_BLOCK : SCALE_SCALAR;
  const kernel_fn kernel = table[type_index][chained ? 1 : 0][scale_kind];
  PA_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, k, v, p->key_cache, p->value_cache, p->slot_mapping, re,
                                 num_slots, scale, rcp, arrays));
  PA_CUDA_TRY(cudaGetLastError());
  return PA_OK;
}
