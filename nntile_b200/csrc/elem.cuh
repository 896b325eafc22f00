// Element type of the fused-attention sources (flash_*.cu, host_tensor.cu).
//
// The reference instantiates its fused pair for bf16_t and fp16_t
// (src/starpu/flash_sdpa_fwd_cudnn.cc:292-293).  Here the same sources are compiled
// twice: as they are for bfloat16, and with -DNB200_FP16 for IEEE half.  Everything
// that depends on the 16-bit format goes through this header: the type, the bit
// pattern of -inf, the pair conversions, the operand format of tcgen05.mma
// kind::f16, the data type of the TMA tensor maps, the suffix of the C entry points
// and an inline namespace that keeps the two builds' symbols apart.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace nb200 {

#ifdef NB200_FP16
#define NB200_ELEM_NS fp16abi
#define NB200_SFX(name) name##_fp16
using elem_t = __half;
constexpr uint32_t ELEM_NINF_BITS = 0xFC00u;            // -inf
constexpr uint32_t ELEM_MMA_FORMAT = 0u;                // kind::f16 operand format: f16
constexpr CUtensorMapDataType ELEM_TMAP_TYPE = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;

__device__ __forceinline__ float elem_to_f(elem_t x) { return __half2float(x); }
__device__ __forceinline__ elem_t f_to_elem(float x) { return __float2half_rn(x); }
// the two values of a 32-bit word (low half first)
__device__ __forceinline__ float elem_lo(uint32_t w)
{
    return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
}
__device__ __forceinline__ float elem_hi(uint32_t w)
{
    return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}
__device__ __forceinline__ uint32_t pack_elem2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
#else
#define NB200_ELEM_NS bf16abi
#define NB200_SFX(name) name##_bf16
using elem_t = __nv_bfloat16;
constexpr uint32_t ELEM_NINF_BITS = 0xFF80u;
constexpr uint32_t ELEM_MMA_FORMAT = 1u;                // kind::f16 operand format: bf16
constexpr CUtensorMapDataType ELEM_TMAP_TYPE = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;

__device__ __forceinline__ float elem_to_f(elem_t x) { return __bfloat162float(x); }
__device__ __forceinline__ elem_t f_to_elem(float x) { return __float2bfloat16_rn(x); }
__device__ __forceinline__ float elem_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float elem_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ uint32_t pack_elem2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
#endif

// value a stored element rounds to
__device__ __forceinline__ float elem_round(float x) { return elem_to_f(f_to_elem(x)); }

} // namespace nb200
