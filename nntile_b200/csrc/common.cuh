// Shared helpers of the nntile_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <atomic>

#include "../../include/nntile_b200.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "nntile_b200 is written for sm_100a only"
#endif

namespace nb200 {

using bf16 = __nv_bfloat16;
typedef int64_t Index;

// Storage <-> compute conversions.  bf16 stores round to nearest even, the rule
// the reference's CUDA build uses (include/nntile/base_types.hh:559-563).
__device__ __forceinline__ float ld(const float &x) { return x; }
__device__ __forceinline__ float ld(const bf16 &x) { return __bfloat162float(x); }
__device__ __forceinline__ void st(float &d, float v) { d = v; }
__device__ __forceinline__ void st(bf16 &d, float v) { d = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
    {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for(int o = 16; o > 0; o >>= 1)
    {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    return v;
}

inline cudaStream_t as_stream(nntile_b200_stream_t s)
{
    return static_cast<cudaStream_t>(s);
}

// Process-wide count of kernels this library has launched (defined in
// vanilla_ops.cu, read through nntile_b200_launch_count()).
extern std::atomic<unsigned long long> g_kernel_launches;

// Status of the `launched` kernel launches issued since the last check.
inline int launch_status(int launched = 1)
{
    g_kernel_launches.fetch_add((unsigned long long)launched, std::memory_order_relaxed);
    return cudaGetLastError() == cudaSuccess ? NNTILE_B200_OK : NNTILE_B200_E_LAUNCH;
}

inline bool aligned16(const void *p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// Number of blocks for a grid-stride elementwise kernel: enough to fill the
// 148 SMs a few times over, never more than the work needs.
inline unsigned grid_for(Index nelems, int threads, int per_thread = 4)
{
    Index want = (nelems + (Index)threads*per_thread - 1)/((Index)threads*per_thread);
    const Index cap = 148*16;
    if(want > cap) want = cap;
    if(want < 1) want = 1;
    return (unsigned)want;
}

} // namespace nb200
