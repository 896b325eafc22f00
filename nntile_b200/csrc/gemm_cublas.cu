// Batched GEMM of the unfused chain behind the C ABI.
//
// In the reference this operation IS a library call: nntile::kernel::cublas::gemm<T>
// (src/kernel/cublas.cc:35-164) converts its arguments and calls
// cublasGemmStridedBatchedEx on the handle of the calling worker.  It stays a
// library call here (the hand-written tensor-core code of this library is the
// fused pair); what this file adds is the C entry point with the reference's
// argument order, so that a C host can run the whole unfused chain through one
// library.  cuBLAS is looked up at run time in the process (the caller already
// holds a cublasHandle_t, so it is loaded), which keeps this library free of a
// link-time dependency on it.
#include <cublas_v2.h>
#include <dlfcn.h>

#include <mutex>

#include "common.cuh"

namespace nb200 {

// the C entry point of cuBLAS (the header also declares a C++ overload for 64-bit sizes)
typedef cublasStatus_t (*GemmStridedBatchedExFn)(cublasHandle_t, cublasOperation_t,
        cublasOperation_t, int, int, int, const void *, const void *, cudaDataType, int,
        long long, const void *, cudaDataType, int, long long, const void *, void *,
        cudaDataType, int, long long, int, cublasComputeType_t, cublasGemmAlgo_t);

struct CublasApi
{
    GemmStridedBatchedExFn gemm = nullptr;
};

static const CublasApi *cublas_api()
{
    static CublasApi api;
    static std::once_flag once;
    std::call_once(once, []() {
        // symbols of an already loaded cuBLAS first, then the usual sonames
        void *h = dlopen(nullptr, RTLD_NOW);
        void *g = h ? dlsym(h, "cublasGemmStridedBatchedEx") : nullptr;
        if(!g)
        {
            for(const char *name : {"libcublas.so.12", "libcublas.so.13", "libcublas.so"})
            {
                h = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
                if(h && (g = dlsym(h, "cublasGemmStridedBatchedEx")) != nullptr)
                {
                    break;
                }
            }
        }
        if(g)
        {
            api.gemm = reinterpret_cast<GemmStridedBatchedExFn>(g);
        }
    });
    return api.gemm ? &api : nullptr;
}

// Column-major C[m x n x batch] = alpha*op(A)*op(B) + beta*C with packed leading
// dimensions and one matrix after the other in memory: the (m, n, k, batch)
// contract of src/kernel/cublas.cc:52-83.  alpha and beta are applied in the fp32
// accumulator before the single rounding to the storage type.
static int gemm_run(void *handle, int transA, int transB, int64_t m, int64_t n, int64_t k,
        int64_t batch, float alpha, const void *A, const void *B, float beta, void *C,
        cudaDataType_t type)
{
    if(m < 0 || n < 0 || k < 0 || batch < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0 || batch == 0) return NNTILE_B200_OK;
    if(!handle || !A || !B || !C) return NNTILE_B200_E_BADARG;
    if(m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || batch > INT32_MAX)
    {
        return NNTILE_B200_E_SHAPE;
    }
    const CublasApi *api = cublas_api();
    if(!api) return NNTILE_B200_E_DEVICE;
    const int M = (int)m, N = (int)n, K = (int)k;
    const int ldA = transA ? K : M, ldB = transB ? N : K, ldC = M;
    const cublasStatus_t st = api->gemm(static_cast<cublasHandle_t>(handle),
            transA ? CUBLAS_OP_T : CUBLAS_OP_N, transB ? CUBLAS_OP_T : CUBLAS_OP_N, M, N, K,
            &alpha, A, type, ldA, (long long)m*k, B, type, ldB, (long long)n*k, &beta, C, type,
            ldC, (long long)m*n, (int)batch, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
    return st == CUBLAS_STATUS_SUCCESS ? NNTILE_B200_OK : NNTILE_B200_E_LAUNCH;
}

} // namespace nb200

extern "C" int nntile_b200_gemm_fp32(void *cublas_handle, int transA, int transB, int64_t m,
        int64_t n, int64_t k, int64_t batch, float alpha, const float *A, const float *B,
        float beta, float *C)
{
    return nb200::gemm_run(cublas_handle, transA, transB, m, n, k, batch, alpha, A, B, beta, C,
            CUDA_R_32F);
}

extern "C" int nntile_b200_gemm_bf16(void *cublas_handle, int transA, int transB, int64_t m,
        int64_t n, int64_t k, int64_t batch, float alpha, const void *A, const void *B,
        float beta, void *C)
{
    return nb200::gemm_run(cublas_handle, transA, transB, m, n, k, batch, alpha, A, B, beta, C,
            CUDA_R_16BF);
}
