// C++ shims that give the C ABI of nntile_b200.h the names and signatures of the
// reference's kernel layer, so that NNTile's codelets compile against it unchanged.
//
// Inside NNTile this header is included AFTER <nntile/base_types.hh>, which
// defines nntile::Index, nntile::Scalar, nntile::fp32_t, nntile::bf16_t and
// nntile::bool_t; stand-alone (NNTILE_B200_STANDALONE_TYPES) it declares
// layout-compatible stand-ins so that it can be compiled and tested on its own.
// The functions keep the reference's contract: noexcept, enqueue-only, stream
// first.  A negative status from the library cannot be thrown here either; it is
// kept in a thread-local that the caller may inspect (nntile_b200::last_status()).
//
// Replaced declarations (paths in the reference tree):
//   include/nntile/kernel/{maxsumexp,softmax_inplace,sumprod_slice,mask_scalar,
//   add_slice_inplace,multiply_inplace,add_inplace,accumulate_attn_output}/cuda.hh:25,
//   include/nntile/kernel/flash_sdpa_fwd_cudnn/cuda.hh:37-76 and
//   include/nntile/kernel/flash_sdpa_bwd_cudnn/cuda.hh:29-59 (execute_graph without
//   the cudnnHandle_t / graph pair),
//   include/nntile/kernel/cublas.hh (cublas::gemm<T>, src/kernel/cublas.cc:35-164).
#pragma once

#include <cstdint>
#include <type_traits>

#include "../nntile_b200.h"

#ifdef NNTILE_B200_STANDALONE_TYPES
namespace nntile
{
using Index = std::int64_t;
using Scalar = float;
struct fp32_t { float value; };
struct bf16_t { std::uint16_t value; };
struct fp16_t { std::uint16_t value; };
struct bool_t { bool value; };
// transposition flag of the reference's GEMM wrappers (include/nntile/constants.hh)
struct TransOp
{
    enum Value : int { NoTrans, Trans } value;
    constexpr explicit TransOp(Value v): value(v) {}
};
} // namespace nntile
typedef struct CUstream_st *cudaStream_t;
typedef struct cublasContext *cublasHandle_t;
#endif

namespace nntile_b200
{
inline int &last_status() noexcept
{
    static thread_local int status = 0;
    return status;
}

template<typename T>
inline constexpr bool is_fp32 = std::is_same_v<T, nntile::fp32_t>;
template<typename T>
inline constexpr bool is_bf16 = std::is_same_v<T, nntile::bf16_t>;
template<typename T>
inline constexpr bool is_fp16 = std::is_same_v<T, nntile::fp16_t>;
} // namespace nntile_b200

#define NNTILE_B200_DISPATCH(T, NAME, ...) \
    do { \
        static_assert(::nntile_b200::is_fp32<T> || ::nntile_b200::is_bf16<T>, \
                "nntile_b200 provides fp32 and bf16 kernels"); \
        if constexpr(::nntile_b200::is_fp32<T>) \
            ::nntile_b200::last_status() = nntile_b200_##NAME##_fp32(__VA_ARGS__); \
        else \
            ::nntile_b200::last_status() = nntile_b200_##NAME##_bf16(__VA_ARGS__); \
    } while(0)

namespace nntile::kernel
{

namespace maxsumexp
{
template<typename T>
void cuda(cudaStream_t stream, Index m, Index n, Index k, const T *src, T *maxsumexp) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, maxsumexp, stream, m, n, k, reinterpret_cast<const P *>(src),
            reinterpret_cast<P *>(maxsumexp));
}
} // namespace maxsumexp

namespace softmax_inplace
{
template<typename T>
void cuda(cudaStream_t stream, Index m, Index n, Index k, const T *maxsumexp, Scalar alpha,
        T *dst) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, softmax_inplace, stream, m, n, k,
            reinterpret_cast<const P *>(maxsumexp), alpha, reinterpret_cast<P *>(dst));
}
} // namespace softmax_inplace

namespace sumprod_slice
{
template<typename T>
void cuda(cudaStream_t stream, Index m, Index n, Index k, Scalar alpha, const T *src1,
        const T *src2, Scalar beta, T *dst) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, sumprod_slice, stream, m, n, k, alpha,
            reinterpret_cast<const P *>(src1), reinterpret_cast<const P *>(src2), beta,
            reinterpret_cast<P *>(dst));
}
} // namespace sumprod_slice

namespace mask_scalar
{
template<typename T>
void cuda(cudaStream_t stream, Index nrows, Index ncols, const bool_t *mask, Scalar val,
        T *data) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, mask_scalar, stream, nrows, ncols,
            reinterpret_cast<const std::uint8_t *>(mask), val, reinterpret_cast<P *>(data));
}
} // namespace mask_scalar

namespace add_slice_inplace
{
template<typename T>
void cuda(cudaStream_t stream, Index m, Index n, Index k, Scalar alpha, const T *src,
        Scalar beta, T *dst) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, add_slice_inplace, stream, m, n, k, alpha,
            reinterpret_cast<const P *>(src), beta, reinterpret_cast<P *>(dst));
}
} // namespace add_slice_inplace

namespace multiply_inplace
{
template<typename T>
void cuda(cudaStream_t stream, Index nelems, Scalar alpha, const T *src, T *dst) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, multiply_inplace, stream, nelems, alpha,
            reinterpret_cast<const P *>(src), reinterpret_cast<P *>(dst));
}
} // namespace multiply_inplace

namespace add_inplace
{
template<typename T>
void cuda(cudaStream_t stream, Index nelems, Scalar alpha, const T *src, Scalar beta,
        T *dst) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, add_inplace, stream, nelems, alpha, reinterpret_cast<const P *>(src),
            beta, reinterpret_cast<P *>(dst));
}
} // namespace add_inplace

namespace accumulate_attn_output
{
template<typename T>
void cuda(cudaStream_t stream, Index head, Index seq, Index batch, const fp32_t *src_lse,
        const T *src_attn, fp32_t *dst_lse, T *dst_attn) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, accumulate_attn_output, stream, head, seq, batch,
            reinterpret_cast<const float *>(src_lse), reinterpret_cast<const P *>(src_attn),
            reinterpret_cast<float *>(dst_lse), reinterpret_cast<P *>(dst_attn));
}
} // namespace accumulate_attn_output

// The library GEMM of the unfused chain, with the reference's argument order; the
// handle is the calling worker's cublasHandle_t, already bound to its stream.
namespace cublas
{
template<typename T>
void gemm(cublasHandle_t handle, TransOp transA, TransOp transB, Index m, Index n, Index k,
        Index batch, Scalar alpha, const T *A, const T *B, Scalar beta, T *C) noexcept
{
    using P = std::conditional_t<nntile_b200::is_fp32<T>, float, void>;
    NNTILE_B200_DISPATCH(T, gemm, handle, transA.value == TransOp::Trans ? 1 : 0,
            transB.value == TransOp::Trans ? 1 : 0, m, n, k, batch, alpha,
            reinterpret_cast<const P *>(A), reinterpret_cast<const P *>(B), beta,
            reinterpret_cast<P *>(C));
}
} // namespace cublas

// The fused pair: pointer order of the reference's execute_graph, stream instead of
// the cuDNN handle and graph.  bf16 and fp16 (fp32 is rejected by the reference too).
namespace flash_sdpa_fwd
{
template<typename T>
void cuda(cudaStream_t stream, Index seq, Index head, Index batch, const T *K, const T *Q,
        const T *mask, fp32_t *scratch_logsumexp, const T *V, T *scratch_A, fp32_t *logsumexp,
        T *A) noexcept
{
    static_assert(nntile_b200::is_bf16<T> || nntile_b200::is_fp16<T>,
            "the fused path takes bf16 or fp16");
    nntile_b200::last_status() = (nntile_b200::is_fp16<T> ? nntile_b200_flash_sdpa_fwd_fp16
            : nntile_b200_flash_sdpa_fwd_bf16)(stream, seq, head, batch, K, Q,
            mask, reinterpret_cast<float *>(scratch_logsumexp), V, scratch_A,
            reinterpret_cast<float *>(logsumexp), A);
}
} // namespace flash_sdpa_fwd

namespace flash_sdpa_bwd
{
template<typename T>
void cuda(cudaStream_t stream, Index seq, Index head, Index batch, const T *K, const T *Q,
        const T *V, const T *A, const T *dA, const T *mask, const fp32_t *logsumexp,
        T *scratch_dK, T *scratch_dQ, T *scratch_dV, T *dK, T *dQ, T *dV) noexcept
{
    static_assert(nntile_b200::is_bf16<T> || nntile_b200::is_fp16<T>,
            "the fused path takes bf16 or fp16");
    nntile_b200::last_status() = (nntile_b200::is_fp16<T> ? nntile_b200_flash_sdpa_bwd_fp16
            : nntile_b200_flash_sdpa_bwd_bf16)(stream, seq, head, batch, K, Q,
            V, A, dA, mask, reinterpret_cast<const float *>(logsumexp), scratch_dK, scratch_dQ,
            scratch_dV, dK, dQ, dV);
}
} // namespace flash_sdpa_bwd

} // namespace nntile::kernel
