// C-callable doors onto the reference's own CPU kernels.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit is compiled together with
// the reference's src/kernel/<op>/cpu.cc and src/kernel/cblas.cc, taken from
// the reference checkout where they lie (nothing is copied), into
// oracle/_ref/libnntile_ref_cpu.so by oracle/build.py.  It lets the test-suite
// pin the C restatement in sdpa_oracle.c against the real thing and lets the
// benchmark time the reference's CPU arithmetic.  The shipped library never
// sees it.
#include <cstdint>
#include <nntile/defs.h>
#include <nntile/base_types.hh>
#include <nntile/constants.hh>
#include <nntile/kernel/accumulate_attn_output/cpu.hh>
#include <nntile/kernel/add_fiber_inplace/cpu.hh>
#include <nntile/kernel/add_inplace/cpu.hh>
#include <nntile/kernel/add_slice_inplace/cpu.hh>
#include <nntile/kernel/cblas.hh>
#include <nntile/kernel/mask_scalar/cpu.hh>
#include <nntile/kernel/maxsumexp/cpu.hh>
#include <nntile/kernel/multiply_inplace/cpu.hh>
#include <nntile/kernel/rope/cpu.hh>
#include <nntile/kernel/softmax_inplace/cpu.hh>
#include <nntile/kernel/sumprod_slice/cpu.hh>
#include <nntile/kernel/transpose/cpu.hh>

namespace nk = nntile::kernel;
using nntile::fp32_t;
using nntile::bf16_t;
using nntile::bool_t;
using nntile::TransOp;
typedef std::int64_t i64;

#define REF_TYPED(suffix, TYPE) \
extern "C" void ref_mask_scalar_##suffix(i64 nrows, i64 ncols, \
        const void *mask, float val, void *data) \
{ \
    nk::mask_scalar::cpu<TYPE>(nrows, ncols, \
            static_cast<const bool_t *>(mask), val, static_cast<TYPE *>(data)); \
} \
extern "C" void ref_maxsumexp_##suffix(i64 m, i64 n, i64 k, \
        const void *src, void *dst) \
{ \
    nk::maxsumexp::cpu<TYPE>(m, n, k, static_cast<const TYPE *>(src), \
            static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_softmax_inplace_##suffix(i64 m, i64 n, i64 k, \
        const void *mse, float alpha, void *dst) \
{ \
    nk::softmax_inplace::cpu<TYPE>(m, n, k, static_cast<const TYPE *>(mse), \
            alpha, static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_sumprod_slice_##suffix(i64 m, i64 n, i64 k, \
        float alpha, const void *a, const void *b, float beta, void *dst) \
{ \
    nk::sumprod_slice::cpu<TYPE>(m, n, k, alpha, static_cast<const TYPE *>(a), \
            static_cast<const TYPE *>(b), beta, static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_add_slice_inplace_##suffix(i64 m, i64 n, i64 k, \
        float alpha, const void *src, float beta, void *dst) \
{ \
    nk::add_slice_inplace::cpu<TYPE>(m, n, k, alpha, \
            static_cast<const TYPE *>(src), beta, static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_multiply_inplace_##suffix(i64 nelems, float alpha, \
        const void *src, void *dst) \
{ \
    nk::multiply_inplace::cpu<TYPE>(nelems, alpha, \
            static_cast<const TYPE *>(src), static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_add_inplace_##suffix(i64 nelems, float alpha, \
        const void *src, float beta, void *dst) \
{ \
    nk::add_inplace::cpu<TYPE>(nelems, alpha, static_cast<const TYPE *>(src), \
            beta, static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_accumulate_attn_output_##suffix(i64 head, i64 seq, \
        i64 batch, const void *src_lse, const void *src_attn, \
        void *dst_lse, void *dst_attn) \
{ \
    nk::accumulate_attn_output::cpu<TYPE>(head, seq, batch, \
            static_cast<const fp32_t *>(src_lse), \
            static_cast<const TYPE *>(src_attn), \
            static_cast<fp32_t *>(dst_lse), static_cast<TYPE *>(dst_attn)); \
}

REF_TYPED(f32, fp32_t)
REF_TYPED(bf16, bf16_t)

// The layout / rotation / bias kernels around the SDPA layer.
#define REF_AROUND(suffix, TYPE) \
extern "C" void ref_transpose_##suffix(i64 m, i64 n, float alpha, \
        const void *src, void *dst) \
{ \
    nk::transpose::cpu<TYPE>(m, n, alpha, static_cast<const TYPE *>(src), \
            static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_rope_##suffix(i64 m, i64 n, const void *sn, \
        const void *cs, const void *src, void *dst) \
{ \
    nk::rope::cpu<TYPE>(m, n, static_cast<const TYPE *>(sn), \
            static_cast<const TYPE *>(cs), static_cast<const TYPE *>(src), \
            static_cast<TYPE *>(dst)); \
} \
extern "C" void ref_add_fiber_inplace_##suffix(i64 m, i64 n, i64 k, \
        i64 batch, float alpha, const void *src, float beta, void *dst) \
{ \
    nk::add_fiber_inplace::cpu<TYPE>(m, n, k, batch, alpha, \
            static_cast<const TYPE *>(src), beta, static_cast<TYPE *>(dst)); \
}

REF_AROUND(f32, fp32_t)
REF_AROUND(bf16, bf16_t)

// Batched column-major sgemm exactly as the reference's CPU codelet calls it.
extern "C" void ref_gemm_f32(int transA, int transB, i64 m, i64 n,
        i64 k, i64 batch, float alpha, const void *A, const void *B,
        float beta, void *C)
{
    nk::cblas::gemm<fp32_t>(
            TransOp(transA ? TransOp::Trans : TransOp::NoTrans),
            TransOp(transB ? TransOp::Trans : TransOp::NoTrans), m, n, k, batch,
            alpha, static_cast<const fp32_t *>(A), static_cast<const fp32_t *>(B),
            beta, static_cast<fp32_t *>(C));
}

// 1 when bf16 stores round to nearest even (the reference's CUDA build), 0 when
// they truncate (its CPU-only build).
extern "C" int ref_bf16_rounds_to_nearest(void)
{
#ifdef NNTILE_USE_CUDA
    return 1;
#else
    return 0;
#endif
}
