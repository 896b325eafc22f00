// The unfused ("vanilla") softmax chain of NNTile's attention layer as sm_100a
// kernels behind the C ABI.  These ops are HBM-bound: every kernel touches each
// input element once with coalesced accesses and sizes its grid from the 148 SMs.
//
// Reference semantics followed (paths relative to the reference tree):
//   mask_scalar            src/kernel/mask_scalar/{cpu.cc:22-49,cuda.cu:21-110}
//   maxsumexp              src/kernel/maxsumexp/{cpu.cc:22-128,cuda.cu:22-323}
//   softmax_inplace        src/kernel/softmax_inplace/{cpu.cc:22-70,cuda.cu:22-181}
//   sumprod_slice          src/kernel/sumprod_slice/{cpu.cc:21-81,cuda.cu:22-214}
//   add_slice_inplace      src/kernel/add_slice_inplace/{cpu.cc:22-70,cuda.cu:22-158}
//   multiply_inplace       src/kernel/multiply_inplace/{cpu.cc:22-40,cuda.cu:21-76}
//   add_inplace            src/kernel/add_inplace/cpu.cc:22-50
//   accumulate_attn_output src/kernel/accumulate_attn_output/cuda.cu:28-135
#include "common.cuh"

namespace nb200 {

std::atomic<unsigned long long> g_kernel_launches{0};

// ------------------------------------------------------- 16-byte vector access
// The hot shapes of the chain (m == 1: fibres are contiguous; whole tensors for the
// elementwise ops) are walked in 16-byte pieces - 8 bf16 or 4 fp32 values per
// thread and access - whenever the fibre length and the pointers allow it; the
// scalar kernels below cover everything else.
template<typename T> struct Vec;
template<> struct Vec<float> { static constexpr int N = 4; };
template<> struct Vec<bf16> { static constexpr int N = 8; };

__device__ __forceinline__ void vload(const float *p, float (&v)[4])
{
    const float4 x = *reinterpret_cast<const float4 *>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}

__device__ __forceinline__ void vload(const bf16 *p, float (&v)[8])
{
    const uint4 x = *reinterpret_cast<const uint4 *>(p);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for(int e = 0; e < 4; ++e)
    {
        v[2*e] = __uint_as_float(w[e] << 16);
        v[2*e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
    }
}

__device__ __forceinline__ void vstore(float *p, const float (&v)[4])
{
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ void vstore(bf16 *p, const float (&v)[8])
{
    uint32_t w[4];
#pragma unroll
    for(int e = 0; e < 4; ++e)
    {
        w[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[2*e]))
                | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v[2*e + 1])) << 16);
    }
    *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

// exp for the vector kernels: the accurate expf for fp32 storage (the chain's 1e-5
// bar), the two-instruction ex2-based form for bf16 storage, whose own rounding
// (2^-9) is four orders of magnitude coarser than that form's error.
__device__ __forceinline__ float exp_for(const float *, float x) { return expf(x); }
__device__ __forceinline__ float exp_for(const bf16 *, float x) { return __expf(x); }

// exp(x - top) with `top` finite and fixed over many x: the bf16 form folds the
// subtraction into the multiply by log2(e) (one fused multiply-add and one ex2)
struct ExpShift
{
    float top, ntop_l2;
    __device__ __forceinline__ explicit ExpShift(float t) : top(t), ntop_l2(-t*1.4426950408889634f) {}
    __device__ __forceinline__ float operator()(const float *, float x) const { return expf(x - top); }
    __device__ __forceinline__ float operator()(const bf16 *, float x) const
    {
        float y;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fmaf(x, 1.4426950408889634f, ntop_l2)));
        return y;
    }
};

template<typename T>
inline bool vec_ok(Index fibre_len, const void *a, const void *b = nullptr, const void *c = nullptr)
{
    return fibre_len % Vec<T>::N == 0 && aligned16(a) && (!b || aligned16(b)) && (!c || aligned16(c));
}

// Lanes that share one fibre of `k` elements: the smallest power of two that gives
// every lane at least one 16-byte piece, at most a warp.
template<typename T>
inline int lanes_per_fibre(Index k)
{
    const Index pieces = k/Vec<T>::N;
    int l = 1;
    while(l < 32 && l < pieces) l <<= 1;
    return l;
}

// Blocks of 256 threads for `n` fibres at `lpf` lanes each: enough to fill the 148
// SMs eight blocks deep, never more than the fibres need.
inline unsigned fibre_grid(Index n, int lpf)
{
    const Index per_block = 256/lpf;
    Index blocks = (n + per_block - 1)/per_block;
    if(blocks > 148*8) blocks = 148*8;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

// ---------------------------------------------------------------- mask_scalar
// Vector form: grid.y walks the columns, threads walk the 16-byte pieces of a
// column.  A piece whose mask bytes are all "keep" is not touched at all, one whose
// bytes are all "drop" is written without being read.
template<typename T>
__global__ void __launch_bounds__(256)
mask_scalar_vec_kernel(Index nrows, Index ncols, const uint8_t *__restrict__ mask, float val,
        T *__restrict__ data)
{
    constexpr int N = Vec<T>::N;
    const Index pieces = nrows/N;
    for(Index col = blockIdx.y; col < ncols; col += gridDim.y)
    {
        T *column = data + col*nrows;
        for(Index v = (Index)blockIdx.x*blockDim.x + threadIdx.x; v < pieces;
                v += (Index)gridDim.x*blockDim.x)
        {
            uint8_t keep[N];
            if(N == 8)
            {
                const uint2 m = *reinterpret_cast<const uint2 *>(mask + v*N);
#pragma unroll
                for(int e = 0; e < 4; ++e)
                {
                    keep[e] = (uint8_t)(m.x >> (8*e));
                    keep[4 + e] = (uint8_t)(m.y >> (8*e));
                }
            }
            else
            {
                const uint32_t m = *reinterpret_cast<const uint32_t *>(mask + v*N);
#pragma unroll
                for(int e = 0; e < N; ++e)
                {
                    keep[e] = (uint8_t)(m >> (8*e));
                }
            }
            bool all_keep = true, all_drop = true;
#pragma unroll
            for(int e = 0; e < N; ++e)
            {
                all_keep &= keep[e] != 0;
                all_drop &= keep[e] == 0;
            }
            if(all_keep)
            {
                continue;
            }
            float x[N];
            if(all_drop)
            {
#pragma unroll
                for(int e = 0; e < N; ++e) x[e] = val;
            }
            else
            {
                vload(column + v*N, x);
#pragma unroll
                for(int e = 0; e < N; ++e) x[e] = keep[e] ? x[e] : val;
            }
            vstore(column + v*N, x);
        }
    }
}

template<typename T>
__global__ void mask_scalar_kernel(Index nrows, Index total, const uint8_t *mask,
        float val, T *data)
{
    const Index stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        if(!mask[x % nrows])
        {
            st(data[x], val);
        }
    }
}

// ------------------------------------------------------------------ maxsumexp
// A partial result is the pair (top, sum) with sum = sum exp(x - top) over the
// finite entries seen so far; (-inf, 0) is the empty pair.
struct MaxSum
{
    float top, sum;
};

__device__ __forceinline__ MaxSum ms_push(MaxSum a, float v)
{
    if(isinf(v))
    {
        return a;
    }
    if(v > a.top)
    {
        a.sum = a.sum*expf(a.top - v) + 1.0f;   // exp(-inf)=0 covers the empty pair
        a.top = v;
    }
    else
    {
        a.sum += expf(v - a.top);
    }
    return a;
}

__device__ __forceinline__ MaxSum ms_join(MaxSum a, MaxSum b)
{
    if(b.sum == 0.0f)
    {
        return a;
    }
    if(a.sum == 0.0f)
    {
        return b;
    }
    MaxSum r;
    r.top = fmaxf(a.top, b.top);
    r.sum = a.sum*expf(a.top - r.top) + b.sum*expf(b.top - r.top);
    return r;
}

template<typename T>
__device__ __forceinline__ void ms_store(MaxSum cur, T *out)
{
    // Nothing finite seen: leave the destination as it is.
    if(cur.sum == 0.0f)
    {
        return;
    }
    const float old_sum = ld(out[1]);
    if(old_sum != 0.0f)
    {
        MaxSum old = {ld(out[0]), old_sum};
        cur = ms_join(old, cur);
    }
    st(out[0], cur.top);
    st(out[1], cur.sum);
}

// m == 1: fibres are contiguous; one warp per fibre, lanes stride over k.
template<typename T>
__global__ void maxsumexp_m1_kernel(Index n, Index k, const T *src, T *dst)
{
    const int lane = threadIdx.x & 31;
    const Index warps = ((Index)gridDim.x*blockDim.x) >> 5;
    for(Index j = (((Index)blockIdx.x*blockDim.x + threadIdx.x) >> 5); j < n; j += warps)
    {
        const T *fib = src + j*k;
        // A leading +inf makes the reference give up on the fibre.
        const bool poisoned = isinf(ld(fib[0])) && ld(fib[0]) > 0.0f;
        MaxSum acc = {-CUDART_INF_F, 0.0f};
        for(Index l = lane; l < k; l += 32)
        {
            acc = ms_push(acc, ld(fib[l]));
        }
#pragma unroll
        for(int o = 16; o > 0; o >>= 1)
        {
            MaxSum other;
            other.top = __shfl_xor_sync(0xffffffffu, acc.top, o);
            other.sum = __shfl_xor_sync(0xffffffffu, acc.sum, o);
            acc = ms_join(acc, other);
        }
        if(lane == 0 && !poisoned)
        {
            ms_store(acc, dst + 2*j);
        }
    }
}

// m == 1, vector form: `lpf` lanes share a fibre and walk it in 16-byte pieces, four
// pieces (four independent loads) per pass.  Per pass: the maximum of the finite
// values, one rescale of the running sum when the maximum grows, then one
// exponential per value of every piece that has a finite one (exp(-inf) = 0 drops
// masked values; a fully masked piece costs no exponentials).
template<typename T>
__global__ void __launch_bounds__(256)
maxsumexp_m1_vec_kernel(Index n, Index k, int lpf, const T *__restrict__ src, T *dst)
{
    constexpr int N = Vec<T>::N;
    constexpr int U = 4;
    const int sub = threadIdx.x & (lpf - 1);
    const Index groups = ((Index)gridDim.x*blockDim.x)/lpf;
    const Index step = (Index)lpf*N;
    for(Index j = ((Index)blockIdx.x*blockDim.x + threadIdx.x)/lpf; j < n; j += groups)
    {
        const T *fib = src + j*k;
        MaxSum acc = {-CUDART_INF_F, 0.0f};
        bool poisoned = false;
        for(Index l0 = (Index)sub*N; l0 < k; l0 += step*U)
        {
            float x[U][N];
            float ptop[U];
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                const Index l = l0 + (Index)u*step;
                if(l < k)
                {
                    vload(fib + l, x[u]);
                }
                else
                {
#pragma unroll
                    for(int e = 0; e < N; ++e) x[u][e] = -CUDART_INF_F;
                }
            }
            if(l0 == 0)
            {
                // a leading +inf makes the reference give up on the fibre
                poisoned = isinf(x[0][0]) && x[0][0] > 0.0f;
            }
            float top = -CUDART_INF_F;
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                ptop[u] = x[u][0];
#pragma unroll
                for(int e = 1; e < N; ++e)
                {
                    ptop[u] = fmaxf(ptop[u], x[u][e]);
                }
                if(ptop[u] == CUDART_INF_F)
                {
                    // rare: +inf is skipped like -inf
                    ptop[u] = -CUDART_INF_F;
#pragma unroll
                    for(int e = 0; e < N; ++e)
                    {
                        x[u][e] = isinf(x[u][e]) ? -CUDART_INF_F : x[u][e];
                        ptop[u] = fmaxf(ptop[u], x[u][e]);
                    }
                }
                top = fmaxf(top, ptop[u]);
            }
            if(top == -CUDART_INF_F)
            {
                continue;
            }
            if(top > acc.top)
            {
                acc.sum *= exp_for(fib, acc.top - top);        // exp(-inf) = 0: empty pair
                acc.top = top;
            }
            const ExpShift shifted(acc.top);
#pragma unroll
            for(int u = 0; u < U; ++u)
            {
                if(ptop[u] == -CUDART_INF_F)
                {
                    continue;
                }
                float part = 0.0f;
#pragma unroll
                for(int e = 0; e < N; ++e)
                {
                    part += shifted(fib, x[u][e]);              // exp(-inf) = 0 drops masked values
                }
                acc.sum += part;
            }
        }
        for(int o = lpf >> 1; o > 0; o >>= 1)
        {
            MaxSum other;
            other.top = __shfl_xor_sync(0xffffffffu, acc.top, o);
            other.sum = __shfl_xor_sync(0xffffffffu, acc.sum, o);
            acc = ms_join(acc, other);
        }
        poisoned = __shfl_sync(0xffffffffu, (int)poisoned, (threadIdx.x & 31) & ~(lpf - 1)) != 0;
        if(sub == 0 && !poisoned)
        {
            ms_store(acc, dst + 2*j);
        }
    }
}

// General m: one thread per (i, j); neighbouring threads read neighbouring i.
template<typename T>
__global__ void maxsumexp_kernel(Index m, Index n, Index k, const T *src, T *dst)
{
    const Index total = m*n, stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        const Index i = x % m, j = x/m;
        const T *fib = src + j*m*k + i;
        const float first = ld(fib[0]);
        if(isinf(first) && first > 0.0f)
        {
            continue;
        }
        MaxSum acc = {-CUDART_INF_F, 0.0f};
        for(Index l = 0; l < k; ++l)
        {
            acc = ms_push(acc, ld(fib[l*m]));
        }
        ms_store(acc, dst + 2*x);
    }
}

// ------------------------------------------------------------ softmax_inplace
template<typename T>
__global__ void softmax_inplace_kernel(Index m, Index k, Index total, const T *mse,
        float alpha, T *dst)
{
    const Index stride = (Index)gridDim.x*blockDim.x, mk = m*k;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        const Index i = x % m, j = x/mk;
        const float v = ld(dst[x]);
        const float top = ld(mse[2*(j*m + i)]), sum = ld(mse[2*(j*m + i) + 1]);
        st(dst[x], isinf(v) ? 0.0f : alpha*expf(v - top)/sum);
    }
}

// m == 1, vector form: the (max, sum) pair and alpha/sum are read and formed once per
// fibre, each value costs one exponential and one product.
template<typename T>
__global__ void __launch_bounds__(256)
softmax_inplace_m1_vec_kernel(Index n, Index k, int lpf, const T *__restrict__ mse, float alpha,
        T *dst)
{
    constexpr int N = Vec<T>::N;
    const int sub = threadIdx.x & (lpf - 1);
    const Index groups = ((Index)gridDim.x*blockDim.x)/lpf;
    for(Index j = ((Index)blockIdx.x*blockDim.x + threadIdx.x)/lpf; j < n; j += groups)
    {
        const float top = ld(mse[2*j]), scale = alpha/ld(mse[2*j + 1]);
        const ExpShift shifted(top);
        T *fib = dst + j*k;
        const Index step = (Index)lpf*N;
        // four pieces (four independent loads) per pass
        for(Index l0 = (Index)sub*N; l0 < k; l0 += 4*step)
        {
            float x[4][N];
#pragma unroll
            for(int u = 0; u < 4; ++u)
            {
                if(l0 + u*step < k)
                {
                    vload(fib + l0 + u*step, x[u]);
                }
            }
#pragma unroll
            for(int u = 0; u < 4; ++u)
            {
                if(l0 + u*step < k)
                {
#pragma unroll
                    for(int e = 0; e < N; ++e)
                    {
                        x[u][e] = isinf(x[u][e]) ? 0.0f : shifted(fib, x[u][e])*scale;
                    }
                    vstore(fib + l0 + u*step, x[u]);
                }
            }
        }
    }
}

// -------------------------------------------------------------- sumprod_slice
template<typename T>
__global__ void __launch_bounds__(256)
sumprod_slice_m1_vec_kernel(Index n, Index k, int lpf, float alpha, const T *__restrict__ a,
        const T *__restrict__ b, float beta, T *dst)
{
    constexpr int N = Vec<T>::N;
    const int sub = threadIdx.x & (lpf - 1);
    const Index groups = ((Index)gridDim.x*blockDim.x)/lpf;
    for(Index j = ((Index)blockIdx.x*blockDim.x + threadIdx.x)/lpf; j < n; j += groups)
    {
        float acc = 0.0f;
        for(Index l = (Index)sub*N; l < k; l += (Index)lpf*N)
        {
            float x[N], y[N];
            vload(a + j*k + l, x);
            vload(b + j*k + l, y);
#pragma unroll
            for(int e = 0; e < N; ++e)
            {
                acc = fmaf(x[e], y[e], acc);
            }
        }
        for(int o = lpf >> 1; o > 0; o >>= 1)
        {
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
        }
        if(sub == 0)
        {
            st(dst[j], beta == 0.0f ? alpha*acc : beta*ld(dst[j]) + alpha*acc);
        }
    }
}

template<typename T>
__global__ void sumprod_slice_m1_kernel(Index n, Index k, float alpha, const T *a,
        const T *b, float beta, T *dst)
{
    const int lane = threadIdx.x & 31;
    const Index warps = ((Index)gridDim.x*blockDim.x) >> 5;
    for(Index j = (((Index)blockIdx.x*blockDim.x + threadIdx.x) >> 5); j < n; j += warps)
    {
        float acc = 0.0f;
        for(Index l = lane; l < k; l += 32)
        {
            acc = fmaf(ld(a[j*k + l]), ld(b[j*k + l]), acc);
        }
        acc = warp_sum(acc);
        if(lane == 0)
        {
            st(dst[j], beta == 0.0f ? alpha*acc : beta*ld(dst[j]) + alpha*acc);
        }
    }
}

template<typename T>
__global__ void sumprod_slice_kernel(Index m, Index n, Index k, float alpha,
        const T *a, const T *b, float beta, T *dst)
{
    const Index total = m*n, stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        const Index i = x % m, j = x/m;
        const T *fa = a + j*m*k + i, *fb = b + j*m*k + i;
        float acc = 0.0f;
        for(Index l = 0; l < k; ++l)
        {
            acc = fmaf(ld(fa[l*m]), ld(fb[l*m]), acc);
        }
        st(dst[x], beta == 0.0f ? alpha*acc : beta*ld(dst[x]) + alpha*acc);
    }
}

// ------------------------------------------------------------- elementwise ops
template<typename T>
__global__ void add_slice_inplace_kernel(Index m, Index k, Index total, float alpha,
        const T *src, float beta, T *dst)
{
    const Index stride = (Index)gridDim.x*blockDim.x, mk = m*k;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        const Index i = x % m, j = x/mk;
        st(dst[x], beta*ld(dst[x]) + alpha*ld(src[j*m + i]));
    }
}

// m == 1, vector form: one slice value per fibre.
template<typename T>
__global__ void __launch_bounds__(256)
add_slice_inplace_m1_vec_kernel(Index n, Index k, int lpf, float alpha, const T *__restrict__ src,
        float beta, T *dst)
{
    constexpr int N = Vec<T>::N;
    const int sub = threadIdx.x & (lpf - 1);
    const Index groups = ((Index)gridDim.x*blockDim.x)/lpf;
    for(Index j = ((Index)blockIdx.x*blockDim.x + threadIdx.x)/lpf; j < n; j += groups)
    {
        const float add = alpha*ld(src[j]);
        T *fib = dst + j*k;
        const Index step = (Index)lpf*N;
        // four pieces (four independent loads) per pass
        for(Index l0 = (Index)sub*N; l0 < k; l0 += 4*step)
        {
            float x[4][N];
#pragma unroll
            for(int u = 0; u < 4; ++u)
            {
                if(l0 + u*step < k)
                {
                    vload(fib + l0 + u*step, x[u]);
                }
            }
#pragma unroll
            for(int u = 0; u < 4; ++u)
            {
                if(l0 + u*step < k)
                {
#pragma unroll
                    for(int e = 0; e < N; ++e)
                    {
                        x[u][e] = beta*x[u][e] + add;
                    }
                    vstore(fib + l0 + u*step, x[u]);
                }
            }
        }
    }
}

// dst = alpha*src*dst (MUL) or alpha*src + beta*dst (ADD), 16 bytes per thread.
template<typename T, bool MUL>
__global__ void __launch_bounds__(256)
binary_inplace_vec_kernel(Index pieces, float alpha, const T *__restrict__ src, float beta, T *dst)
{
    constexpr int N = Vec<T>::N;
    const Index stride = (Index)gridDim.x*blockDim.x;
    for(Index v = (Index)blockIdx.x*blockDim.x + threadIdx.x; v < pieces; v += stride)
    {
        float x[N], y[N];
        vload(src + v*N, x);
        vload(dst + v*N, y);
#pragma unroll
        for(int e = 0; e < N; ++e)
        {
            y[e] = MUL ? alpha*y[e]*x[e] : alpha*x[e] + beta*y[e];
        }
        vstore(dst + v*N, y);
    }
}

template<typename T>
__global__ void multiply_inplace_kernel(Index total, float alpha, const T *src, T *dst)
{
    const Index stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        st(dst[x], alpha*ld(dst[x])*ld(src[x]));
    }
}

template<typename T>
__global__ void add_inplace_kernel(Index total, float alpha, const T *src, float beta,
        T *dst)
{
    const Index stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        st(dst[x], alpha*ld(src[x]) + beta*ld(dst[x]));
    }
}

__global__ void fill_kernel(Index total, float val, float *dst)
{
    const Index stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        dst[x] = val;
    }
}

// ----------------------------------------------------- accumulate_attn_output
// One warp per (seq, batch) row: lane 0's weights are broadcast, the head
// elements are spread over the lanes.
template<typename T>
__global__ void accumulate_attn_output_kernel(Index head, Index rows,
        const float *src_lse, const T *src_attn, float *dst_lse, T *dst_attn)
{
    const int lane = threadIdx.x & 31;
    const Index warps = ((Index)gridDim.x*blockDim.x) >> 5;
    for(Index r = (((Index)blockIdx.x*blockDim.x + threadIdx.x) >> 5); r < rows; r += warps)
    {
        const float in = src_lse[r];
        if(!isfinite(in))
        {
            continue;
        }
        const float old = dst_lse[r];
        float top, e, w_dst, w_src;
        if(old > in)
        {
            top = old;
            e = expf(in - top);
            w_dst = 1.0f/(1.0f + e);
            w_src = e*w_dst;
        }
        else
        {
            top = in;
            e = expf(old - top);
            w_src = 1.0f/(1.0f + e);
            w_dst = e*w_src;
        }
        __syncwarp();
        if(lane == 0)
        {
            dst_lse[r] = top + logf(1.0f + e);
        }
        for(Index h = lane; h < head; h += 32)
        {
            const Index x = r*head + h;
            st(dst_attn[x], w_dst*ld(dst_attn[x]) + w_src*ld(src_attn[x]));
        }
    }
}

// --------------------------------------------------------------- host drivers
template<typename T>
int mask_scalar_run(cudaStream_t s, Index nrows, Index ncols, const uint8_t *mask,
        float val, T *data)
{
    if(nrows < 0 || ncols < 0) return NNTILE_B200_E_BADARG;
    if(nrows == 0 || ncols == 0) return NNTILE_B200_OK;
    if(!mask || !data) return NNTILE_B200_E_BADARG;
    const Index total = nrows*ncols;
    if(vec_ok<T>(nrows, data) && (reinterpret_cast<uintptr_t>(mask) & 7u) == 0)
    {
        const Index pieces = nrows/Vec<T>::N;
        Index gx = (pieces + 255)/256, gy = ncols;
        if(gx > 148*4) gx = 148*4;
        if(gy > 1024) gy = 1024;
        while(gx*gy > 148*32 && gy > 1) gy = (gy + 1)/2;
        mask_scalar_vec_kernel<T><<<dim3((unsigned)gx, (unsigned)gy), 256, 0, s>>>(nrows, ncols,
                mask, val, data);
        return launch_status();
    }
    mask_scalar_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(nrows, total, mask, val, data);
    return launch_status();
}

template<typename T>
int maxsumexp_run(cudaStream_t s, Index m, Index n, Index k, const T *src, T *dst)
{
    if(m < 0 || n < 0 || k < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0 || k == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    if(m == 1 && vec_ok<T>(k, src))
    {
        const int lpf = lanes_per_fibre<T>(k);
        maxsumexp_m1_vec_kernel<T><<<fibre_grid(n, lpf), 256, 0, s>>>(n, k, lpf, src, dst);
    }
    else if(m == 1)
    {
        // 8 warps per block, one fibre per warp per pass
        Index blocks = (n + 7)/8;
        if(blocks > 148*8) blocks = 148*8;
        maxsumexp_m1_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(n, k, src, dst);
    }
    else
    {
        maxsumexp_kernel<T><<<grid_for(m*n, 128, 1), 128, 0, s>>>(m, n, k, src, dst);
    }
    return launch_status();
}

template<typename T>
int softmax_inplace_run(cudaStream_t s, Index m, Index n, Index k, const T *mse,
        float alpha, T *dst)
{
    if(m < 0 || n < 0 || k < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0 || k == 0) return NNTILE_B200_OK;
    if(!mse || !dst) return NNTILE_B200_E_BADARG;
    const Index total = m*n*k;
    if(m == 1 && vec_ok<T>(k, dst))
    {
        const int lpf = lanes_per_fibre<T>(k);
        softmax_inplace_m1_vec_kernel<T><<<fibre_grid(n, lpf), 256, 0, s>>>(n, k, lpf, mse, alpha,
                dst);
        return launch_status();
    }
    softmax_inplace_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(m, k, total, mse, alpha, dst);
    return launch_status();
}

template<typename T>
int sumprod_slice_run(cudaStream_t s, Index m, Index n, Index k, float alpha,
        const T *a, const T *b, float beta, T *dst)
{
    if(m < 0 || n < 0 || k < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0) return NNTILE_B200_OK;
    if(!dst || (k > 0 && (!a || !b))) return NNTILE_B200_E_BADARG;
    if(m == 1 && k > 0 && vec_ok<T>(k, a, b))
    {
        const int lpf = lanes_per_fibre<T>(k);
        sumprod_slice_m1_vec_kernel<T><<<fibre_grid(n, lpf), 256, 0, s>>>(n, k, lpf, alpha, a, b,
                beta, dst);
    }
    else if(m == 1)
    {
        Index blocks = (n + 7)/8;
        if(blocks > 148*8) blocks = 148*8;
        sumprod_slice_m1_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(n, k, alpha, a, b, beta, dst);
    }
    else
    {
        sumprod_slice_kernel<T><<<grid_for(m*n, 128, 1), 128, 0, s>>>(m, n, k, alpha, a, b, beta, dst);
    }
    return launch_status();
}

template<typename T>
int add_slice_inplace_run(cudaStream_t s, Index m, Index n, Index k, float alpha,
        const T *src, float beta, T *dst)
{
    if(m < 0 || n < 0 || k < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0 || k == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    const Index total = m*n*k;
    if(m == 1 && vec_ok<T>(k, dst))
    {
        const int lpf = lanes_per_fibre<T>(k);
        add_slice_inplace_m1_vec_kernel<T><<<fibre_grid(n, lpf), 256, 0, s>>>(n, k, lpf, alpha, src,
                beta, dst);
        return launch_status();
    }
    add_slice_inplace_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(m, k, total, alpha, src, beta, dst);
    return launch_status();
}

template<typename T>
int multiply_inplace_run(cudaStream_t s, Index nelems, float alpha, const T *src, T *dst)
{
    if(nelems < 0) return NNTILE_B200_E_BADARG;
    if(nelems == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    if(vec_ok<T>(nelems, src, dst))
    {
        const Index pieces = nelems/Vec<T>::N;
        binary_inplace_vec_kernel<T, true><<<grid_for(pieces, 256, 2), 256, 0, s>>>(pieces, alpha,
                src, 0.0f, dst);
        return launch_status();
    }
    multiply_inplace_kernel<T><<<grid_for(nelems, 256), 256, 0, s>>>(nelems, alpha, src, dst);
    return launch_status();
}

template<typename T>
int add_inplace_run(cudaStream_t s, Index nelems, float alpha, const T *src, float beta,
        T *dst)
{
    if(nelems < 0) return NNTILE_B200_E_BADARG;
    if(nelems == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    if(vec_ok<T>(nelems, src, dst))
    {
        const Index pieces = nelems/Vec<T>::N;
        binary_inplace_vec_kernel<T, false><<<grid_for(pieces, 256, 2), 256, 0, s>>>(pieces, alpha,
                src, beta, dst);
        return launch_status();
    }
    add_inplace_kernel<T><<<grid_for(nelems, 256), 256, 0, s>>>(nelems, alpha, src, beta, dst);
    return launch_status();
}

template<typename T>
int accumulate_run(cudaStream_t s, Index head, Index seq, Index batch,
        const float *src_lse, const T *src_attn, float *dst_lse, T *dst_attn)
{
    if(head < 0 || seq < 0 || batch < 0) return NNTILE_B200_E_BADARG;
    if(head == 0 || seq == 0 || batch == 0) return NNTILE_B200_OK;
    if(!src_lse || !src_attn || !dst_lse || !dst_attn) return NNTILE_B200_E_BADARG;
    const Index rows = seq*batch;
    Index blocks = (rows + 7)/8;
    if(blocks > 148*8) blocks = 148*8;
    accumulate_attn_output_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(head, rows,
            src_lse, src_attn, dst_lse, dst_attn);
    return launch_status();
}

} // namespace nb200

using namespace nb200;

#define NB200_OPS(SFX, CT, VT) \
extern "C" int nntile_b200_mask_scalar_##SFX(nntile_b200_stream_t s, int64_t nrows, \
        int64_t ncols, const uint8_t *mask, float val, VT *data) \
{ return mask_scalar_run<CT>(as_stream(s), nrows, ncols, mask, val, (CT *)data); } \
extern "C" int nntile_b200_maxsumexp_##SFX(nntile_b200_stream_t s, int64_t m, int64_t n, \
        int64_t k, const VT *src, VT *dst) \
{ return maxsumexp_run<CT>(as_stream(s), m, n, k, (const CT *)src, (CT *)dst); } \
extern "C" int nntile_b200_softmax_inplace_##SFX(nntile_b200_stream_t s, int64_t m, \
        int64_t n, int64_t k, const VT *mse, float alpha, VT *dst) \
{ return softmax_inplace_run<CT>(as_stream(s), m, n, k, (const CT *)mse, alpha, (CT *)dst); } \
extern "C" int nntile_b200_sumprod_slice_##SFX(nntile_b200_stream_t s, int64_t m, \
        int64_t n, int64_t k, float alpha, const VT *a, const VT *b, float beta, VT *dst) \
{ return sumprod_slice_run<CT>(as_stream(s), m, n, k, alpha, (const CT *)a, (const CT *)b, beta, (CT *)dst); } \
extern "C" int nntile_b200_add_slice_inplace_##SFX(nntile_b200_stream_t s, int64_t m, \
        int64_t n, int64_t k, float alpha, const VT *src, float beta, VT *dst) \
{ return add_slice_inplace_run<CT>(as_stream(s), m, n, k, alpha, (const CT *)src, beta, (CT *)dst); } \
extern "C" int nntile_b200_multiply_inplace_##SFX(nntile_b200_stream_t s, int64_t nelems, \
        float alpha, const VT *src, VT *dst) \
{ return multiply_inplace_run<CT>(as_stream(s), nelems, alpha, (const CT *)src, (CT *)dst); } \
extern "C" int nntile_b200_add_inplace_##SFX(nntile_b200_stream_t s, int64_t nelems, \
        float alpha, const VT *src, float beta, VT *dst) \
{ return add_inplace_run<CT>(as_stream(s), nelems, alpha, (const CT *)src, beta, (CT *)dst); } \
extern "C" int nntile_b200_accumulate_attn_output_##SFX(nntile_b200_stream_t s, \
        int64_t head, int64_t seq, int64_t batch, const float *src_lse, \
        const VT *src_attn, float *dst_lse, VT *dst_attn) \
{ return accumulate_run<CT>(as_stream(s), head, seq, batch, src_lse, (const CT *)src_attn, dst_lse, (CT *)dst_attn); }

NB200_OPS(fp32, float, float)
NB200_OPS(bf16, bf16, void)

extern "C" int nntile_b200_fill_fp32(nntile_b200_stream_t s, int64_t nelems, float val,
        float *dst)
{
    if(nelems < 0) return NNTILE_B200_E_BADARG;
    if(nelems == 0) return NNTILE_B200_OK;
    if(!dst) return NNTILE_B200_E_BADARG;
    fill_kernel<<<grid_for(nelems, 256), 256, 0, as_stream(s)>>>(nelems, val, dst);
    return launch_status();
}

extern "C" int nntile_b200_clear(nntile_b200_stream_t s, int64_t nbytes, void *dst)
{
    if(nbytes < 0) return NNTILE_B200_E_BADARG;
    if(nbytes == 0) return NNTILE_B200_OK;
    if(!dst) return NNTILE_B200_E_BADARG;
    return cudaMemsetAsync(dst, 0, (size_t)nbytes, as_stream(s)) == cudaSuccess
            ? NNTILE_B200_OK : NNTILE_B200_E_LAUNCH;
}

extern "C" unsigned long long nntile_b200_launch_count(void)
{
    return g_kernel_launches.load(std::memory_order_relaxed);
}

extern "C" int nntile_b200_version(void)
{
    return 100;
}

extern "C" const char *nntile_b200_status_string(int status)
{
    switch(status)
    {
        case NNTILE_B200_OK: return "ok";
        case NNTILE_B200_E_BADARG: return "bad argument";
        case NNTILE_B200_E_SHAPE: return "shape not supported";
        case NNTILE_B200_E_ALIGN: return "pointer not 16-byte aligned";
        case NNTILE_B200_E_SCRATCH: return "scratch too small";
        case NNTILE_B200_E_LAUNCH: return "CUDA launch failed";
        case NNTILE_B200_E_DEVICE: return "device is not sm_100";
        default: return "unknown status";
    }
}
