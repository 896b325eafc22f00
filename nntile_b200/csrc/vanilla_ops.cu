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

// ---------------------------------------------------------------- mask_scalar
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

// -------------------------------------------------------------- sumprod_slice
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
    mask_scalar_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(nrows, total, mask, val, data);
    return launch_status();
}

template<typename T>
int maxsumexp_run(cudaStream_t s, Index m, Index n, Index k, const T *src, T *dst)
{
    if(m < 0 || n < 0 || k < 0) return NNTILE_B200_E_BADARG;
    if(m == 0 || n == 0 || k == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    if(m == 1)
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
    if(m == 1)
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
    add_slice_inplace_kernel<T><<<grid_for(total, 256), 256, 0, s>>>(m, k, total, alpha, src, beta, dst);
    return launch_status();
}

template<typename T>
int multiply_inplace_run(cudaStream_t s, Index nelems, float alpha, const T *src, T *dst)
{
    if(nelems < 0) return NNTILE_B200_E_BADARG;
    if(nelems == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
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
