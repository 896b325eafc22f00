// Layout change in front of and behind the SDPA layer, fused with what the
// reference runs as separate passes next to it (HBM-bound; one read and one
// write of the tensor instead of two or three of each).
//
// The projections of the reference's attention layers produce
// [lead, head, seq, batch] with lead = (group, kv_heads) or (kv_heads) fastest;
// the SDPA layer wants [head, seq, batch, lead].  The reference gets there with
//   transpose_async(1.0, proj_out, q, ndim)         src/kernel/transpose/cuda.cu:24-99
//   rope_async(sin, cos, q, q_rope)                 src/kernel/rope/cuda.cu:21-57
//     (wrappers/python/nntile/model/llama_attention.py:592-625)
// or, in GPT-2,
//   transpose_async + add_fiber_inplace_async(1.0, bias, 1.0, q, 0, 1)
//     (wrappers/python/nntile/model/gpt2_attention.py:258-273)
// and transposes the attention output back for the output projection.  With the
// grouped-query entry points of the fused pair there is no K/V replication pass
// (add_slice_inplace) left either.
//
// One CTA handles `tp` consecutive (seq, batch) positions at a time: their
// lead*head*tp source elements are one contiguous run, and for every value of
// `lead` the tp*head destination elements are one contiguous run too.  The run is
// staged in shared memory as [position*head + d][lead] with an odd row stride in
// 32-bit words; a warp then reads one `lead` column for 32 consecutive (d, d+1)
// pairs and writes 128 contiguous bytes.
//
// Arithmetic matches the reference's kernels bit for bit: the transposition is
// exact, RoPE is round(round(c*a) - round(s*b)) in fp32 (no fused multiply-add,
// as its CPU kernel src/kernel/rope/cpu.cc:24-49 computes it) rounded once to
// bf16, the bias is added in fp32 and rounded once.
#include "common.cuh"

namespace nb200 {

enum : int { PRO_PLAIN = 0, PRO_ROPE = 1, PRO_BIAS = 2 };

constexpr int PRO_THREADS = 256;

__host__ __device__ inline int pro_stride_words(int lead)
{
    // words per staged row: lead/2 rounded up to an odd number
    const int w = (lead + 1)/2;
    return (w & 1) ? w : w + 1;
}

template<int MODE>
__global__ void __launch_bounds__(PRO_THREADS)
transpose_in_kernel(int lead, int head, Index npos, int tp, const bf16 *__restrict__ aux0,
        const bf16 *__restrict__ aux1, const bf16 *__restrict__ src, bf16 *__restrict__ dst)
{
    extern __shared__ uint32_t tile[];
    const int sw = pro_stride_words(lead);
    const Index nchunks = (npos + tp - 1)/tp;
    const int hp = head/2;                                // (d, d+1) pairs per position
    const int hp_shift = (hp & (hp - 1)) == 0 ? 31 - __clz(hp) : -1;
    for(Index c = blockIdx.x; c < nchunks; c += gridDim.x)
    {
        const Index pos0 = c*tp;
        const int np = (int)((npos - pos0) < tp ? (npos - pos0) : tp);
        const int rows = np*head;
        // ---- stage: contiguous run of rows*lead elements; 16 bytes per thread when a
        // row holds whole 16-byte pieces, 4 bytes otherwise (e.g. 12 heads)
        if((lead & 7) == 0)
        {
            const uint4 *g = reinterpret_cast<const uint4 *>(src + pos0*(Index)head*lead);
            const int nvec = rows*lead/8;
            for(int v = threadIdx.x; v < nvec; v += PRO_THREADS)
            {
                const uint4 x = g[v];
                const int e = 8*v, row = e/lead, col = e - row*lead;
                uint32_t *t = tile + row*sw + (col >> 1);
                t[0] = x.x;
                t[1] = x.y;
                t[2] = x.z;
                t[3] = x.w;
            }
        }
        else
        {
            const uint32_t *g = reinterpret_cast<const uint32_t *>(src + pos0*(Index)head*lead);
            const int nw = rows*lead/2, lw = lead/2;
            for(int v = threadIdx.x; v < nw; v += PRO_THREADS)
            {
                const int row = v/lw;
                tile[row*sw + (v - row*lw)] = g[v];
            }
        }
        __syncthreads();
        // ---- emit: a warp takes one lead index at a time and walks its np*hp pairs
        // = np*head contiguous destination elements
        const int run = np*hp;
        for(int n = threadIdx.x >> 5; n < lead; n += PRO_THREADS/32)
        for(int rem = threadIdx.x & 31; rem < run; rem += 32)
        {
            const int pp = hp_shift >= 0 ? (rem >> hp_shift) : rem/hp, p = rem - pp*hp;
            const int row = pp*head + 2*p;
            const uint32_t w0 = tile[row*sw + (n >> 1)], w1 = tile[(row + 1)*sw + (n >> 1)];
            const uint32_t h0 = (n & 1) ? (w0 >> 16) : (w0 & 0xFFFFu);
            const uint32_t h1 = (n & 1) ? (w1 >> 16) : (w1 & 0xFFFFu);
            uint32_t out = h0 | (h1 << 16);
            if(MODE == PRO_ROPE)
            {
                const Index i = (pos0 + pp)*(Index)hp + p;      // index into sin / cos
                const float s = __bfloat162float(aux0[i]), co = __bfloat162float(aux1[i]);
                const float a = __uint_as_float(h0 << 16), b = __uint_as_float(h1 << 16);
                const float x = __fsub_rn(__fmul_rn(co, a), __fmul_rn(s, b));
                const float y = __fadd_rn(__fmul_rn(s, a), __fmul_rn(co, b));
                out = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x))
                        | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y)) << 16);
            }
            else if(MODE == PRO_BIAS)
            {
                const uint32_t bw = *reinterpret_cast<const uint32_t *>(
                        aux0 + (Index)n*head + 2*p);            // bias[d, n], d fastest
                const float x = __fadd_rn(__uint_as_float(h0 << 16), __uint_as_float(bw << 16));
                const float y = __fadd_rn(__uint_as_float(h1 << 16),
                        __uint_as_float(bw & 0xFFFF0000u));
                out = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(x))
                        | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(y)) << 16);
            }
            *reinterpret_cast<uint32_t *>(dst + (Index)n*npos*head + pos0*(Index)head + 2*rem) = out;
        }
        __syncthreads();
    }
}

// dst[n, d, pos] = src[d, pos, n]: the inverse layout change.
__global__ void __launch_bounds__(PRO_THREADS)
transpose_out_kernel(int lead, int head, Index npos, int tp, const bf16 *__restrict__ src,
        bf16 *__restrict__ dst)
{
    extern __shared__ uint32_t tile[];
    uint16_t *tile16 = reinterpret_cast<uint16_t *>(tile);
    const int sw = pro_stride_words(lead);
    const Index nchunks = (npos + tp - 1)/tp;
    const int hp = head/2;
    for(Index c = blockIdx.x; c < nchunks; c += gridDim.x)
    {
        const Index pos0 = c*tp;
        const int np = (int)((npos - pos0) < tp ? (npos - pos0) : tp);
        const int rows = np*head;
        const int run = np*hp;
        for(int n = threadIdx.x >> 5; n < lead; n += PRO_THREADS/32)
        for(int rem = threadIdx.x & 31; rem < run; rem += 32)
        {
            const uint32_t w = *reinterpret_cast<const uint32_t *>(
                    src + (Index)n*npos*head + pos0*(Index)head + 2*rem);
            const int row = 2*rem;                               // = pp*head + 2*p
            tile16[2*(row*sw) + n] = (uint16_t)(w & 0xFFFFu);
            tile16[2*((row + 1)*sw) + n] = (uint16_t)(w >> 16);
        }
        __syncthreads();
        if((lead & 7) == 0)
        {
            uint4 *g = reinterpret_cast<uint4 *>(dst + pos0*(Index)head*lead);
            const int nvec = rows*lead/8;
            for(int v = threadIdx.x; v < nvec; v += PRO_THREADS)
            {
                const int e = 8*v, row = e/lead, col = e - row*lead;
                const uint32_t *t = tile + row*sw + (col >> 1);
                g[v] = make_uint4(t[0], t[1], t[2], t[3]);
            }
        }
        else
        {
            uint32_t *g = reinterpret_cast<uint32_t *>(dst + pos0*(Index)head*lead);
            const int nw = rows*lead/2, lw = lead/2;
            for(int v = threadIdx.x; v < nw; v += PRO_THREADS)
            {
                const int row = v/lw;
                g[v] = tile[row*sw + (v - row*lw)];
            }
        }
        __syncthreads();
    }
}

struct ProPlan
{
    int tp;
    size_t smem;
    unsigned grid;
};

static int pro_check(int64_t lead, int64_t head, int64_t seq, int64_t batch)
{
    if(lead < 0 || head < 0 || seq < 0 || batch < 0) return NNTILE_B200_E_BADARG;
    // two `lead` indices per 32-bit word and (d, d+1) pairs
    if(lead % 2 != 0 || head % 2 != 0 || lead > 1024 || head > 1024) return NNTILE_B200_E_SHAPE;
    if(seq*batch >= ((int64_t)1 << 40)) return NNTILE_B200_E_SHAPE;
    return NNTILE_B200_OK;
}

static ProPlan pro_plan(int lead, int head, Index npos)
{
    ProPlan p;
    const size_t row_bytes = (size_t)pro_stride_words(lead)*4;
    // positions per chunk: up to about 32 KB of staging, at least one position
    int tp = (int)((size_t)32768/(row_bytes*head));
    if(tp < 1) tp = 1;
    if(tp > 8) tp = 8;
    if((Index)tp > npos) tp = (int)npos;
    p.tp = tp;
    p.smem = row_bytes*head*tp;
    const Index nchunks = (npos + tp - 1)/tp;
    const Index cap = 148*6;
    p.grid = (unsigned)(nchunks < cap ? nchunks : cap);
    return p;
}

template<typename Kernel>
static bool pro_optin(Kernel kernel, size_t smem)
{
    // one position of a large (lead, head) may need more than the default 48 KB
    return smem <= 48*1024 || cudaFuncSetAttribute(kernel,
            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
}

} // namespace nb200

using namespace nb200;

extern "C" int nntile_b200_transpose_rope_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *sin, const void *cos,
        const void *src, void *dst)
{
    int st = pro_check(lead, head, seq, batch);
    if(st != NNTILE_B200_OK) return st;
    const Index npos = seq*batch;
    if(lead == 0 || head == 0 || npos == 0) return NNTILE_B200_OK;
    if(!src || !dst || ((sin == nullptr) != (cos == nullptr))) return NNTILE_B200_E_BADARG;
    if(!aligned16(src) || !aligned16(dst)) return NNTILE_B200_E_ALIGN;
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(sin)
    {
        if(!pro_optin(transpose_in_kernel<PRO_ROPE>, p.smem)) return NNTILE_B200_E_LAUNCH;
        transpose_in_kernel<PRO_ROPE><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>(
                (int)lead, (int)head, npos, p.tp, (const bf16 *)sin, (const bf16 *)cos,
                (const bf16 *)src, (bf16 *)dst);
    }
    else
    {
        if(!pro_optin(transpose_in_kernel<PRO_PLAIN>, p.smem)) return NNTILE_B200_E_LAUNCH;
        transpose_in_kernel<PRO_PLAIN><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>(
                (int)lead, (int)head, npos, p.tp, nullptr, nullptr, (const bf16 *)src,
                (bf16 *)dst);
    }
    return launch_status();
}

extern "C" int nntile_b200_transpose_bias_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *bias, const void *src, void *dst)
{
    int st = pro_check(lead, head, seq, batch);
    if(st != NNTILE_B200_OK) return st;
    const Index npos = seq*batch;
    if(lead == 0 || head == 0 || npos == 0) return NNTILE_B200_OK;
    if(!src || !dst || !bias) return NNTILE_B200_E_BADARG;
    if(!aligned16(src) || (reinterpret_cast<uintptr_t>(dst) & 3u)
            || (reinterpret_cast<uintptr_t>(bias) & 3u))
    {
        return NNTILE_B200_E_ALIGN;
    }
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(!pro_optin(transpose_in_kernel<PRO_BIAS>, p.smem)) return NNTILE_B200_E_LAUNCH;
    transpose_in_kernel<PRO_BIAS><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>((int)lead,
            (int)head, npos, p.tp, (const bf16 *)bias, nullptr, (const bf16 *)src, (bf16 *)dst);
    return launch_status();
}

extern "C" int nntile_b200_transpose_heads_back_bf16(nntile_b200_stream_t stream, int64_t lead,
        int64_t head, int64_t seq, int64_t batch, const void *src, void *dst)
{
    int st = pro_check(lead, head, seq, batch);
    if(st != NNTILE_B200_OK) return st;
    const Index npos = seq*batch;
    if(lead == 0 || head == 0 || npos == 0) return NNTILE_B200_OK;
    if(!src || !dst) return NNTILE_B200_E_BADARG;
    if(!aligned16(dst) || !aligned16(src)) return NNTILE_B200_E_ALIGN;
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(!pro_optin(transpose_out_kernel, p.smem)) return NNTILE_B200_E_LAUNCH;
    transpose_out_kernel<<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>((int)lead, (int)head,
            npos, p.tp, (const bf16 *)src, (bf16 *)dst);
    return launch_status();
}
