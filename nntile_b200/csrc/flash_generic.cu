// Fused flash-SDPA tile tasks for shapes the tcgen05 kernels do not take (any
// seq, any head <= 256): plain CUDA-core kernels, one warp per attention row,
// online max / sum-exp in registers, dot products reduced with warp shuffles.
// They define the semantics of the C entry points for every shape and are the
// path the reference's own small test shapes (seq 16..64, head 8..64) run on.
//
// Semantics follow src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:145-202 (attention of
// one (Q tile, K/V tile) pair with an additive bias, then the log-sum-exp merge
// of src/kernel/accumulate_attn_output/cuda.cu:28-113 into (lse, A)) and
// src/kernel/flash_sdpa_bwd_cudnn/cuda.cc:171-218 (gradients from the given A and
// lse, rounded to the storage type, then added into dK, dQ, dV).
#include "common.cuh"
#include "flash.cuh"

namespace nb200 {
inline namespace NB200_ELEM_NS {

constexpr int GEN_MAX_EPL = 8;      // elements of a head vector per lane
constexpr int GEN_WARPS = 4;

// Load the lane's slice [lane*epl, lane*epl+epl) of a row of `head` elements.
template<int EPL>
__device__ __forceinline__ void load_slice(const elem_t *row, int head, int lane,
        float (&out)[EPL])
{
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        const int h = lane*EPL + t;
        out[t] = h < head ? elem_to_f(row[h]) : 0.0f;
    }
}

template<int EPL>
__device__ __forceinline__ float dot_slice(const float (&a)[EPL], const float (&b)[EPL])
{
    float acc = 0.0f;
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        acc = fmaf(a[t], b[t], acc);
    }
    return acc;
}

// -------------------------------------------------------------------- forward
template<int EPL>
__global__ void __launch_bounds__(GEN_WARPS*32)
flash_fwd_generic_kernel(int seq, int head, Index rows, float scale,
        const elem_t *__restrict__ K, const elem_t *__restrict__ Q,
        const elem_t *__restrict__ mask, const elem_t *__restrict__ V,
        float *__restrict__ lse, elem_t *__restrict__ A)
{
    const int lane = threadIdx.x & 31;
    const Index r = (Index)blockIdx.x*GEN_WARPS + (threadIdx.x >> 5);
    if(r >= rows)
    {
        return;
    }
    const Index b = r/seq;
    const int i = (int)(r - b*seq);
    const elem_t *Kb = K + b*seq*head, *Vb = V + b*seq*head;
    float q[EPL], o[EPL], kv[EPL];
    load_slice<EPL>(Q + r*head, head, lane, q);
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        o[t] = 0.0f;
    }
    float top = -CUDART_INF_F, sum = 0.0f;
    const elem_t *mrow = mask + (Index)i*seq;
    for(int j = 0; j < seq; ++j)
    {
        const float bias = elem_to_f(mrow[j]);
        if(bias == -CUDART_INF_F)
        {
            continue;                       // warp-uniform: the key is masked
        }
        load_slice<EPL>(Kb + (Index)j*head, head, lane, kv);
        const float s = warp_sum(dot_slice<EPL>(q, kv))*scale + bias;
        if(s == -CUDART_INF_F)
        {
            continue;
        }
        const float ntop = fmaxf(top, s);
        const float shrink = expf(top - ntop);      // 0 on the first key
        const float p = expf(s - ntop);
        sum = sum*shrink + p;
        load_slice<EPL>(Vb + (Index)j*head, head, lane, kv);
#pragma unroll
        for(int t = 0; t < EPL; ++t)
        {
            o[t] = o[t]*shrink + p*kv[t];
        }
        top = ntop;
    }
    // Merge with the running (lse, A): accumulate_attn_output, CUDA rules.
    const float in = sum > 0.0f ? top + logf(sum) : -CUDART_INF_F;
    if(!isfinite(in))
    {
        return;
    }
    const float old = lse[r];
    float e, w_dst, w_src, big;
    if(old > in)
    {
        big = old;
        e = expf(in - big);
        w_dst = 1.0f/(1.0f + e);
        w_src = e*w_dst;
    }
    else
    {
        big = in;
        e = expf(old - big);
        w_src = 1.0f/(1.0f + e);
        w_dst = e*w_src;
    }
    if(lane == 0)
    {
        lse[r] = big + logf(1.0f + e);
    }
    const float inv = 1.0f/sum;
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        const int h = lane*EPL + t;
        if(h < head)
        {
            // the tile result is rounded to storage before the merge, as the
            // reference's scratch output is
            const float part = elem_round((o[t]*inv));
            const float prev = elem_to_f(A[r*head + h]);
            A[r*head + h] = f_to_elem(w_dst*prev + w_src*part);
        }
    }
}

// ------------------------------------------------------------------- backward
// delta[r] = sum_h A[r,h]*dA[r,h]
__global__ void flash_bwd_delta_kernel(int head, Index rows, const elem_t *__restrict__ A,
        const elem_t *__restrict__ dA, float *__restrict__ delta)
{
    const int lane = threadIdx.x & 31;
    const Index r = (Index)blockIdx.x*(blockDim.x >> 5) + (threadIdx.x >> 5);
    if(r >= rows)
    {
        return;
    }
    float acc = 0.0f;
    for(int h = lane; h < head; h += 32)
    {
        acc = fmaf(elem_to_f(A[r*head + h]), elem_to_f(dA[r*head + h]), acc);
    }
    acc = warp_sum(acc);
    if(lane == 0)
    {
        delta[r] = acc;
    }
}

// dQ: one warp per query row, loop over keys.
template<int EPL>
__global__ void __launch_bounds__(GEN_WARPS*32)
flash_bwd_dq_generic_kernel(int seq, int head, Index rows, float scale,
        const elem_t *__restrict__ K, const elem_t *__restrict__ Q,
        const elem_t *__restrict__ V, const elem_t *__restrict__ dA,
        const elem_t *__restrict__ mask, const float *__restrict__ lse,
        const float *__restrict__ delta, elem_t *__restrict__ dQ)
{
    const int lane = threadIdx.x & 31;
    const Index r = (Index)blockIdx.x*GEN_WARPS + (threadIdx.x >> 5);
    if(r >= rows)
    {
        return;
    }
    const Index b = r/seq;
    const int i = (int)(r - b*seq);
    const elem_t *Kb = K + b*seq*head, *Vb = V + b*seq*head;
    float q[EPL], g[EPL], acc[EPL], kk[EPL], vv[EPL];
    load_slice<EPL>(Q + r*head, head, lane, q);
    load_slice<EPL>(dA + r*head, head, lane, g);
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        acc[t] = 0.0f;
    }
    const float row_lse = lse[r], row_delta = delta[r];
    const elem_t *mrow = mask + (Index)i*seq;
    for(int j = 0; j < seq; ++j)
    {
        const float bias = elem_to_f(mrow[j]);
        if(bias == -CUDART_INF_F)
        {
            continue;
        }
        load_slice<EPL>(Kb + (Index)j*head, head, lane, kk);
        load_slice<EPL>(Vb + (Index)j*head, head, lane, vv);
        const float s = warp_sum(dot_slice<EPL>(q, kk))*scale + bias;
        const float dp = warp_sum(dot_slice<EPL>(g, vv));
        const float p = s == -CUDART_INF_F ? 0.0f : expf(s - row_lse);
        const float ds = p*(dp - row_delta)*scale;
#pragma unroll
        for(int t = 0; t < EPL; ++t)
        {
            acc[t] = fmaf(ds, kk[t], acc[t]);
        }
    }
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        const int h = lane*EPL + t;
        if(h < head)
        {
            const float part = elem_round((acc[t]));
            dQ[r*head + h] = f_to_elem(part + elem_to_f(dQ[r*head + h]));
        }
    }
}

// dK, dV: one warp per key row, loop over queries.
template<int EPL>
__global__ void __launch_bounds__(GEN_WARPS*32)
flash_bwd_dkv_generic_kernel(int seq, int head, Index rows, float scale,
        const elem_t *__restrict__ K, const elem_t *__restrict__ Q,
        const elem_t *__restrict__ V, const elem_t *__restrict__ dA,
        const elem_t *__restrict__ mask, const float *__restrict__ lse,
        const float *__restrict__ delta, elem_t *__restrict__ dK, elem_t *__restrict__ dV)
{
    const int lane = threadIdx.x & 31;
    const Index r = (Index)blockIdx.x*GEN_WARPS + (threadIdx.x >> 5);
    if(r >= rows)
    {
        return;
    }
    const Index b = r/seq;
    const int j = (int)(r - b*seq);
    const elem_t *Qb = Q + b*seq*head, *Gb = dA + b*seq*head;
    float kk[EPL], vv[EPL], gk[EPL], gv[EPL], qq[EPL], gg[EPL];
    load_slice<EPL>(K + r*head, head, lane, kk);
    load_slice<EPL>(V + r*head, head, lane, vv);
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        gk[t] = 0.0f;
        gv[t] = 0.0f;
    }
    for(int i = 0; i < seq; ++i)
    {
        const float bias = elem_to_f(mask[(Index)i*seq + j]);
        if(bias == -CUDART_INF_F)
        {
            continue;
        }
        load_slice<EPL>(Qb + (Index)i*head, head, lane, qq);
        load_slice<EPL>(Gb + (Index)i*head, head, lane, gg);
        const float s = warp_sum(dot_slice<EPL>(qq, kk))*scale + bias;
        const float dp = warp_sum(dot_slice<EPL>(gg, vv));
        const float p = s == -CUDART_INF_F ? 0.0f : expf(s - lse[b*seq + i]);
        const float ds = p*(dp - delta[b*seq + i])*scale;
#pragma unroll
        for(int t = 0; t < EPL; ++t)
        {
            gv[t] = fmaf(p, gg[t], gv[t]);
            gk[t] = fmaf(ds, qq[t], gk[t]);
        }
    }
#pragma unroll
    for(int t = 0; t < EPL; ++t)
    {
        const int h = lane*EPL + t;
        if(h < head)
        {
            const float pk = elem_round((gk[t]));
            const float pv = elem_round((gv[t]));
            dK[r*head + h] = f_to_elem(pk + elem_to_f(dK[r*head + h]));
            dV[r*head + h] = f_to_elem(pv + elem_to_f(dV[r*head + h]));
        }
    }
}

template<int EPL>
static int fwd_launch(cudaStream_t s, int seq, int head, Index rows, float scale,
        const elem_t *K, const elem_t *Q, const elem_t *mask, const elem_t *V, float *lse, elem_t *A)
{
    const unsigned blocks = (unsigned)((rows + GEN_WARPS - 1)/GEN_WARPS);
    flash_fwd_generic_kernel<EPL><<<blocks, GEN_WARPS*32, 0, s>>>(seq, head, rows, scale,
            K, Q, mask, V, lse, A);
    return launch_status();
}

int flash_fwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *mask, const elem_t *V, float *lse, elem_t *A)
{
    const Index rows = seq*batch;
    const float scale = 1.0f/sqrtf((float)head);
    const int epl = (int)((head + 31)/32);
    switch(epl)
    {
        case 1: return fwd_launch<1>(s, (int)seq, (int)head, rows, scale, K, Q, mask, V, lse, A);
        case 2: return fwd_launch<2>(s, (int)seq, (int)head, rows, scale, K, Q, mask, V, lse, A);
        case 3: case 4:
            return fwd_launch<4>(s, (int)seq, (int)head, rows, scale, K, Q, mask, V, lse, A);
        default:
            return fwd_launch<GEN_MAX_EPL>(s, (int)seq, (int)head, rows, scale, K, Q, mask, V, lse, A);
    }
}

template<int EPL>
static int bwd_launch(cudaStream_t s, int seq, int head, Index rows, float scale,
        const elem_t *K, const elem_t *Q, const elem_t *V, const elem_t *dA, const elem_t *mask,
        const float *lse, const float *delta, elem_t *dK, elem_t *dQ, elem_t *dV)
{
    const unsigned blocks = (unsigned)((rows + GEN_WARPS - 1)/GEN_WARPS);
    flash_bwd_dq_generic_kernel<EPL><<<blocks, GEN_WARPS*32, 0, s>>>(seq, head, rows,
            scale, K, Q, V, dA, mask, lse, delta, dQ);
    flash_bwd_dkv_generic_kernel<EPL><<<blocks, GEN_WARPS*32, 0, s>>>(seq, head, rows,
            scale, K, Q, V, dA, mask, lse, delta, dK, dV);
    return launch_status(2);
}

int flash_bwd_delta(cudaStream_t s, Index head, Index rows, const elem_t *A, const elem_t *dA,
        float *delta)
{
    flash_bwd_delta_kernel<<<(unsigned)((rows + 7)/8), 256, 0, s>>>((int)head, rows, A, dA, delta);
    return launch_status();
}

int flash_bwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *V, const elem_t *A, const elem_t *dA, const elem_t *mask,
        const float *lse, float *delta, elem_t *dK, elem_t *dQ, elem_t *dV)
{
    const Index rows = seq*batch;
    const float scale = 1.0f/sqrtf((float)head);
    int st = flash_bwd_delta(s, head, rows, A, dA, delta);
    if(st != NNTILE_B200_OK)
    {
        return st;
    }
    const int epl = (int)((head + 31)/32);
    switch(epl)
    {
        case 1: return bwd_launch<1>(s, (int)seq, (int)head, rows, scale, K, Q, V, dA, mask, lse, delta, dK, dQ, dV);
        case 2: return bwd_launch<2>(s, (int)seq, (int)head, rows, scale, K, Q, V, dA, mask, lse, delta, dK, dQ, dV);
        case 3: case 4:
            return bwd_launch<4>(s, (int)seq, (int)head, rows, scale, K, Q, V, dA, mask, lse, delta, dK, dQ, dV);
        default:
            return bwd_launch<GEN_MAX_EPL>(s, (int)seq, (int)head, rows, scale, K, Q, V, dA, mask, lse, delta, dK, dQ, dV);
    }
}

} // inline namespace
} // namespace nb200
