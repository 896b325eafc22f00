// Split-KV decode attention: one new query token per (batch, query head) against
// a KV cache, the cache streamed from HBM exactly once.
//
// The kernel is HBM-bound (2 bytes moved per 4*group flops), so the design goal
// is bytes in flight, not math rate:
//   - every K and V row is fetched with coalesced 128-bit loads straight into
//     registers, already in the operand layout of the warp-level bf16 MMA
//     (m16n8k16, fp32 accumulate) - no shared-memory staging, no shuffles in the
//     inner loop;
//   - the `group` query heads that share a KV head ride in the M dimension of the
//     same MMA, so the cache is read once for all of them (the reference
//     replicates K and V `group` times and re-reads them,
//     wrappers/python/nntile/model/llama_attention.py:533-585);
//   - the cache length is cut into chunks; one CTA (4 warps, 16 key rows per warp
//     step) owns one chunk of one (batch, kv head) and keeps an online
//     max / sum-exp per query head in registers (quad shuffles only); chunk
//     results are merged by log-sum-exp, the arithmetic of
//     src/kernel/accumulate_attn_output/cuda.cu:43-71.
//   - 16 warps per SM x 8 KB of loads in flight per warp keep > 100 KB per SM in
//     flight, well above the ~35 KB that HBM latency x bandwidth asks for.
//
// Layouts (reference: include/nntile/graph/kv_cache.hh:38-39 and
// wrappers/python/nntile/layer/cache_utils.py:117-144): q/out are
// [head, 1, batch, group, kv_heads], caches are [head, max_seq, batch, kv_heads],
// Fortran order, i.e. every (batch, kv head) owns a row-major [max_seq][head]
// block.
#include "common.cuh"

namespace nb200 {

constexpr int DEC_WARPS = 4;
constexpr int DEC_ROWS_PER_STEP = 16;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
            : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
        uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i)
{
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// One CTA = one chunk of the cache of one (batch, kv head); all `group` query
// heads at once.  D is the head size (64 or 128), group <= 8.
//
// Fragment bookkeeping (n = lane/4, t = lane%4).  The dot product over the head
// dimension does not care in which order the head elements are visited, so the
// 16-byte piece that lane (n, t) loads from key row n (elements 8c..8c+7 with
// c = t + 4j) feeds TWO k-steps of the MMA: words 0,1 are the (k=2t.., k=2t+8..)
// operands of step 2j, words 2,3 those of step 2j+1.  The query fragments are
// gathered once with the same element order.  For P.V the key index is the MMA's
// k dimension; lane (n, t) loads the 16-byte piece n (+8 per 64 head elements)
// of key rows 2t, 2t+1, 2t+8, 2t+9 and a byte permute pairs up the two rows.
template<int D>
__global__ void __launch_bounds__(DEC_WARPS*32, 3)
decode_splitkv_kernel(int length, int max_seq, int batch, int group, int rows_per_cta,
        float scale_log2, const bf16 *__restrict__ q, const bf16 *__restrict__ Kc,
        const bf16 *__restrict__ Vc, float *__restrict__ part_o,
        float *__restrict__ part_lse, int nsplit)
{
    constexpr int KSTEPS = D/16;     // MMA k-steps over the head dimension
    constexpr int JN = D/32;         // 16-byte pieces per lane per key row
    constexpr int HH = D/64;         // 64-element halves of the head dimension
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = lane >> 2, t = lane & 3;
    const int split = blockIdx.x;
    const int unit = blockIdx.y;                 // = kvh*batch + b
    const int b = unit % batch, kvh = unit/batch;
    const int row_begin = split*rows_per_cta;
    const int row_end = min(length, row_begin + rows_per_cta);

    const bf16 *Kb = Kc + (size_t)unit*max_seq*D;
    const bf16 *Vb = Vc + (size_t)unit*max_seq*D;

    // Query fragments for head n of the group (zero rows beyond the group).
    uint32_t qa[KSTEPS][2];
    {
        const bf16 *qrow = q + ((size_t)(kvh*group + min(n, group - 1))*batch + b)*D;
#pragma unroll
        for(int j = 0; j < JN; ++j)
        {
            uint4 v = *reinterpret_cast<const uint4 *>(qrow + 8*(t + 4*j));
            if(n >= group)
            {
                v = make_uint4(0u, 0u, 0u, 0u);
            }
            qa[2*j][0] = v.x;
            qa[2*j][1] = v.y;
            qa[2*j + 1][0] = v.z;
            qa[2*j + 1][1] = v.w;
        }
    }

    float acc[HH][8][4];
#pragma unroll
    for(int hh = 0; hh < HH; ++hh)
#pragma unroll
        for(int e = 0; e < 8; ++e)
#pragma unroll
            for(int x = 0; x < 4; ++x)
                acc[hh][e][x] = 0.0f;
    float top = -CUDART_INF_F, sum = 0.0f;      // per query head n, log2 domain

    for(int r0 = row_begin + warp*DEC_ROWS_PER_STEP; r0 < row_end;
            r0 += DEC_WARPS*DEC_ROWS_PER_STEP)
    {
        // ---- issue every load of this step (rows clamped into the valid part)
        const int last = length - 1;
        uint4 kreg[2][JN];
#pragma unroll
        for(int blk = 0; blk < 2; ++blk)
        {
            const int row = min(r0 + 8*blk + n, last);
#pragma unroll
            for(int j = 0; j < JN; ++j)
            {
                kreg[blk][j] = ldg_stream(Kb + (size_t)row*D + 8*(t + 4*j));
            }
        }
        uint4 vreg[4][HH];
#pragma unroll
        for(int role = 0; role < 4; ++role)
        {
            const int row = min(r0 + 2*t + (role & 1) + 8*(role >> 1), last);
#pragma unroll
            for(int hh = 0; hh < HH; ++hh)
            {
                vreg[role][hh] = ldg_stream(Vb + (size_t)row*D + 8*(n + 8*hh));
            }
        }
        // ---- S = q K^T for 16 keys: two 16x8 blocks
        float s[2][4];
#pragma unroll
        for(int blk = 0; blk < 2; ++blk)
        {
            s[blk][0] = s[blk][1] = s[blk][2] = s[blk][3] = 0.0f;
#pragma unroll
            for(int j = 0; j < JN; ++j)
            {
                mma_bf16_16816(s[blk], qa[2*j][0], 0u, qa[2*j][1], 0u,
                        kreg[blk][j].x, kreg[blk][j].y);
                mma_bf16_16816(s[blk], qa[2*j + 1][0], 0u, qa[2*j + 1][1], 0u,
                        kreg[blk][j].z, kreg[blk][j].w);
            }
        }
        // lane holds head n, keys r0 + 8*blk + 2t + {0,1}
        float p[2][2];
        float step_top = -CUDART_INF_F;
#pragma unroll
        for(int blk = 0; blk < 2; ++blk)
#pragma unroll
            for(int x = 0; x < 2; ++x)
            {
                const int row = r0 + 8*blk + 2*t + x;
                p[blk][x] = row < row_end ? s[blk][x]*scale_log2 : -CUDART_INF_F;
                step_top = fmaxf(step_top, p[blk][x]);
            }
        step_top = fmaxf(step_top, __shfl_xor_sync(0xffffffffu, step_top, 1));
        step_top = fmaxf(step_top, __shfl_xor_sync(0xffffffffu, step_top, 2));
        const float ntop = fmaxf(top, step_top);     // finite: row r0 is valid
        const float shrink = exp2f(top - ntop);
        float psum = 0.0f;
#pragma unroll
        for(int blk = 0; blk < 2; ++blk)
#pragma unroll
            for(int x = 0; x < 2; ++x)
            {
                p[blk][x] = exp2f(p[blk][x] - ntop);
                psum += p[blk][x];
            }
        sum = sum*shrink + psum;
        top = ntop;
        const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]);
        const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]);
        // ---- O = O*shrink + P V
#pragma unroll
        for(int hh = 0; hh < HH; ++hh)
        {
#pragma unroll
            for(int e = 0; e < 8; ++e)
            {
                acc[hh][e][0] *= shrink;
                acc[hh][e][1] *= shrink;
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(word_of(vreg[0][hh], e >> 1),
                        word_of(vreg[1][hh], e >> 1), sel);
                const uint32_t b1 = __byte_perm(word_of(vreg[2][hh], e >> 1),
                        word_of(vreg[3][hh], e >> 1), sel);
                mma_bf16_16816(acc[hh][e], pa0, 0u, pa2, 0u, b0, b1);
            }
        }
    }

    // ---- merge the warps of the CTA (log-sum-exp weights) -------------------
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    __shared__ float o_s[DEC_WARPS][8][D];
    __shared__ float top_s[DEC_WARPS][8], sum_s[DEC_WARPS][8];
    if(t == 0)
    {
        top_s[warp][n] = top;
        sum_s[warp][n] = sum;
    }
#pragma unroll
    for(int hh = 0; hh < HH; ++hh)
#pragma unroll
        for(int e = 0; e < 8; ++e)
        {
            o_s[warp][n][8*(2*t + 8*hh) + e] = acc[hh][e][0];
            o_s[warp][n][8*(2*t + 1 + 8*hh) + e] = acc[hh][e][1];
        }
    __syncthreads();
    for(int x = threadIdx.x; x < group*D; x += DEC_WARPS*32)
    {
        const int g = x/D, d = x - g*D;
        float big = -CUDART_INF_F;
#pragma unroll
        for(int w = 0; w < DEC_WARPS; ++w)
        {
            big = fmaxf(big, top_s[w][g]);
        }
        float den = 0.0f, num = 0.0f;
#pragma unroll
        for(int w = 0; w < DEC_WARPS; ++w)
        {
            const float wgt = sum_s[w][g] > 0.0f ? exp2f(top_s[w][g] - big) : 0.0f;
            den += wgt*sum_s[w][g];
            num += wgt*o_s[w][g][d];
        }
        const size_t slot = ((size_t)unit*nsplit + split)*group + g;
        part_o[slot*D + d] = den > 0.0f ? num/den : 0.0f;
        if(d == 0)
        {
            part_lse[slot] = den > 0.0f ? big + log2f(den) : -CUDART_INF_F;
        }
    }
}

// Generic variant: any head <= 256, one query head per CTA row (the cache is
// re-read once per head of the group), CUDA-core dot products.
template<int EPL>
__global__ void __launch_bounds__(DEC_WARPS*32)
decode_generic_kernel(int D, int length, int max_seq, int batch, int group,
        int rows_per_cta, float scale_log2, const bf16 *__restrict__ q,
        const bf16 *__restrict__ Kc, const bf16 *__restrict__ Vc,
        float *__restrict__ part_o, float *__restrict__ part_lse, int nsplit)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x;
    const int qh = blockIdx.y;                    // = (kvh*group + g)*batch + b
    const int b = qh % batch, kvh = qh/(batch*group);
    const size_t cache = ((size_t)kvh*batch + b)*max_seq*D;
    const int row_begin = split*rows_per_cta;
    const int row_end = min(length, row_begin + rows_per_cta);
    float qv[EPL], o[EPL];
#pragma unroll
    for(int x = 0; x < EPL; ++x)
    {
        const int h = lane*EPL + x;
        qv[x] = h < D ? __bfloat162float(q[(size_t)qh*D + h]) : 0.0f;
        o[x] = 0.0f;
    }
    float top = -CUDART_INF_F, sum = 0.0f;
    for(int r = row_begin + warp; r < row_end; r += DEC_WARPS)
    {
        float part = 0.0f, kv[EPL];
#pragma unroll
        for(int x = 0; x < EPL; ++x)
        {
            const int h = lane*EPL + x;
            kv[x] = h < D ? __bfloat162float(Kc[cache + (size_t)r*D + h]) : 0.0f;
            part = fmaf(qv[x], kv[x], part);
        }
        const float s = warp_sum(part)*scale_log2;
        const float ntop = fmaxf(top, s);
        const float shrink = exp2f(top - ntop), p = exp2f(s - ntop);
        sum = sum*shrink + p;
        top = ntop;
#pragma unroll
        for(int x = 0; x < EPL; ++x)
        {
            const int h = lane*EPL + x;
            const float v = h < D ? __bfloat162float(Vc[cache + (size_t)r*D + h]) : 0.0f;
            o[x] = o[x]*shrink + p*v;
        }
    }
    __shared__ float o_s[DEC_WARPS][256];
    __shared__ float top_s[DEC_WARPS], sum_s[DEC_WARPS];
    if(lane == 0)
    {
        top_s[warp] = top;
        sum_s[warp] = sum;
    }
#pragma unroll
    for(int x = 0; x < EPL; ++x)
    {
        const int h = lane*EPL + x;
        if(h < D)
        {
            o_s[warp][h] = o[x];
        }
    }
    __syncthreads();
    for(int d = threadIdx.x; d < D; d += DEC_WARPS*32)
    {
        float big = -CUDART_INF_F;
        for(int w = 0; w < DEC_WARPS; ++w)
        {
            big = fmaxf(big, top_s[w]);
        }
        float den = 0.0f, num = 0.0f;
        for(int w = 0; w < DEC_WARPS; ++w)
        {
            const float wgt = sum_s[w] > 0.0f ? exp2f(top_s[w] - big) : 0.0f;
            den += wgt*sum_s[w];
            num += wgt*o_s[w][d];
        }
        const size_t slot = (size_t)qh*nsplit + split;
        part_o[slot*D + d] = den > 0.0f ? num/den : 0.0f;
        if(d == 0)
        {
            part_lse[slot] = den > 0.0f ? big + log2f(den) : -CUDART_INF_F;
        }
    }
}

// Merge the chunks of one query head: one warp per (unit, g).
// part_o[(unit*nsplit + split)*group + g][D], part_lse likewise (log2 domain).
__global__ void decode_merge_kernel(int D, int nsplit, int group, int batch, int heads_total,
        const float *__restrict__ part_o, const float *__restrict__ part_lse,
        bf16 *__restrict__ out, float *__restrict__ lse_out)
{
    const int lane = threadIdx.x & 31;
    const int w = blockIdx.x*(blockDim.x >> 5) + (threadIdx.x >> 5);
    if(w >= heads_total)
    {
        return;
    }
    const int unit = w/group, g = w - unit*group;
    const int b = unit % batch, kvh = unit/batch;
    float big = -CUDART_INF_F;
    for(int s = 0; s < nsplit; ++s)
    {
        big = fmaxf(big, part_lse[((size_t)unit*nsplit + s)*group + g]);
    }
    float den = 0.0f;
    for(int s = 0; s < nsplit; ++s)
    {
        const float l = part_lse[((size_t)unit*nsplit + s)*group + g];
        den += l > -CUDART_INF_F ? exp2f(l - big) : 0.0f;
    }
    const size_t qh = ((size_t)kvh*group + g)*batch + b;
    for(int d = lane; d < D; d += 32)
    {
        float num = 0.0f;
        for(int s = 0; s < nsplit; ++s)
        {
            const size_t slot = ((size_t)unit*nsplit + s)*group + g;
            const float l = part_lse[slot];
            if(l > -CUDART_INF_F)
            {
                num += exp2f(l - big)*part_o[slot*D + d];
            }
        }
        out[qh*D + d] = __float2bfloat16_rn(den > 0.0f ? num/den : 0.0f);
    }
    if(lane == 0 && lse_out)
    {
        lse_out[qh] = den > 0.0f ? (big + log2f(den))*LN2 : -CUDART_INF_F;
    }
}

struct DecodePlan
{
    int rows_per_cta, nsplit;
    bool fast;
    size_t bytes;
};

static DecodePlan decode_plan(Index head, Index length, Index batch, Index group,
        Index kv_heads)
{
    DecodePlan p;
    p.fast = (head == 64 || head == 128) && group >= 1 && group <= 8;
    // Chunks per cache unit.  Two things cost: a CTA's fixed part (prologue, the
    // exposed latency of its first loads, the partial result it writes: worth about
    // 600 key rows of streaming) and a last wave of CTAs that leaves SMs idle (148 SMs
    // x 3 resident CTAs).  Every candidate is scored as waves x (rows per chunk + 600)
    // and the cheapest wins.  Measured on config 5's cache length (8192) this picks
    // 4 chunks at 512 units (0.36 ms, 0.92 of the copy bandwidth), 3 at 256 and 128
    // units, 6 at 64 units (58 us against 105 us with the former "about 2048 CTAs"
    // rule) - the per-GPU shares of config 5 on 1, 2, 4 and 8 GPUs.
    // The fast kernel shares a chunk among the query heads of a group, the generic
    // one runs one CTA row per query head.
    const Index units = p.fast ? batch*kv_heads : batch*group*kv_heads;
    const Index resident = 148*3;
    Index max_split = (length + 255)/256;                // at least 256 keys per chunk
    if(max_split > 64) max_split = 64;
    if(max_split < 1) max_split = 1;
    Index nsplit = 1, best = -1;
    for(Index n = 1; n <= max_split; ++n)
    {
        Index r = (length + n - 1)/n;
        r = (r + 63)/64*64;
        const Index waves = (units*n + resident - 1)/resident;
        const Index cost = waves*(r + 600);
        if(best < 0 || cost < best)
        {
            best = cost;
            nsplit = n;
        }
    }
    Index rows = (length + nsplit - 1)/nsplit;
    rows = (rows + 63)/64*64;                            // whole steps of the 4 warps
    p.rows_per_cta = (int)rows;
    p.nsplit = (int)((length + rows - 1)/rows);
    if(p.nsplit < 1) p.nsplit = 1;
    const size_t heads = (size_t)batch*group*kv_heads;
    p.bytes = heads*p.nsplit*(size_t)(head + 1)*sizeof(float);
    return p;
}

} // namespace nb200

using namespace nb200;

extern "C" size_t nntile_b200_decode_sdpa_workspace_bytes(int64_t head, int64_t length,
        int64_t batch, int64_t group, int64_t kv_heads)
{
    if(head <= 0 || length <= 0 || batch <= 0 || group <= 0 || kv_heads <= 0)
    {
        return 0;
    }
    return decode_plan(head, length, batch, group, kv_heads).bytes;
}

extern "C" int nntile_b200_decode_sdpa_bf16(nntile_b200_stream_t stream, int64_t head,
        int64_t max_seq, int64_t length, int64_t batch, int64_t group, int64_t kv_heads,
        const void *q, const void *Kcache, const void *Vcache, void *out, float *lse_out,
        void *workspace, size_t workspace_bytes)
{
    if(head < 0 || max_seq < 0 || length < 0 || batch < 0 || group < 0 || kv_heads < 0
            || length > max_seq)
    {
        return NNTILE_B200_E_BADARG;
    }
    if(head == 0 || batch == 0 || group == 0 || kv_heads == 0)
    {
        return NNTILE_B200_OK;
    }
    if(length == 0 || head > 256 || batch*group*kv_heads > 65535)
    {
        return NNTILE_B200_E_SHAPE;     // softmax over an empty cache is undefined
    }
    if(!q || !Kcache || !Vcache || !out || !workspace)
    {
        return NNTILE_B200_E_BADARG;
    }
    const DecodePlan plan = decode_plan(head, length, batch, group, kv_heads);
    if(workspace_bytes < plan.bytes)
    {
        return NNTILE_B200_E_SCRATCH;
    }
    if(!aligned16(workspace) || (plan.fast && (!aligned16(q) || !aligned16(Kcache)
            || !aligned16(Vcache))))
    {
        return NNTILE_B200_E_ALIGN;
    }
    cudaStream_t s = as_stream(stream);
    const size_t heads = (size_t)batch*group*kv_heads;
    float *part_o = static_cast<float *>(workspace);
    float *part_lse = part_o + heads*plan.nsplit*(size_t)head;
    const float scale_log2 = LOG2E/sqrtf((float)head);
    const bf16 *qp = (const bf16 *)q, *kp = (const bf16 *)Kcache, *vp = (const bf16 *)Vcache;
    if(plan.fast)
    {
        dim3 grid(plan.nsplit, (unsigned)(batch*kv_heads));
        if(head == 128)
        {
            decode_splitkv_kernel<128><<<grid, DEC_WARPS*32, 0, s>>>((int)length,
                    (int)max_seq, (int)batch, (int)group, plan.rows_per_cta, scale_log2,
                    qp, kp, vp, part_o, part_lse, plan.nsplit);
        }
        else
        {
            decode_splitkv_kernel<64><<<grid, DEC_WARPS*32, 0, s>>>((int)length,
                    (int)max_seq, (int)batch, (int)group, plan.rows_per_cta, scale_log2,
                    qp, kp, vp, part_o, part_lse, plan.nsplit);
        }
        if(launch_status() != NNTILE_B200_OK) return NNTILE_B200_E_LAUNCH;
        decode_merge_kernel<<<(unsigned)((heads + 3)/4), 128, 0, s>>>((int)head,
                plan.nsplit, (int)group, (int)batch, (int)heads, part_o, part_lse,
                (bf16 *)out, lse_out);
        return launch_status();
    }
    dim3 grid(plan.nsplit, (unsigned)heads);
    const int epl = (int)((head + 31)/32);
#define NB200_DEC_GEN(E) decode_generic_kernel<E><<<grid, DEC_WARPS*32, 0, s>>>((int)head, \
        (int)length, (int)max_seq, (int)batch, (int)group, plan.rows_per_cta, scale_log2, \
        qp, kp, vp, part_o, part_lse, plan.nsplit)
    if(epl <= 1) NB200_DEC_GEN(1);
    else if(epl <= 2) NB200_DEC_GEN(2);
    else if(epl <= 4) NB200_DEC_GEN(4);
    else NB200_DEC_GEN(8);
#undef NB200_DEC_GEN
    if(launch_status() != NNTILE_B200_OK) return NNTILE_B200_E_LAUNCH;
    // every query head is its own unit here: group 1, "batch" = all heads
    decode_merge_kernel<<<(unsigned)((heads + 3)/4), 128, 0, s>>>((int)head, plan.nsplit, 1,
            (int)heads, (int)heads, part_o, part_lse, (bf16 *)out, lse_out);
    return launch_status();
}

// ---------------------------------------------------------------------------
// Decode without a caller-provided workspace
// ---------------------------------------------------------------------------
// Some hosts of this library have no way to obtain device memory for the
// chunk-merge workspace: a StarPU codelet body (or any task-runtime worker
// callback) runs where cudaMalloc is off limits - it would serialise the whole
// device and bypass the runtime's memory accounting - and the reference's decode
// path has no scratch handle to lend because this operation does not exist
// there; a plain C host may simply hold device pointers it was given and no
// allocator at all.  For them the workspace below is part of the library image:
// a fixed array in device memory that every GPU which loads the library keeps
// until the process exits.
//
// In host code `g_decode_scratch` is only a stand-in for the symbol, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked
// once per device with that device current.
constexpr size_t DECODE_SCRATCH_BYTES = (size_t)32 << 20;       // 32 MiB per GPU
constexpr int DECODE_MAX_DEVICES = 64;
static __device__ __align__(256) unsigned char g_decode_scratch[DECODE_SCRATCH_BYTES];

static void *g_decode_scratch_addr[DECODE_MAX_DEVICES];
static std::atomic<int> g_decode_scratch_state[DECODE_MAX_DEVICES];   // 0 unset, 1 ready

// Device address of the scratch array on the current device, or nullptr.
static void *decode_scratch_for_current_device()
{
    int dev = -1;
    if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= DECODE_MAX_DEVICES)
    {
        return nullptr;
    }
    if(g_decode_scratch_state[dev].load(std::memory_order_acquire) == 1)
    {
        return g_decode_scratch_addr[dev];
    }
    void *ptr = nullptr;
    if(cudaGetSymbolAddress(&ptr, g_decode_scratch) != cudaSuccess || ptr == nullptr)
    {
        return nullptr;
    }
    // two threads racing here both obtain the same address for this device
    g_decode_scratch_addr[dev] = ptr;
    g_decode_scratch_state[dev].store(1, std::memory_order_release);
    return ptr;
}

extern "C" size_t nntile_b200_decode_sdpa_noalloc_max_bytes(void)
{
    return DECODE_SCRATCH_BYTES;
}

extern "C" int nntile_b200_decode_sdpa_noalloc_bf16(nntile_b200_stream_t stream,
        int64_t head, int64_t max_seq, int64_t length, int64_t batch, int64_t group,
        int64_t kv_heads, const void *q, const void *Kcache, const void *Vcache, void *out,
        float *lse_out)
{
    if(head > 0 && length > 0 && batch > 0 && group > 0 && kv_heads > 0
            && nntile_b200_decode_sdpa_workspace_bytes(head, length, batch, group, kv_heads)
                    > DECODE_SCRATCH_BYTES)
    {
        return NNTILE_B200_E_SCRATCH;      // problem too large for the built-in array
    }
    void *scratch = decode_scratch_for_current_device();
    if(scratch == nullptr)
    {
        return NNTILE_B200_E_DEVICE;
    }
    // Every chunk slot the merge step reads is written by the chunk kernel of the
    // same call first, so nothing in the array has to start at zero.
    return nntile_b200_decode_sdpa_bf16(stream, head, max_seq, length, batch, group,
            kv_heads, q, Kcache, Vcache, out, lse_out, scratch, DECODE_SCRATCH_BYTES);
}

// ------------------------------------------------------------------ cache append
// cache[:, cache_len : cache_len + new_seq, b, kh] = src[:, :, b, kh] for every
// (batch entry, kv head): per unit one contiguous run of head*new_seq elements.
namespace nb200 {

__global__ void __launch_bounds__(256)
kv_append_kernel(bool vec16, Index run_bytes, Index src_unit_bytes, Index dst_unit_bytes,
        Index dst_off_bytes, const uint8_t *__restrict__ src, uint8_t *__restrict__ dst)
{
    const uint8_t *s = src + (Index)blockIdx.y*src_unit_bytes;
    uint8_t *d = dst + (Index)blockIdx.y*dst_unit_bytes + dst_off_bytes;
    const Index stride = (Index)gridDim.x*blockDim.x;
    const Index first = (Index)blockIdx.x*blockDim.x + threadIdx.x;
    if(vec16)
    {
        for(Index i = first; i < run_bytes/16; i += stride)
        {
            reinterpret_cast<uint4 *>(d)[i] = reinterpret_cast<const uint4 *>(s)[i];
        }
    }
    else
    {
        for(Index i = first; i < run_bytes/2; i += stride)
        {
            reinterpret_cast<uint16_t *>(d)[i] = reinterpret_cast<const uint16_t *>(s)[i];
        }
    }
}

} // namespace nb200

extern "C" int nntile_b200_kv_cache_append_bf16(nntile_b200_stream_t stream, int64_t head,
        int64_t max_seq, int64_t batch, int64_t kv_heads, int64_t cache_len, int64_t new_seq,
        const void *src, void *cache)
{
    using namespace nb200;
    if(head < 1 || max_seq < 1 || batch < 1 || kv_heads < 1 || cache_len < 0 || new_seq < 0
            || cache_len + new_seq > max_seq)
    {
        return NNTILE_B200_E_BADARG;        // the append would run past the cache
    }
    if(batch*kv_heads > 65535)
    {
        return NNTILE_B200_E_SHAPE;
    }
    if(new_seq == 0)
    {
        return NNTILE_B200_OK;
    }
    if(!src || !cache)
    {
        return NNTILE_B200_E_BADARG;
    }
    if((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(cache)) & 1)
    {
        return NNTILE_B200_E_ALIGN;
    }
    const Index run = head*new_seq*2, unit = head*max_seq*2, off = head*cache_len*2;
    const bool vec16 = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(cache)
            | (uintptr_t)run | (uintptr_t)unit | (uintptr_t)off) & 15) == 0;
    const unsigned bx = (unsigned)std::min<Index>(64, std::max<Index>(1, run/16/256));
    kv_append_kernel<<<dim3(bx, (unsigned)(batch*kv_heads)), 256, 0,
            static_cast<cudaStream_t>(stream)>>>(vec16, run, run, unit, off,
            static_cast<const uint8_t *>(src), static_cast<uint8_t *>(cache));
    return launch_status();
}
