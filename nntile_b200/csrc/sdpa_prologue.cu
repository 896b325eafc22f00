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
// Two forms.  With lead a multiple of 4 a thread transposes an 8-row block of 8 (or,
// for lead = 12, 20 ..., 4) columns in registers (transpose_in_reg_kernel below).
// Otherwise (lead only even) one CTA handles `tp` consecutive (seq, batch) positions at a time: their
// lead*head*tp source elements are one contiguous run, and for every value of
// `lead` the tp*head destination elements are one contiguous run too.  The run is
// staged in shared memory transposed, as tile[lead index][position*head + d], so
// that both global sides move 16 bytes per thread and access: the staging side
// scatters the 8 lead values of a piece with 2-byte shared-memory stores, the other
// side reads 8 consecutive d of one lead index as one 16-byte piece.  The 16-byte
// pieces of a row are XOR-swizzled by the row's group of 8, which keeps the 2-byte
// accesses of a warp (4 row groups x 8 consecutive d) on distinct banks.
//
// Arithmetic matches the reference's kernels bit for bit: the transposition is
// exact, RoPE is round(round(c*a) - round(s*b)) in fp32 (no fused multiply-add,
// as its CPU kernel src/kernel/rope/cpu.cc:24-49 computes it) rounded once to
// bf16, the bias is added in fp32 and rounded once.
#include "common.cuh"

namespace nb200 {

enum : int { PRO_PLAIN = 0, PRO_ROPE = 1, PRO_BIAS = 2 };

constexpr int PRO_THREADS = 256;

// halfword index of element (row n, offset h) in the staged tile; `row` = halfwords
// per row (tp*head), `swz` = 7 when rows hold whole groups of 8 pieces, else 0
__device__ __forceinline__ int pro_at(int n, int h, int row, int swz)
{
    return n*row + ((((h >> 3) ^ ((n >> 3) & swz)) << 3) | (h & 7));
}

__device__ __forceinline__ uint32_t pro_bf16x2(float lo, float hi)
{
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo))
            | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}

template<int MODE>
__global__ void __launch_bounds__(PRO_THREADS)
transpose_in_kernel(int lead, int head, Index npos, int tp, int swz, const bf16 *__restrict__ aux0,
        const bf16 *__restrict__ aux1, const bf16 *__restrict__ src, bf16 *__restrict__ dst)
{
    extern __shared__ __align__(16) uint16_t tile[];
    const int row = tp*head;
    const Index nchunks = (npos + tp - 1)/tp;
    for(Index c = blockIdx.x; c < nchunks; c += gridDim.x)
    {
        const Index pos0 = c*tp;
        const int np = (int)((npos - pos0) < tp ? (npos - pos0) : tp);
        const int rows = np*head;                          // (position, d) pairs in this run
        // ---- stage: contiguous run of rows*lead elements, lead index fastest
        if((lead & 7) == 0)
        {
            const uint4 *g = reinterpret_cast<const uint4 *>(src + pos0*(Index)head*lead);
            const int per = lead >> 3, nvec = rows*per;
            for(int v = threadIdx.x; v < nvec; v += PRO_THREADS)
            {
                const uint4 x = g[v];
                const int h = v/per, n0 = (v - h*per) << 3;
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for(int e = 0; e < 4; ++e)
                {
                    tile[pro_at(n0 + 2*e, h, row, swz)] = (uint16_t)(w[e] & 0xFFFFu);
                    tile[pro_at(n0 + 2*e + 1, h, row, swz)] = (uint16_t)(w[e] >> 16);
                }
            }
        }
        else
        {
            const uint32_t *g = reinterpret_cast<const uint32_t *>(src + pos0*(Index)head*lead);
            const int per = lead >> 1, nw = rows*per;
            for(int v = threadIdx.x; v < nw; v += PRO_THREADS)
            {
                const uint32_t w = g[v];
                const int h = v/per, n0 = (v - h*per) << 1;
                tile[pro_at(n0, h, row, swz)] = (uint16_t)(w & 0xFFFFu);
                tile[pro_at(n0 + 1, h, row, swz)] = (uint16_t)(w >> 16);
            }
        }
        __syncthreads();
        // ---- emit: for every lead index a contiguous run of `rows` elements, 8 per thread
        const int per_row = rows >> 3, total = lead*per_row;
        for(int v = threadIdx.x; v < total; v += PRO_THREADS)
        {
            const int n = v/per_row, h = (v - n*per_row) << 3;
            const uint4 x = *reinterpret_cast<const uint4 *>(&tile[pro_at(n, h, row, swz)]);
            uint32_t w[4] = {x.x, x.y, x.z, x.w};
            if(MODE == PRO_ROPE)
            {
                // (position, d/2) index of the first of this piece's four pairs
                const Index i = (pos0*(Index)head + h) >> 1;
                const uint2 sv = *reinterpret_cast<const uint2 *>(aux0 + i);
                const uint2 cv = *reinterpret_cast<const uint2 *>(aux1 + i);
                const uint32_t sw[2] = {sv.x, sv.y}, cw[2] = {cv.x, cv.y};
#pragma unroll
                for(int e = 0; e < 4; ++e)
                {
                    const uint32_t sb = sw[e >> 1], cb = cw[e >> 1];
                    const float sn = __uint_as_float((e & 1) ? (sb & 0xFFFF0000u) : (sb << 16));
                    const float co = __uint_as_float((e & 1) ? (cb & 0xFFFF0000u) : (cb << 16));
                    const float a = __uint_as_float(w[e] << 16);
                    const float b = __uint_as_float(w[e] & 0xFFFF0000u);
                    w[e] = pro_bf16x2(__fsub_rn(__fmul_rn(co, a), __fmul_rn(sn, b)),
                            __fadd_rn(__fmul_rn(sn, a), __fmul_rn(co, b)));
                }
            }
            else if(MODE == PRO_BIAS)
            {
                // bias[d, n], d fastest; the piece lies inside one position
                const int d = h % head;
                const uint4 bv = *reinterpret_cast<const uint4 *>(aux0 + (Index)n*head + d);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for(int e = 0; e < 4; ++e)
                {
                    w[e] = pro_bf16x2(
                            __fadd_rn(__uint_as_float(w[e] << 16), __uint_as_float(bw[e] << 16)),
                            __fadd_rn(__uint_as_float(w[e] & 0xFFFF0000u),
                                    __uint_as_float(bw[e] & 0xFFFF0000u)));
                }
            }
            *reinterpret_cast<uint4 *>(dst + (Index)n*npos*head + pos0*(Index)head + h) =
                    make_uint4(w[0], w[1], w[2], w[3]);
        }
        __syncthreads();
    }
}

// dst[n, d, pos] = src[d, pos, n]: the inverse layout change.
__global__ void __launch_bounds__(PRO_THREADS)
transpose_out_kernel(int lead, int head, Index npos, int tp, int swz, const bf16 *__restrict__ src,
        bf16 *__restrict__ dst)
{
    extern __shared__ __align__(16) uint16_t tile[];
    const int row = tp*head;
    const Index nchunks = (npos + tp - 1)/tp;
    for(Index c = blockIdx.x; c < nchunks; c += gridDim.x)
    {
        const Index pos0 = c*tp;
        const int np = (int)((npos - pos0) < tp ? (npos - pos0) : tp);
        const int rows = np*head;
        const int per_row = rows >> 3, total = lead*per_row;
        for(int v = threadIdx.x; v < total; v += PRO_THREADS)
        {
            const int n = v/per_row, h = (v - n*per_row) << 3;
            *reinterpret_cast<uint4 *>(&tile[pro_at(n, h, row, swz)]) =
                    *reinterpret_cast<const uint4 *>(src + (Index)n*npos*head + pos0*(Index)head + h);
        }
        __syncthreads();
        if((lead & 7) == 0)
        {
            uint4 *g = reinterpret_cast<uint4 *>(dst + pos0*(Index)head*lead);
            const int per = lead >> 3, nvec = rows*per;
            for(int v = threadIdx.x; v < nvec; v += PRO_THREADS)
            {
                const int h = v/per, n0 = (v - h*per) << 3;
                uint32_t w[4];
#pragma unroll
                for(int e = 0; e < 4; ++e)
                {
                    w[e] = (uint32_t)tile[pro_at(n0 + 2*e, h, row, swz)]
                            | ((uint32_t)tile[pro_at(n0 + 2*e + 1, h, row, swz)] << 16);
                }
                g[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        else
        {
            uint32_t *g = reinterpret_cast<uint32_t *>(dst + pos0*(Index)head*lead);
            const int per = lead >> 1, nw = rows*per;
            for(int v = threadIdx.x; v < nw; v += PRO_THREADS)
            {
                const int h = v/per, n0 = (v - h*per) << 1;
                g[v] = (uint32_t)tile[pro_at(n0, h, row, swz)]
                        | ((uint32_t)tile[pro_at(n0 + 1, h, row, swz)] << 16);
            }
        }
        __syncthreads();
    }
}

// ---- lead a multiple of 4: no staging at all.  The tensor is a [rows = position*head]
// x [lead] matrix to transpose; a thread takes an 8 x 8 block of it as eight 16-byte
// loads (eight consecutive rows, which lie in one position because head is a
// multiple of 8), transposes it in registers with byte permutes and writes eight
// 16-byte pieces, one per lead index (8 x 4 blocks and 8-byte loads when lead is a
// multiple of 4 only).  Consecutive threads take consecutive column
// blocks of the same rows, then the next rows: a warp's loads cover whole 32-byte
// sectors and its stores are runs of at least 128 bytes.
// 16-bit element e of each of the eight row pieces, in row order: CB = 8 (pieces of
// 16 bytes) or 4 (pieces of 8 bytes, for head counts that are multiples of 4 only)
template<int CB> struct ProPiece;
template<> struct ProPiece<8>
{
    typedef uint4 type;
    static __device__ __forceinline__ uint32_t word(const uint4 &v, int i)
    {
        return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
    }
    static __device__ __forceinline__ uint4 make(const uint32_t (&w)[4])
    {
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template<> struct ProPiece<4>
{
    typedef uint2 type;
    static __device__ __forceinline__ uint32_t word(const uint2 &v, int i)
    {
        return i == 0 ? v.x : v.y;
    }
    static __device__ __forceinline__ uint2 make(const uint32_t (&w)[2])
    {
        return make_uint2(w[0], w[1]);
    }
};

// column e of an 8-row block: element e of each of the eight row pieces
template<int CB>
__device__ __forceinline__ uint4 pro_column(const typename ProPiece<CB>::type (&in)[8], int e)
{
    const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
    uint32_t w[4];
#pragma unroll
    for(int k = 0; k < 4; ++k)
    {
        w[k] = __byte_perm(ProPiece<CB>::word(in[2*k], e >> 1), ProPiece<CB>::word(in[2*k + 1], e >> 1),
                sel);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// row r of a CB-column block held as CB pieces of eight rows each
template<int CB>
__device__ __forceinline__ typename ProPiece<CB>::type pro_row(const uint4 (&in)[CB], int r)
{
    const uint32_t sel = (r & 1) ? 0x7632u : 0x5410u;
    uint32_t w[CB/2];
#pragma unroll
    for(int k = 0; k < CB/2; ++k)
    {
        w[k] = __byte_perm(ProPiece<8>::word(in[2*k], r >> 1), ProPiece<8>::word(in[2*k + 1], r >> 1), sel);
    }
    return ProPiece<CB>::make(w);
}

template<int MODE, int CB>
__global__ void __launch_bounds__(PRO_THREADS)
transpose_in_reg_kernel(int lead, int head, Index nrows, const bf16 *__restrict__ aux0,
        const bf16 *__restrict__ aux1, const bf16 *__restrict__ src, bf16 *__restrict__ dst)
{
    typedef typename ProPiece<CB>::type piece_t;
    const int pb = lead/CB;
    const Index items = (nrows >> 3)*pb;
    for(Index v = (Index)blockIdx.x*PRO_THREADS + threadIdx.x; v < items;
            v += (Index)gridDim.x*PRO_THREADS)
    {
        const Index rg = v/pb;
        const int p = (int)(v - rg*pb);
        const Index r0 = rg << 3;
        const piece_t *g = reinterpret_cast<const piece_t *>(src + r0*lead + CB*p);
        piece_t in[8];
#pragma unroll
        for(int r = 0; r < 8; ++r)
        {
            in[r] = g[(Index)r*pb];
        }
        uint32_t sw[2] = {0u, 0u}, cw[2] = {0u, 0u};
        if(MODE == PRO_ROPE)
        {
            // (position, d/2) index of the first of the four pairs of these rows
            const uint2 sv = *reinterpret_cast<const uint2 *>(aux0 + (r0 >> 1));
            const uint2 cv = *reinterpret_cast<const uint2 *>(aux1 + (r0 >> 1));
            sw[0] = sv.x; sw[1] = sv.y; cw[0] = cv.x; cw[1] = cv.y;
        }
#pragma unroll
        for(int e = 0; e < CB; ++e)
        {
            const uint4 col = pro_column<CB>(in, e);
            uint32_t w[4] = {col.x, col.y, col.z, col.w};
            const int n = CB*p + e;
            if(MODE == PRO_ROPE)
            {
#pragma unroll
                for(int q = 0; q < 4; ++q)
                {
                    const uint32_t sb = sw[q >> 1], cb = cw[q >> 1];
                    const float sn = __uint_as_float((q & 1) ? (sb & 0xFFFF0000u) : (sb << 16));
                    const float co = __uint_as_float((q & 1) ? (cb & 0xFFFF0000u) : (cb << 16));
                    const float a = __uint_as_float(w[q] << 16);
                    const float b = __uint_as_float(w[q] & 0xFFFF0000u);
                    w[q] = pro_bf16x2(__fsub_rn(__fmul_rn(co, a), __fmul_rn(sn, b)),
                            __fadd_rn(__fmul_rn(sn, a), __fmul_rn(co, b)));
                }
            }
            else if(MODE == PRO_BIAS)
            {
                // bias[d, n], d fastest
                const int d = (int)(r0 % head);
                const uint4 bv = *reinterpret_cast<const uint4 *>(aux0 + (Index)n*head + d);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for(int q = 0; q < 4; ++q)
                {
                    w[q] = pro_bf16x2(
                            __fadd_rn(__uint_as_float(w[q] << 16), __uint_as_float(bw[q] << 16)),
                            __fadd_rn(__uint_as_float(w[q] & 0xFFFF0000u),
                                    __uint_as_float(bw[q] & 0xFFFF0000u)));
                }
            }
            *reinterpret_cast<uint4 *>(dst + (Index)n*nrows + r0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template<int CB>
__global__ void __launch_bounds__(PRO_THREADS)
transpose_out_reg_kernel(int lead, Index nrows, const bf16 *__restrict__ src, bf16 *__restrict__ dst)
{
    typedef typename ProPiece<CB>::type piece_t;
    const int pb = lead/CB;
    const Index items = (nrows >> 3)*pb;
    for(Index v = (Index)blockIdx.x*PRO_THREADS + threadIdx.x; v < items;
            v += (Index)gridDim.x*PRO_THREADS)
    {
        const Index rg = v/pb;
        const int p = (int)(v - rg*pb);
        const Index r0 = rg << 3;
        uint4 in[CB];
#pragma unroll
        for(int e = 0; e < CB; ++e)
        {
            in[e] = *reinterpret_cast<const uint4 *>(src + (Index)(CB*p + e)*nrows + r0);
        }
        piece_t *g = reinterpret_cast<piece_t *>(dst + r0*lead + CB*p);
#pragma unroll
        for(int r = 0; r < 8; ++r)
        {
            g[(Index)r*pb] = pro_row<CB>(in, r);
        }
    }
}

static unsigned pro_reg_grid(int lead, int cb, Index nrows)
{
    const Index items = (nrows >> 3)*(lead/cb);
    const Index blocks = (items + PRO_THREADS - 1)/PRO_THREADS;
    const Index cap = 148*16;
    return (unsigned)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
}

struct ProPlan
{
    int tp, swz;
    size_t smem;
    unsigned grid;
};

static int pro_check(int64_t lead, int64_t head, int64_t seq, int64_t batch)
{
    if(lead < 0 || head < 0 || seq < 0 || batch < 0) return NNTILE_B200_E_BADARG;
    // two `lead` indices per 32-bit word; a 16-byte piece of 8 head elements must not
    // straddle two positions
    if(lead % 2 != 0 || head % 8 != 0 || lead > 1024 || head > 1024) return NNTILE_B200_E_SHAPE;
    if(seq*batch >= ((int64_t)1 << 40)) return NNTILE_B200_E_SHAPE;
    return NNTILE_B200_OK;
}

static ProPlan pro_plan(int lead, int head, Index npos)
{
    ProPlan p;
    // positions per chunk: about 32 KB of staging, rows of whole groups of 8 pieces
    // (64 elements) when the head size allows it
    int tp = (int)((size_t)32768/((size_t)lead*head*2));
    if(tp < 1) tp = 1;
    if(tp > 16) tp = 16;
    if((Index)tp > npos) tp = (int)npos;
    while(tp > 1 && (tp*head) % 64 != 0) --tp;
    p.tp = tp;
    p.swz = (tp*head) % 64 == 0 ? 7 : 0;
    p.smem = (size_t)lead*tp*head*2;
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
    if(!aligned16(src) || !aligned16(dst) || (sin && (!aligned16(sin) || !aligned16(cos))))
    {
        return NNTILE_B200_E_ALIGN;
    }
    if(lead % 4 == 0)
    {
        const Index nrows = npos*head;
        const int cb = lead % 8 == 0 ? 8 : 4;
        const unsigned grid = pro_reg_grid((int)lead, cb, nrows);
        const bf16 *s0 = (const bf16 *)sin, *c0 = (const bf16 *)cos, *x = (const bf16 *)src;
        bf16 *y = (bf16 *)dst;
        cudaStream_t st_ = as_stream(stream);
        if(sin && cb == 8)
        {
            transpose_in_reg_kernel<PRO_ROPE, 8><<<grid, PRO_THREADS, 0, st_>>>((int)lead, (int)head, nrows, s0, c0, x, y);
        }
        else if(sin)
        {
            transpose_in_reg_kernel<PRO_ROPE, 4><<<grid, PRO_THREADS, 0, st_>>>((int)lead, (int)head, nrows, s0, c0, x, y);
        }
        else if(cb == 8)
        {
            transpose_in_reg_kernel<PRO_PLAIN, 8><<<grid, PRO_THREADS, 0, st_>>>((int)lead, (int)head, nrows, nullptr, nullptr, x, y);
        }
        else
        {
            transpose_in_reg_kernel<PRO_PLAIN, 4><<<grid, PRO_THREADS, 0, st_>>>((int)lead, (int)head, nrows, nullptr, nullptr, x, y);
        }
        return launch_status();
    }
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(sin)
    {
        if(!pro_optin(transpose_in_kernel<PRO_ROPE>, p.smem)) return NNTILE_B200_E_LAUNCH;
        transpose_in_kernel<PRO_ROPE><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>(
                (int)lead, (int)head, npos, p.tp, p.swz, (const bf16 *)sin, (const bf16 *)cos,
                (const bf16 *)src, (bf16 *)dst);
    }
    else
    {
        if(!pro_optin(transpose_in_kernel<PRO_PLAIN>, p.smem)) return NNTILE_B200_E_LAUNCH;
        transpose_in_kernel<PRO_PLAIN><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>(
                (int)lead, (int)head, npos, p.tp, p.swz, nullptr, nullptr, (const bf16 *)src,
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
    if(!aligned16(src) || !aligned16(dst) || !aligned16(bias))
    {
        return NNTILE_B200_E_ALIGN;
    }
    if(lead % 4 == 0)
    {
        const Index nrows = npos*head;
        const int cb = lead % 8 == 0 ? 8 : 4;
        const unsigned grid = pro_reg_grid((int)lead, cb, nrows);
        if(cb == 8)
        {
            transpose_in_reg_kernel<PRO_BIAS, 8><<<grid, PRO_THREADS, 0, as_stream(stream)>>>((int)lead,
                    (int)head, nrows, (const bf16 *)bias, nullptr, (const bf16 *)src, (bf16 *)dst);
        }
        else
        {
            transpose_in_reg_kernel<PRO_BIAS, 4><<<grid, PRO_THREADS, 0, as_stream(stream)>>>((int)lead,
                    (int)head, nrows, (const bf16 *)bias, nullptr, (const bf16 *)src, (bf16 *)dst);
        }
        return launch_status();
    }
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(!pro_optin(transpose_in_kernel<PRO_BIAS>, p.smem)) return NNTILE_B200_E_LAUNCH;
    transpose_in_kernel<PRO_BIAS><<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>((int)lead,
            (int)head, npos, p.tp, p.swz, (const bf16 *)bias, nullptr, (const bf16 *)src, (bf16 *)dst);
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
    if(lead % 4 == 0)
    {
        const Index nrows = npos*head;
        const int cb = lead % 8 == 0 ? 8 : 4;
        const unsigned grid = pro_reg_grid((int)lead, cb, nrows);
        if(cb == 8)
        {
            transpose_out_reg_kernel<8><<<grid, PRO_THREADS, 0, as_stream(stream)>>>((int)lead, nrows,
                    (const bf16 *)src, (bf16 *)dst);
        }
        else
        {
            transpose_out_reg_kernel<4><<<grid, PRO_THREADS, 0, as_stream(stream)>>>((int)lead, nrows,
                    (const bf16 *)src, (bf16 *)dst);
        }
        return launch_status();
    }
    const ProPlan p = pro_plan((int)lead, (int)head, npos);
    if(p.smem > 200*1024) return NNTILE_B200_E_SHAPE;
    if(!pro_optin(transpose_out_kernel, p.smem)) return NNTILE_B200_E_LAUNCH;
    transpose_out_kernel<<<p.grid, PRO_THREADS, p.smem, as_stream(stream)>>>((int)lead, (int)head,
            npos, p.tp, p.swz, (const bf16 *)src, (bf16 *)dst);
    return launch_status();
}
