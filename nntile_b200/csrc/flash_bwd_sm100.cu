// Fused flash-SDPA backward tile task for B200: five tcgen05 MMAs per
// (query block, key block) pair with TMEM accumulators, tiles staged by TMA.
//
// Replaces, for head in {64, 128} and seq a multiple of 128, what
// src/kernel/flash_sdpa_bwd_cudnn/cuda.cc:171-218 does with a cuDNN backward
// graph into scratch followed by three add_inplace passes: gradients of one
// (Q tile, K/V tile) task from the GIVEN A and lse, rounded to elem_t and ADDED
// into dK, dQ, dV.
//
// One CTA owns one block of 128 keys of one batch entry: K and V stay in shared
// memory, dK and dV stay in TMEM for the whole loop over the query blocks that
// see these keys.  Everything is computed transposed (rows = keys):
//   S^T  = K Q^T          (shared x shared, both K-major)
//   dP^T = V dO^T         (shared x shared)
//   P^T  = exp2(S^T*c - lse2), dS^T = P^T o (dP^T - delta)      softmax warps
//   dV  += P^T dO         (P^T from TMEM, where the softmax warps wrote it over
//                          S^T; dO MN-major from shared memory)
//   dK  += dS^T Q         (dS^T from TMEM, written over dP^T; Q MN-major)
//   dQ_i = dS K           (dS^T also written to shared memory by the softmax warps,
//                          read as an MN-major operand; K MN-major)
// dQ_i is added into an fp32 accumulator in global memory with red.add (several
// key blocks contribute to a query row), converted and added into dQ by a small
// epilogue kernel.  TMEM: S^T 128 + dP^T 128 + dV D + dK D columns; for head 128
// that is all 512, so dQ_i reuses the dP^T columns once dK has consumed dS^T (the
// MMA pipe runs in issue order) and the next dP^T waits for the drain warps to
// read dQ_i out.  (Reading dS^T for dK from shared memory instead, so that dQ_i
// could go first, was slower: with both operands of four of the five products in
// shared memory its 128 bytes per clock are the busiest resource of the SM.)
//
// The chip's L2 takes about 21 bytes of fp32 reductions per clock and SM; a
// drain warp that issues its 128 reductions back to back fills the load/store
// queue for 3000 clocks and every shared-memory and TMEM access of the softmax
// warps waits behind them, so the drain issues four at a time on a clock schedule
// just below that rate.
//
// 512 threads: warp 0 TMA producer (K/V right at the start, then Q/dO with the
// softmax statistics through a 2-stage ring), warp 1 MMA issuer, warps 4-7 dQ
// drain, warps 8-15 softmax (two warps per TMEM lane quarter, 64 query columns
// each); during the set-up warp 2 reads the status word and warp 3 compacts the
// class table into the list of query blocks to walk.  dK and dV leave through
// shared memory as TMA element-wise additions ("+=" without reading the old
// values), which is also what lets several CTAs share a dK/dV tile in the
// grouped-query form.
//
// The fp32 dQ accumulator, delta = rowsum(A o dA), lse*log2(e) and the mask
// class table live in the three scratch buffers the reference's tile layer
// hands to every task (they only ever held cuDNN's scratch gradients), so the
// library allocates nothing.  All waits are bounded (sm100.cuh).
#include "flash.cuh"
#include "per_device.hh"
#include "sm100.cuh"

namespace nb200 {
inline namespace NB200_ELEM_NS {

using namespace sm100;

namespace bwd {

// Optional cycle accounting of the roles (build with -DNB200_PROF).
#ifdef NB200_PROF
__device__ unsigned long long g_prof[32];
#define PROF_T(var) const long long var = clock64()
#define PROF_DECL unsigned long long prof_loc[32]; for(int i_ = 0; i_ < 32; ++i_) prof_loc[i_] = 0
#define PROF_ADD(slot, a, b) prof_loc[slot] += (unsigned long long)((b) - (a))
#define PROF_INC(slot) prof_loc[slot] += 1ull
#define PROF_FLUSH if((threadIdx.x >> 5) != 1 || (threadIdx.x & 31) == 0) \
    for(int i_ = 0; i_ < 32; ++i_) if(prof_loc[i_]) atomicAdd(&g_prof[i_], prof_loc[i_])
#else
#define PROF_T(var)
#define PROF_DECL
#define PROF_ADD(slot, a, b)
#define PROF_INC(slot)
#define PROF_FLUSH
#endif

constexpr int BLK = 128;
constexpr int THREADS = 512;
constexpr int RED_PACE = 24, RED_BURST = 4;   // dQ drain: 4 reductions, then wait for the schedule
constexpr int MAX_BLOCKS = 256;      // seq <= 32768
constexpr float LOG2E_F = 1.4426950408889634f;

template<int D>
struct Smem
{
    static constexpr int TILE_BYTES = BLK*D*2;
    uint8_t k[TILE_BYTES];
    uint8_t v[TILE_BYTES];
    uint8_t q[2][TILE_BYTES];
    uint8_t g[2][TILE_BYTES];            // dO
    uint8_t ds[BLK*BLK*2];               // dS^T, [key rows][query cols], swizzled
    float stats[2][2][BLK];              // per Q stage: [0] -lse*log2e, [1] -delta
    uint64_t kv_full;
    uint64_t q_full[2], q_empty[2], g_full[2], g_empty[2];
    uint64_t s_full, dp_full, p_full, ds_full, dq_full, dq_empty, acc_full, dv_full;
    uint32_t tmem_base;
    uint32_t abort_flag;
    int nact;
    uint8_t qlist[MAX_BLOCKS];           // query blocks that see this key block, in order
    uint8_t qcls[MAX_BLOCKS];            // and the class of each (never CLS_SKIP)
};

// delta[r] = -sum_h A[r,h]*dA[r,h];  lse2[r] = -lse[r]*log2(e)  (both are only ever
// used negated by the main kernel)
// Also clears the fp32 dQ accumulator (split at half_rows over two buffers).  head/8
// threads per row, 16 bytes of A and of dA per thread; head is 64 or 128.
__global__ void __launch_bounds__(256)
bwd_prep_kernel(int head, Index rows, Index half_rows, const elem_t *__restrict__ A,
        const elem_t *__restrict__ dA, const float *__restrict__ lse,
        float *__restrict__ delta, float *__restrict__ lse2, float *__restrict__ acc_lo,
        float *__restrict__ acc_hi)
{
    const int tpr = head >> 3;                            // threads per row: 8 or 16
    const Index idx = (Index)blockIdx.x*blockDim.x + threadIdx.x;
    const Index r = idx/tpr;
    const int piece = (int)(idx - r*tpr);
    float acc = 0.0f;
    if(r < rows)
    {
        const uint4 a = *reinterpret_cast<const uint4 *>(A + r*head + 8*piece);
        const uint4 g = *reinterpret_cast<const uint4 *>(dA + r*head + 8*piece);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for(int e = 0; e < 4; ++e)
        {
            acc = fmaf(elem_lo(aw[e]), elem_lo(gw[e]), acc);
            acc = fmaf(elem_hi(aw[e]), elem_hi(gw[e]), acc);
        }
        float4 *z = reinterpret_cast<float4 *>(
                (r < half_rows ? acc_lo + r*head : acc_hi + (r - half_rows)*head) + 8*piece);
        z[0] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        z[1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    // rows never straddle a warp: 32 is a multiple of tpr and blockDim of 32
#pragma unroll
    for(int off = 8; off >= 1; off >>= 1)
    {
        if(off < tpr)
        {
            acc += __shfl_xor_sync(0xffffffffu, acc, off);
        }
    }
    if(r < rows && piece == 0)
    {
        delta[r] = -acc;
        lse2[r] = -lse[r]*LOG2E_F;
    }
}

// dQ[r,h] += elem_t(scale * acc[r,h]); the accumulator is split over two buffers.
__global__ void bwd_dq_finish_kernel(int head, Index rows, Index half_rows, float scale,
        const float *__restrict__ acc_lo, const float *__restrict__ acc_hi,
        elem_t *__restrict__ dQ)
{
    const Index total = rows*head/4, stride = (Index)gridDim.x*blockDim.x;
    for(Index x = (Index)blockIdx.x*blockDim.x + threadIdx.x; x < total; x += stride)
    {
        const Index e = 4*x, r = e/head;
        const float *src = r < half_rows ? acc_lo + e : acc_hi + (e - half_rows*head);
        const float4 a = *reinterpret_cast<const float4 *>(src);
        uint2 old = *reinterpret_cast<const uint2 *>(dQ + e);
        const float o0 = elem_lo(old.x), o1 = elem_hi(old.x);
        const float o2 = elem_lo(old.y), o3 = elem_hi(old.y);
        const float g0 = elem_round(a.x*scale), g1 = elem_round(a.y*scale);
        const float g2 = elem_round(a.z*scale), g3 = elem_round(a.w*scale);
        old.x = pack_elem2(o0 + g0, o1 + g1);
        old.y = pack_elem2(o2 + g2, o3 + g3);
        *reinterpret_cast<uint2 *>(dQ + e) = old;
    }
}

template<int D>
__device__ __forceinline__ void load_tile(uint8_t *dst, const CUtensorMap *map, uint64_t *bar,
        int row)
{
#pragma unroll
    for(int p = 0; p < D/64; ++p)
    {
        tma_load_2d(dst + p*(BLK*128), map, bar, 64*p, row);
    }
}

// The issue helpers build each operand descriptor as (low word of the tile) +
// constant, high word constant (sm100.cuh), so that one MMA costs the issuing
// thread two integer adds.

// C[128 x 128] = A B^T with A, B both [128 rows][D] K-major tiles.
template<int D>
__device__ __forceinline__ void issue_kmajor(uint32_t d_tmem, const uint8_t *a, const uint8_t *b)
{
    constexpr uint32_t idesc = idesc_16(BLK, BLK, 0, 0, ELEM_MMA_FORMAT);
    constexpr uint32_t hi = smem_desc_hi(1024);
    const uint32_t a_lo = smem_desc_lo(smem_u32(a), 16), b_lo = smem_desc_lo(smem_u32(b), 16);
#pragma unroll
    for(int ks = 0; ks < D/16; ++ks)
    {
        const uint32_t off = (uint32_t)(((ks >> 2)*(BLK*128) + (ks & 3)*32) >> 4);
        if(ks == 0)
        {
            mma_ss_c<false>(d_tmem, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi),
                    idesc);
        }
        else
        {
            mma_ss_c<true>(d_tmem, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi),
                    idesc);
        }
    }
}

// C[128 x D] (+)= A B with A = elem_t [128 lanes x 128] in TMEM, stored as two
// 32-column pieces at a_tmem and a_tmem + 64, and B = [128 rows][D] tile read
// MN-major (rows are the contraction index).
template<int D>
__device__ __forceinline__ void issue_ts(uint32_t d_tmem, uint32_t a_tmem, const uint8_t *b,
        bool accumulate)
{
    constexpr uint32_t idesc = idesc_16(BLK, D, 0, 1, ELEM_MMA_FORMAT);
    constexpr uint32_t hi = smem_desc_hi(1024);
    const uint32_t b_lo = smem_desc_lo(smem_u32(b), BLK*128);
    if(accumulate)
    {
        mma_ts_c<true>(d_tmem, a_tmem, smem_desc_join(b_lo, hi), idesc);
    }
    else
    {
        mma_ts_c<false>(d_tmem, a_tmem, smem_desc_join(b_lo, hi), idesc);
    }
#pragma unroll
    for(int ks = 1; ks < BLK/16; ++ks)
    {
        const uint32_t a = a_tmem + (ks < 4 ? 8*ks : 64 + 8*(ks - 4));
        mma_ts_c<true>(d_tmem, a, smem_desc_join(b_lo + (uint32_t)((ks*2048) >> 4), hi), idesc);
    }
}

// dQ[128 q x D] = dS K with dS^T [128 key rows][128 q] in shared memory (MN-major A)
// and K [128 key rows][D] (MN-major B) - or, with the operands swapped at head
// 128, dQ^T[D x 128 q] = K^T dS^T.  Both tiles are read with the keys as the
// contraction index, 16 key rows = 2048 bytes per step.
template<int D>
__device__ __forceinline__ void issue_dq(uint32_t d_tmem, const uint8_t *ds, const uint8_t *k)
{
    constexpr uint32_t idesc = idesc_16(BLK, D, 1, 1, ELEM_MMA_FORMAT);
    constexpr uint32_t hi = smem_desc_hi(1024);
    const uint32_t a_lo = smem_desc_lo(smem_u32(ds), BLK*128);
    const uint32_t b_lo = smem_desc_lo(smem_u32(k), BLK*128);
#pragma unroll
    for(int ks = 0; ks < BLK/16; ++ks)
    {
        const uint32_t off = (uint32_t)((ks*2048) >> 4);
        if(ks == 0)
        {
            mma_ss_c<false>(d_tmem, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi),
                    idesc);
        }
        else
        {
            mma_ss_c<true>(d_tmem, smem_desc_join(a_lo + off, hi), smem_desc_join(b_lo + off, hi),
                    idesc);
        }
    }
}

template<int D>
__global__ void __launch_bounds__(THREADS, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmap_k,
        const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_q,
        const __grid_constant__ CUtensorMap tmap_g, const __grid_constant__ CUtensorMap tmap_dk,
        const __grid_constant__ CUtensorMap tmap_dv, int seq, int batch, int gsz, int kv_group,
        int kv_batch, float scale_log2,
        float scale, const elem_t *__restrict__ mask, const uint8_t *__restrict__ cls_tab,
        const float *__restrict__ delta, const float *__restrict__ lse2,
        float *__restrict__ acc_lo, float *__restrict__ acc_hi, Index half_rows,
        uint32_t *status)
{
    constexpr bool ALIAS = D == 128;     // dQ_i lives in the dP^T columns
    // At head 128 the MMA produces dQ_i^T (lanes = head elements), so that the 32
    // lanes of a drain warp add into 128 contiguous bytes: 8 times fewer L2
    // reduction requests than one 16-byte piece per lane and row.
    constexpr bool DQ_TRANSPOSED = D == 128;
    // The tiles need 1024-byte alignment (128-byte swizzle atoms) and at head 128 the
    // structure fills the 227 KB of a CTA to within 600 bytes, so there is no room
    // for a round-up: the alignment is requested from the toolchain and verified.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    if((smem_u32(smem_raw) & 1023u) != 0u)
    {
        if(threadIdx.x == 0)
        {
            atomicCAS(status, 0u, STATUS_BWD_SMEM_ALIGN);
        }
        return;
    }
    Smem<D> &sm = *reinterpret_cast<Smem<D> *>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblk = seq/BLK;
    int kb, b;                                   // early key blocks see most queries: first
    group_decode(blockIdx.x, nblk, batch, gsz, kb, b);
    const int row_base = b*seq;
    // K, V, dK, dV may be shared by `kv_group` consecutive groups of `kv_batch`
    // entries (grouped-query attention on un-replicated K/V; 1 and `batch`
    // otherwise): the CTAs of a group then add into the same dK / dV tile, which the
    // element-wise TMA additions of the epilogue allow
    const int kv_row_base = ((b % kv_batch) + kv_batch*(b/(kv_batch*kv_group)))*seq;
    volatile uint32_t *abort_flag = &sm.abort_flag;
    PROF_DECL;
    PROF_T(c0);
#ifdef NB200_PROF
    const unsigned long long gt0 = global_timer_ns();
#endif

    if(tid == 0)
    {
        mbar_init(&sm.kv_full, 1);
        for(int i = 0; i < 2; ++i)
        {
            mbar_init(&sm.q_full[i], 1);
            mbar_init(&sm.q_empty[i], 1);
            mbar_init(&sm.g_full[i], 1);
            mbar_init(&sm.g_empty[i], 1);
        }
        mbar_init(&sm.s_full, 1);
        mbar_init(&sm.dp_full, 1);
        mbar_init(&sm.p_full, 256);
        mbar_init(&sm.ds_full, 256);
        mbar_init(&sm.dq_full, 1);
        mbar_init(&sm.dq_empty, 128);
        mbar_init(&sm.acc_full, 1);
        mbar_init(&sm.dv_full, 1);
        fence_mbar_init();
        // K and V of this key block are wanted whatever the class table says: their
        // copies start now, under the set-up of the other warps (a CTA with nothing
        // to do waits for them in the tear-down)
        mbar_arrive_expect_tx(&sm.kv_full, 2*Smem<D>::TILE_BYTES);
        load_tile<D>(sm.k, &tmap_k, &sm.kv_full, kv_row_base + kb*BLK);
        load_tile<D>(sm.v, &tmap_v, &sm.kv_full, kv_row_base + kb*BLK);
        prefetch_tensormap(&tmap_q);
        prefetch_tensormap(&tmap_g);
        prefetch_tensormap(&tmap_dk);
        prefetch_tensormap(&tmap_dv);
    }
    if(warp == 1)
    {
        tmem_alloc(&sm.tmem_base, 512);
    }
    if(warp == 2 && lane == 0)
    {
        // a CTA of this launch that gave up earlier tells the others to skip their work
        sm.abort_flag = *reinterpret_cast<volatile uint32_t *>(status) != 0u ? 1u : 0u;
    }
    if(warp == 3)
    {
        // compact list of the query blocks with anything unmasked against this key
        // block (ballot compaction); the roles below walk the list, not the table
        static_assert(MAX_BLOCKS <= 256, "query block numbers are stored in bytes");
        int count = 0;
        for(int base = 0; base < nblk; base += 32)
        {
            const int qb = base + lane;
            uint8_t c = CLS_SKIP;
            if(qb < nblk)
            {
                c = cls_tab[(size_t)qb*nblk + kb];
            }
            const uint32_t m = __ballot_sync(0xffffffffu, c != CLS_SKIP);
            if(c != CLS_SKIP)
            {
                const int pos = count + __popc(m & ((1u << lane) - 1u));
                sm.qlist[pos] = (uint8_t)qb;
                sm.qcls[pos] = c;
            }
            count += __popc(m);
        }
        if(lane == 0)
        {
            sm.nact = count;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const int nact = sm.abort_flag != 0u ? 0 : sm.nact;
    PROF_T(c1);
    constexpr uint32_t TILE_BYTES = Smem<D>::TILE_BYTES;
    const uint32_t st_tm = tmem, dpt_tm = tmem + 128, dv_tm = tmem + 256, dk_tm = tmem + 256 + D;
    const uint32_t dq_tm = ALIAS ? tmem + 128 : tmem + 384;

    if(warp < 4)
    {
    // control warpgroup: hand registers to the drain warpgroup, which holds a whole
    // dQ_i tile (128 columns) and frees the TMEM columns after one load round, and to
    // the softmax warpgroups.  An increase is only ever served from registers a
    // warpgroup of this CTA gave up, and waits for them without a bound, so released
    // must equal requested: launch 128 x 512 = control 80 x 128 + drain 144 x 128 +
    // softmax 144 x 256.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if(warp == 0)
    {
        // =============================== TMA producer ==========================
        if(lane == 0 && nact > 0)
        {
            bool ok = true;
            int n = 0;
            for(int qi = 0; qi < nact && ok; ++qi)
            {
                const int qb = sm.qlist[qi];
                const int st = n & 1;
                const uint32_t ph = (uint32_t)(n >> 1) & 1u;
                ok = mbar_wait(&sm.q_empty[st], ph ^ 1u, abort_flag);
                if(!ok) break;
                mbar_arrive_expect_tx(&sm.q_full[st], TILE_BYTES + 2*BLK*4);
                load_tile<D>(sm.q[st], &tmap_q, &sm.q_full[st], row_base + qb*BLK);
                bulk_load_1d(sm.stats[st][0], lse2 + (Index)row_base + (Index)qb*BLK, BLK*4,
                        &sm.q_full[st]);
                bulk_load_1d(sm.stats[st][1], delta + (Index)row_base + (Index)qb*BLK, BLK*4,
                        &sm.q_full[st]);
                ok = mbar_wait(&sm.g_empty[st], ph ^ 1u, abort_flag);
                if(!ok) break;
                mbar_arrive_expect_tx(&sm.g_full[st], TILE_BYTES);
                load_tile<D>(sm.g[st], &tmap_g, &sm.g_full[st], row_base + qb*BLK);
                ++n;
            }
            if(!ok)
            {
                atomicCAS(status, 0u, STATUS_BWD_PRODUCER);
            }
        }
    }
    else if(warp == 1)
    {
        // ================================ MMA issuer ===========================
        // (all 32 lanes walk the loop with warp-wide waits; one elected lane issues, so
        // that the operand descriptors are formed in converged code)
        if(nact > 0)
        {
            // Issue order.  The loop-carried chain is
            //   dS^T(n) -> dK(n), dQ(n) -> drain -> dP^T(n+1) -> dS^T(n+1);
            // dV(n+1) is slotted into the drain window and S^T(n+2) behind dP^T(n+1),
            // where the softmax warps are busy with dS^T(n+1), so the tensor pipe
            // has work whenever the chain leaves it idle.
            bool ok = mbar_wait_warp(&sm.kv_full, 0, abort_flag);
            ok = ok && mbar_wait_warp(&sm.q_full[0], 0, abort_flag);
            if(ok)
            {
                tc_fence_after_sync();
                if(elect_one())
                {
                    issue_kmajor<D>(st_tm, sm.k, sm.q[0]);           // S^T(0)
                    tc_commit(&sm.s_full);
                }
                __syncwarp();
            }
            ok = ok && mbar_wait_warp(&sm.g_full[0], 0, abort_flag);
            if(ok)
            {
                tc_fence_after_sync();
                if(elect_one())
                {
                    issue_kmajor<D>(dpt_tm, sm.v, sm.g[0]);          // dP^T(0)
                    tc_commit(&sm.dp_full);
                }
                __syncwarp();
            }
            ok = ok && mbar_wait_warp(&sm.p_full, 0, abort_flag);
            if(ok)
            {
                tc_fence_after_sync();
                if(elect_one())
                {
                    issue_ts<D>(dv_tm, st_tm, sm.g[0], false);       // dV = P^T(0) dO
                    tc_commit(&sm.g_empty[0]);
                    if(nact == 1)
                    {
                        tc_commit(&sm.dv_full);  // dV is complete one step before dK
                    }
                }
                __syncwarp();
            }
            if(ok && nact > 1)
            {
                ok = mbar_wait_warp(&sm.q_full[1], 0, abort_flag);
                if(ok)
                {
                    tc_fence_after_sync();
                    if(elect_one())
                    {
                        issue_kmajor<D>(st_tm, sm.k, sm.q[1]);       // S^T(1)
                        tc_commit(&sm.s_full);
                    }
                    __syncwarp();
                }
            }
            bool s_pending = false;
            for(int n = 0; n < nact && ok; ++n)
            {
                const int st = n & 1, s2 = (n + 1) & 1;
                PROF_T(m0);
                ok = mbar_wait_warp(&sm.ds_full, (uint32_t)n & 1u, abort_flag);
                if(!ok) break;
                tc_fence_after_sync();
                PROF_T(m1);
                if(elect_one())
                {
                    issue_ts<D>(dk_tm, dpt_tm, sm.q[st], n > 0);     // dK += dS^T Q
                    tc_commit(&sm.q_empty[st]);
                }
                __syncwarp();
                if(!ALIAS && n > 0)
                {
                    ok = mbar_wait_warp(&sm.dq_empty, (uint32_t)(n - 1) & 1u, abort_flag);
                    if(!ok) break;
                    tc_fence_after_sync();
                }
                if(elect_one())
                {
                    if(DQ_TRANSPOSED)
                    {
                        issue_dq<D>(dq_tm, sm.k, sm.ds);             // dQ_i^T = K^T dS^T
                    }
                    else
                    {
                        issue_dq<D>(dq_tm, sm.ds, sm.k);             // dQ_i = dS K
                    }
                    tc_commit(&sm.dq_full);
                }
                __syncwarp();
                if(s_pending)
                {
                    ok = mbar_wait_warp(&sm.q_full[s2], (uint32_t)((n + 1) >> 1) & 1u, abort_flag);
                    if(!ok) break;
                    tc_fence_after_sync();
                    if(elect_one())
                    {
                        issue_kmajor<D>(st_tm, sm.k, sm.q[s2]);      // the deferred S^T(n+1)
                        tc_commit(&sm.s_full);
                    }
                    __syncwarp();
                    s_pending = false;
                }
                PROF_T(m2);
#ifdef NB200_PROF
                const bool steady = n >= 2 && n + 2 < nact;
                if(steady)
                {
                PROF_ADD(0, m0, m1);        // MMA: wait for dS^T
                PROF_ADD(1, m1, m2);        // MMA: issue dK, dQ
                PROF_INC(7);
                }
#endif
                if(n + 1 >= nact)
                {
                    if(elect_one())
                    {
                        tc_commit(&sm.acc_full);
                    }
                    __syncwarp();
                    break;
                }
                const uint32_t ph1 = (uint32_t)((n + 1) >> 1) & 1u;
                ok = mbar_wait_warp(&sm.g_full[s2], ph1, abort_flag);
                if(!ok) break;
                PROF_T(m3);
                // dV(n+1) goes first only if P^T(n+1) is already there; otherwise the
                // chain (dP^T) must not wait for it
                bool dv_issued = false;
                if(__all_sync(0xffffffffu, mbar_try_wait(&sm.p_full, (uint32_t)(n + 1) & 1u)))
                {
                    tc_fence_after_sync();
                    if(elect_one())
                    {
                        issue_ts<D>(dv_tm, st_tm, sm.g[s2], true);   // dV += P^T(n+1) dO
                    }
                    __syncwarp();
                    dv_issued = true;
                }
                PROF_T(m4);
                PROF_T(m5);
                if(ALIAS)
                {
                    ok = mbar_wait_warp(&sm.dq_empty, (uint32_t)n & 1u, abort_flag);
                    if(!ok) break;
                    tc_fence_after_sync();
                }
                PROF_T(m6);
                if(elect_one())
                {
                    issue_kmajor<D>(dpt_tm, sm.v, sm.g[s2]);         // dP^T(n+1)
                    tc_commit(&sm.dp_full);
                }
                __syncwarp();
                if(!dv_issued)
                {
                    ok = mbar_wait_warp(&sm.p_full, (uint32_t)(n + 1) & 1u, abort_flag);
                    if(!ok) break;
                    tc_fence_after_sync();
                }
                if(elect_one())
                {
                    if(!dv_issued)
                    {
                        issue_ts<D>(dv_tm, st_tm, sm.g[s2], true);   // dV += P^T(n+1) dO
                    }
                    tc_commit(&sm.g_empty[s2]);
                    if(n + 2 == nact)
                    {
                        tc_commit(&sm.dv_full);
                    }
                }
                __syncwarp();
                PROF_T(m7);
                if(n + 2 < nact)
                {
                    // Q(n+2) reuses the stage dK(n) has just released; if its copy has
                    // not landed yet, S^T(n+2) is issued after the next dK, dQ instead
                    if(__all_sync(0xffffffffu, mbar_try_wait(&sm.q_full[st], (uint32_t)((n + 2) >> 1) & 1u)))
                    {
                        tc_fence_after_sync();
                        if(elect_one())
                        {
                            issue_kmajor<D>(st_tm, sm.k, sm.q[st]);  // S^T(n+2)
                            tc_commit(&sm.s_full);
                        }
                        __syncwarp();
                    }
                    else
                    {
                        s_pending = true;
                    }
                }
                PROF_T(m8);
#ifdef NB200_PROF
                if(steady)
                {
                PROF_ADD(2, m3, m4);        // MMA: wait for P^T(n+1)
                PROF_ADD(3, m4, m5);        // MMA: issue dV
                PROF_ADD(4, m5, m6);        // MMA: wait for the dQ drain
                PROF_ADD(5, m6, m7);        // MMA: issue dP^T
                PROF_ADD(6, m7, m8);        // MMA: wait Q + issue S^T(n+2)
                PROF_ADD(11, m2, m3);       // MMA: wait for dO(n+1)
                }
#endif
            }
            if(!ok && lane == 0)
            {
                atomicCAS(status, 0u, STATUS_BWD_MMA);
            }
        }
    }
    }
    else if(warp < 8)
    {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
        // ================================ dQ drain =============================
        const int r = 32*(warp & 3) + lane;
        const uint32_t src = dq_tm + ((uint32_t)(32*(warp & 3)) << 16);
        bool ok = true;
        int n = 0;
        for(int qi = 0; qi < nact && ok; ++qi)
        {
            const int qb = sm.qlist[qi];
            PROF_T(d0);
            ok = mbar_wait(&sm.dq_full, (uint32_t)n & 1u, abort_flag);
            if(!ok) break;
            tc_fence_after_sync();
            PROF_T(d1);
            if(DQ_TRANSPOSED)
            {
                // TMEM holds dQ_i^T: lane = head element r, column = query.  The whole
                // tile goes into registers in one round, the columns are handed back
                // to the MMA pipe at once, and only then the reductions are issued:
                // one red per query, the 32 lanes of a warp adding 128 contiguous bytes.
                uint32_t o[4][32];
                tmem_ld32(src, o[0]);
                tmem_ld32(src + 32, o[1]);
                tmem_ld32(src + 64, o[2]);
                tmem_ld32(src + 96, o[3]);
                tmem_ld_wait();
                tc_fence_before_sync();
                mbar_arrive(&sm.dq_empty);
                const long long red_t0 = clock64();
#pragma unroll
                for(int cc = 0; cc < BLK/32; ++cc)
                {
                    // the accumulator is split at half_rows, a multiple of 64 rows
                    const Index R0 = (Index)row_base + (Index)qb*BLK + 32*cc;
                    float *dst = (R0 < half_rows ? acc_lo + R0*D : acc_hi + (R0 - half_rows)*D) + r;
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        red_add_f32(dst + (Index)j*D, __uint_as_float(o[cc][j]));
                        if((j % RED_BURST) == RED_BURST - 1)
                        {
                            // stay behind the schedule of one reduction per RED_PACE clocks
                            const long long due = red_t0 + (long long)(32*cc + j + 1)*RED_PACE;
                            while(clock64() < due)
                            {
                                __nanosleep(20);
                            }
                        }
                    }
                }
            }
            else
            {
                const Index R = (Index)row_base + (Index)qb*BLK + r;
                float *dst = R < half_rows ? acc_lo + R*D : acc_hi + (R - half_rows)*D;
#pragma unroll
                for(int cc = 0; cc < D/32; ++cc)
                {
                    uint32_t o[32];
                    tmem_ld32(src + 32*cc, o);
                    tmem_ld_wait();
                    if(cc == D/32 - 1)
                    {
                        tc_fence_before_sync();
                        mbar_arrive(&sm.dq_empty);
                    }
#pragma unroll
                    for(int j = 0; j < 8; ++j)
                    {
                        red_add_v4(dst + 32*cc + 4*j, __uint_as_float(o[4*j]),
                                __uint_as_float(o[4*j + 1]), __uint_as_float(o[4*j + 2]),
                                __uint_as_float(o[4*j + 3]));
                    }
                }
            }
#ifdef NB200_PROF
            if(r == 0 && n >= 2 && n + 2 < nact)
            {
                PROF_T(d2);
                PROF_ADD(8, d0, d1);        // drain: wait for dQ
                PROF_ADD(9, d1, d2);        // drain: TMEM loads + reds
                PROF_INC(10);
            }
#endif
            ++n;
        }
        if(!ok && lane == 0)
        {
            atomicCAS(status, 0u, STATUS_BWD_DRAIN);
        }
    }
    else
    {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
        // ================================= softmax =============================
        const int ts = tid - 256;                     // 0..255
        const int h = ts >> 7;                        // query-column half
        const int r = 32*(warp & 3) + lane;           // key row inside the block
        const uint32_t lane_sel = (uint32_t)(32*(warp & 3)) << 16;
        bool ok = true;
        int n = 0;
        for(int qi = 0; qi < nact && ok; ++qi)
        {
            const int qb = sm.qlist[qi];
            const uint8_t c = sm.qcls[qi];
            // -lse*log2e and -delta of the query block arrive with the Q tile (bulk
            // copies on the same barrier); this thread handles 64 of the 128 queries
            PROF_T(sq);
            ok = mbar_wait(&sm.q_full[n & 1], (uint32_t)(n >> 1) & 1u, abort_flag);
            if(!ok) break;
            const float4 *nl4 = reinterpret_cast<const float4 *>(&sm.stats[n & 1][0][64*h]);
            const float4 *nd4 = reinterpret_cast<const float4 *>(&sm.stats[n & 1][1][64*h]);
            // ---- phase A: P^T = exp2(S^T*c - lse2 [+ bias]) for this thread's 64 query
            // columns, kept as packed elem_t in registers and written over the S^T
            // columns; needs S^T only, so it overlaps the MMAs of the previous block
            PROF_T(s0);
            ok = mbar_wait(&sm.s_full, (uint32_t)n & 1u, abort_flag);
            if(!ok) break;
            tc_fence_after_sync();
            PROF_T(s1);
            uint32_t pk[2][16];                   // [32-column half][packed pair]
            {
                uint32_t s[2][32];
                tmem_ld32(st_tm + lane_sel + 64*h, s[0]);
                tmem_ld32(st_tm + lane_sel + 64*h + 32, s[1]);
                tmem_ld_wait();
                const uint64_t scale2 = pack_f32x2(scale_log2, scale_log2);
#pragma unroll
                for(int c2 = 0; c2 < 2; ++c2)
                {
#pragma unroll
                    for(int j = 0; j < 32; j += 4)
                    {
                        const int qc = 64*h + 32*c2 + j;          // query inside the block
                        const float4 nl = nl4[(32*c2 + j) >> 2];
                        float x[4];
                        unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(s[c2][j]),
                                __uint_as_float(s[c2][j + 1])), scale2, pack_f32x2(nl.x, nl.y)),
                                x[0], x[1]);
                        unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(s[c2][j + 2]),
                                __uint_as_float(s[c2][j + 3])), scale2, pack_f32x2(nl.z, nl.w)),
                                x[2], x[3]);
                        if(c == CLS_CAUSAL)
                        {
#pragma unroll
                            for(int u = 0; u < 4; ++u)
                            {
                                x[u] = r > qc + u ? -CUDART_INF_F : x[u];
                            }
                        }
                        else if(c == CLS_GENERIC)
                        {
#pragma unroll
                            for(int u = 0; u < 4; ++u)
                            {
                                const float bias = elem_to_f(
                                        mask[(size_t)(qb*BLK + qc + u)*seq + (size_t)kb*BLK + r]);
                                x[u] = bias == -CUDART_INF_F ? -CUDART_INF_F
                                                             : fmaf(bias, LOG2E_F, x[u]);
                            }
                        }
                        // all four on the MUFU unit: a cubic on the FMA pipe for part of
                        // them was measured slower (the warps are short of issue slots)
                        const float e2 = ex2(x[2]), e3 = ex2(x[3]);
                        pk[c2][j >> 1] = pack_elem2(ex2(x[0]), ex2(x[1]));
                        pk[c2][(j >> 1) + 1] = pack_elem2(e2, e3);
                    }
                }
            }
            {
                tmem_st16(st_tm + lane_sel + 64*h, pk[0]);
                tmem_st16(st_tm + lane_sel + 64*h + 16, pk[1]);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_full);
            // ---- phase B: dS^T = P^T o (dP^T - delta), to TMEM (for dK) and to shared
            // memory (for dQ); this is the part on the loop-carried chain
            PROF_T(s2);
            ok = mbar_wait(&sm.dp_full, (uint32_t)n & 1u, abort_flag);
            if(!ok) break;
            tc_fence_after_sync();
            PROF_T(s3);
            uint32_t dp2[2][32];
            tmem_ld32(dpt_tm + lane_sel + 64*h, dp2[0]);
            tmem_ld32(dpt_tm + lane_sel + 64*h + 32, dp2[1]);
            tmem_ld_wait();
            PROF_T(b0);
#pragma unroll
            for(int c2 = 0; c2 < 2; ++c2)
            {
                uint32_t pd[16];
                const uint32_t (&dp)[32] = dp2[c2];
#pragma unroll
                for(int j = 0; j < 32; j += 4)
                {
                    const float4 nd = nd4[(32*c2 + j) >> 2];
                    const uint32_t w0 = pk[c2][j >> 1], w1 = pk[c2][(j >> 1) + 1];
                    float d[4];
                    unpack_f32x2(fmul2(pack_f32x2(elem_lo(w0), elem_hi(w0)),
                            fadd2(pack_f32x2(__uint_as_float(dp[j]), __uint_as_float(dp[j + 1])),
                                    pack_f32x2(nd.x, nd.y))), d[0], d[1]);
                    unpack_f32x2(fmul2(pack_f32x2(elem_lo(w1), elem_hi(w1)),
                            fadd2(pack_f32x2(__uint_as_float(dp[j + 2]), __uint_as_float(dp[j + 3])),
                                    pack_f32x2(nd.z, nd.w))), d[2], d[3]);
                    pd[j >> 1] = pack_elem2(d[0], d[1]);
                    pd[(j >> 1) + 1] = pack_elem2(d[2], d[3]);
                }
                tmem_st16(dpt_tm + lane_sel + 64*h + 16*c2, pd);
                // dS^T row r, query columns 64h+32c2 .. +31: four 16-byte pieces of
                // panel h, 128-byte swizzle
                uint8_t *row = sm.ds + h*(BLK*128) + r*128;
#pragma unroll
                for(int i = 0; i < 4; ++i)
                {
                    const int ch = 4*c2 + i;
                    *reinterpret_cast<uint4 *>(row + ((ch ^ (r & 7)) << 4)) =
                            make_uint4(pd[4*i], pd[4*i + 1], pd[4*i + 2], pd[4*i + 3]);
                }
            }
            PROF_T(b1);
            tmem_st_wait();
            fence_proxy_async();
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_full);
#ifdef NB200_PROF
            if(ts == 0 && n >= 2 && n + 2 < nact)
            {
                PROF_T(s4);
                PROF_ADD(22, sq, s0);       // softmax: wait for Q(n) and its statistics
                PROF_ADD(12, s0, s1);       // softmax: wait for S^T
                PROF_ADD(13, s1, s2);       // softmax: phase A
                PROF_ADD(14, s2, s3);       // softmax: wait for dP^T
                PROF_ADD(16, s3, s4);       // softmax: phase B
                PROF_ADD(23, s3, b0);       //   of which TMEM load of dP^T
                PROF_ADD(24, b0, b1);       //   arithmetic, TMEM and shared-memory stores
                PROF_ADD(25, b1, s4);       //   store wait, fences, arrive
                PROF_INC(15);
            }
#endif
            ++n;
        }
        // ---- epilogue: dV (half 0) / dK (half 1) += accumulators ------------------
        // Each warp owns 32 key rows of dV (h = 0) or dK (h = 1).  The gradient is
        // rounded to elem_t and written into the warp's part of the Q stage (dV) or dO
        // stage (dK) that the LAST query block did not use, as 64-column panels with
        // 128-byte rows and the 128-byte swizzle of the tensor maps, and one lane
        // hands the panels to the TMA unit as element-wise elem_t additions into dV /
        // dK: the reference's "+=" without this SM reading the old values or
        // waiting for them.  That stage was last touched by the block before the
        // last one; its hand-back barrier is waited for first.
        PROF_T(e0);
        const int sf = nact & 1;
        if(ok && nact > 0)
        {
            // the last dV product is issued a whole step before the last dK, dQ
            ok = mbar_wait(h == 0 ? &sm.dv_full : &sm.acc_full, 0, abort_flag);
        }
        if(ok && nact >= 2)
        {
            ok = mbar_wait(h == 0 ? &sm.q_empty[sf] : &sm.g_empty[sf],
                    (uint32_t)((nact - 2) >> 1) & 1u, abort_flag);
        }
        ok = __all_sync(0xffffffffu, ok);     // the epilogue is warp-collective
        PROF_T(e1);
        if(ok && nact > 0)
        {
            tc_fence_after_sync();
            constexpr int PANELS = D/64;
            uint8_t *stage = (h == 0 ? sm.q[sf] : sm.g[sf]) + (warp & 3)*(PANELS*4096);
            const uint32_t src = (h == 0 ? dv_tm : dk_tm) + lane_sel;
            const float mult = h == 0 ? 1.0f : scale;
#pragma unroll
            for(int p = 0; p < PANELS; ++p)
            {
                // one 64-column panel per round: pieces 0..7 of the panel's 128-byte rows
                uint32_t o[2][32];
                tmem_ld32(src + 64*p, o[0]);
                tmem_ld32(src + 64*p + 32, o[1]);
                tmem_ld_wait();
                uint8_t *prow = stage + p*4096 + lane*128;
#pragma unroll
                for(int g8 = 0; g8 < 8; ++g8)
                {
                    uint32_t w[4];
#pragma unroll
                    for(int e2 = 0; e2 < 4; ++e2)
                    {
                        w[e2] = pack_elem2(__uint_as_float(o[g8 >> 2][8*(g8 & 3) + 2*e2])*mult,
                                __uint_as_float(o[g8 >> 2][8*(g8 & 3) + 2*e2 + 1])*mult);
                    }
                    *reinterpret_cast<uint4 *>(prow + ((g8 ^ (lane & 7)) << 4)) =
                            make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            fence_proxy_async();
            __syncwarp();
            if(lane == 0)
            {
                const int row0 = kv_row_base + kb*BLK + 32*(warp & 3);
#pragma unroll
                for(int p = 0; p < PANELS; ++p)
                {
                    tma_reduce_add_2d(h == 0 ? &tmap_dv : &tmap_dk, stage + p*4096, 64*p, row0);
                }
                bulk_commit_group();
                bulk_wait_read_all();
            }
        }
        if(!ok && lane == 0)
        {
            atomicCAS(status, 0u, STATUS_BWD_SOFTMAX);
        }
#ifdef NB200_PROF
        if(ts == 0)
        {
            PROF_T(e2);
            PROF_ADD(19, e0, e1);           // epilogue: wait for the last MMAs
            PROF_ADD(20, e1, e2);           // epilogue: read-modify-write of dK, dV
            PROF_ADD(17, c0, e2);           // CTA lifetime seen by a softmax thread
            PROF_ADD(18, c0, c1);           // prologue up to the first __syncthreads
            PROF_INC(21);
        }
#endif
    }
    // ---- tear-down ---------------------------------------------------------------
    PROF_FLUSH;
    if(tid == 0)
    {
        // the K/V copies issued at the start must have landed before the shared
        // memory goes away, also when nobody needed them
        mbar_wait(&sm.kv_full, 0, abort_flag);
    }
    if(*abort_flag != 0u && tid == 0)
    {
        for(int i = 0; i < 64; ++i)
        {
            __nanosleep(1000);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if(warp == 1)
    {
        tmem_dealloc(tmem, 512);
    }
#ifdef NB200_PROF
    if(tid == 0)
    {
        const unsigned long long gt1 = global_timer_ns();
        atomicAdd(&g_prof[26], gt1 - gt0);          // sum of CTA lifetimes (ns)
        atomicMin(&g_prof[27], gt0);                // first CTA start
        atomicMax(&g_prof[28], gt1);                // last CTA end
    }
#endif
}

} // namespace bwd

#if defined(NB200_PROF) && !defined(NB200_FP16)
extern "C" void nntile_b200_debug_prof_bwd(unsigned long long *out32, int reset)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out32, bwd::g_prof, sizeof(unsigned long long)*32);
    if(reset)
    {
        unsigned long long z[32] = {0};
        z[27] = ~0ull;
        cudaMemcpyToSymbol(bwd::g_prof, z, sizeof(z));
    }
}
#endif

size_t bwd_aux_bytes(Index seq, Index batch)
{
    const Index rows = batch*seq, nblk = seq/bwd::BLK;
    return (size_t)(((CLS_OFFSET + nblk*nblk + 255) & ~(Index)255) + 8*rows);
}

bool flash_bwd_sm100_supports(Index seq, Index head, Index batch)
{
    if(!((head == 64 || head == 128) && seq >= bwd::BLK && seq % bwd::BLK == 0
            && seq/bwd::BLK <= bwd::MAX_BLOCKS && batch >= 1 && batch*seq < ((Index)1 << 31)))
    {
        return false;
    }
    // scratch_dV must hold status + class table + delta + lse2
    return bwd_aux_bytes(seq, batch) <= (size_t)(batch*seq*head*2);
}

BwdAux bwd_aux_from_scratch(Index seq, Index batch, void *scratch_dK, void *scratch_dQ,
        void *scratch_dV)
{
    const Index rows = batch*seq, nblk = seq/bwd::BLK;
    uint8_t *sc = static_cast<uint8_t *>(scratch_dV);
    const size_t stats_off = (CLS_OFFSET + (size_t)nblk*nblk + 255) & ~(size_t)255;
    BwdAux aux;
    aux.status = reinterpret_cast<uint32_t *>(sc);
    aux.cls = sc + CLS_OFFSET;
    aux.delta = reinterpret_cast<float *>(sc + stats_off);
    aux.lse2 = aux.delta + rows;
    aux.acc_lo = static_cast<float *>(scratch_dQ);
    aux.acc_hi = static_cast<float *>(scratch_dK);
    aux.half_rows = rows/2;
    aux.phases = BWD_ALL;
    return aux;
}

template<int D>
static int bwd_run(cudaStream_t s, Index seq, Index batch, Index kv_group, Index kv_batch,
        const elem_t *K, const elem_t *Q,
        const elem_t *V, const elem_t *A, const elem_t *dA, const elem_t *mask, const float *lse,
        const BwdAux &aux, elem_t *dK, elem_t *dQ, elem_t *dV)
{
    using namespace bwd;
    const Index rows = batch*seq;
    const int nblk = (int)(seq/BLK);
    const float scale = 1.0f/sqrtf((float)D);
    if(aux.phases & BWD_CLASSIFY)
    {
        const int st = launch_mask_classify(s, (int)seq, mask, aux.cls, aux.status);
        if(st != NNTILE_B200_OK)
        {
            return st;
        }
    }
    if(aux.phases & BWD_PREP)
    {
        bwd_prep_kernel<<<(unsigned)((rows*(D/8) + 255)/256), 256, 0, s>>>(D, rows, aux.half_rows,
                A, dA, lse, aux.delta, aux.lse2, aux.acc_lo, aux.acc_hi);
        if(launch_status() != NNTILE_B200_OK)
        {
            return NNTILE_B200_E_LAUNCH;
        }
    }
    if(aux.phases & BWD_MAIN)
    {
        CUtensorMap tk, tv, tq, tg, tdk, tdv;
        const Index kv_rows = rows/kv_group;
        if(!make_tmap_16_sw128(&tk, K, kv_rows, D, BLK, ELEM_TMAP_TYPE)
                || !make_tmap_16_sw128(&tv, V, kv_rows, D, BLK, ELEM_TMAP_TYPE)
                || !make_tmap_16_sw128(&tq, Q, rows, D, BLK, ELEM_TMAP_TYPE)
                || !make_tmap_16_sw128(&tg, dA, rows, D, BLK, ELEM_TMAP_TYPE)
                || !make_tmap_16_sw128(&tdk, dK, kv_rows, D, 32, ELEM_TMAP_TYPE)
                || !make_tmap_16_sw128(&tdv, dV, kv_rows, D, 32, ELEM_TMAP_TYPE))
        {
            return NNTILE_B200_E_LAUNCH;
        }
        static_assert(sizeof(Smem<D>) <= 232448, "Smem exceeds the 227 KB a CTA can have");
        // The opt-in to more than 48 KB of dynamic shared memory belongs to the kernel
        // ON ONE DEVICE: a process that drives several GPUs needs it on each of them.
        constexpr size_t smem_bytes = sizeof(Smem<D>);
        static PerDeviceOnce optin;
        int dev = -1;
        if(cudaGetDevice(&dev) != cudaSuccess || !optin.ensure(dev, []() {
                return cudaFuncSetAttribute(flash_bwd_kernel<D>,
                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes)
                        == cudaSuccess; }))
        {
            return NNTILE_B200_E_LAUNCH;
        }
        // Q, K, V, dO, dK, dV (elem_t) and the fp32 dQ accumulator of one batch entry
        const int gsz = l2_group_size(batch, (size_t)seq*D*(2*6 + 4));
        flash_bwd_kernel<D><<<(unsigned)(nblk*batch), THREADS, smem_bytes, s>>>(tk, tv, tq, tg,
                tdk, tdv, (int)seq, (int)batch, gsz, (int)kv_group, (int)kv_batch, scale*LOG2E_F,
                scale, mask, aux.cls, aux.delta, aux.lse2, aux.acc_lo, aux.acc_hi, aux.half_rows,
                aux.status);
        if(launch_status() != NNTILE_B200_OK)
        {
            return NNTILE_B200_E_LAUNCH;
        }
    }
    if(aux.phases & BWD_FINISH)
    {
        bwd_dq_finish_kernel<<<grid_for(rows*D/4, 256), 256, 0, s>>>(D, rows, aux.half_rows, scale,
                aux.acc_lo, aux.acc_hi, dQ);
        return launch_status();
    }
    return NNTILE_B200_OK;
}

int flash_bwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *V, const elem_t *A, const elem_t *dA, const elem_t *mask,
        const float *lse, const BwdAux &aux, elem_t *dK, elem_t *dQ, elem_t *dV, Index kv_group,
        Index kv_batch)
{
    if(kv_group < 1 || kv_batch < 1 || batch % (kv_group*kv_batch) != 0 || !aux.status || !aux.cls
            || !aux.delta || !aux.lse2 || !aux.acc_lo || !aux.acc_hi)
    {
        return NNTILE_B200_E_BADARG;
    }
    return head == 128
            ? bwd_run<128>(s, seq, batch, kv_group, kv_batch, K, Q, V, A, dA, mask, lse, aux,
                    dK, dQ, dV)
            : bwd_run<64>(s, seq, batch, kv_group, kv_batch, K, Q, V, A, dA, mask, lse, aux,
                    dK, dQ, dV);
}

} // inline namespace
} // namespace nb200
