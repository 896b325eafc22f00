// Fused flash-SDPA forward tile task for B200: tcgen05 MMA with TMEM
// accumulators, Q/K/V staged by TMA, online max / sum-exp in registers, and the
// log-sum-exp merge into the running (lse, A) fused into the epilogue.
//
// Replaces, for head in {64, 128} and seq a multiple of 128, what
// src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:145-202 does with a cuDNN graph, a
// scratch copy of the tile result and accumulate_attn_output
// (src/kernel/accumulate_attn_output/cuda.cu:28-113).
//
// Work decomposition.  One CTA owns two 128-row query tiles of one batch entry
// (one (batch, head) slice) and walks the 128-key blocks that at least one of
// them needs.  384 threads (three warpgroups) in three roles; the control
// warpgroup hands most of its registers to the softmax warpgroups (setmaxnreg):
//   warp 0      TMA producer: the two Q tiles right at the start (before the
//               block list exists), then K and V blocks through two 2-stage
//               rings (64-column panels, 128-byte swizzle)
//   warp 1      MMA issuer: S_t = Q_t K^T (operands in shared memory) and
//               O_t += P_t V (P_t read from TMEM, V MN-major from shared memory);
//               owns the TMEM allocation (512 columns: S_0 S_1 O_0 O_1).  The whole
//               warp walks the loop and one elected lane issues: in converged code
//               the descriptors stay in uniform registers, which makes a group of
//               8 MMAs about 40 % cheaper to issue than from a lone thread
//   warps 4-11  two softmax groups of 128 threads, one per query tile, one thread
//               per query row: tcgen05.ld of the S row, bias, running max with a
//               lazy rescale of O (only when the max grows by more than 2^8),
//               exp2, elem_t P written back into the S columns, and at the end the
//               normalisation, the merge with the stored (lse, A) and the store
//               (staged through shared memory; a TMA store when nothing is merged).
// During the set-up warp 1 allocates TMEM, warp 2 reads the status word and
// warp 3 compacts the class table into the list of key blocks to walk.
// While one group is busy with exponentials the tensor pipe works for the other
// tile (PV_0, QK_0', PV_1, QK_1' ...), so MUFU and MMA overlap.
//
// The additive mask is a general bias in the reference.  A small pre-pass
// classifies every 128x128 block of it as all-zero, all -inf, exact causal
// diagonal or generic; -inf blocks are never loaded or multiplied, zero blocks
// never read the mask, diagonal blocks compare indices, generic blocks add the
// bias from global memory.  The class table lives in the scratch buffer the
// reference's tile layer provides to every task, so nothing is allocated here.
//
// Every mbarrier wait is bounded (sm100.cuh); a wait that gives up sets a status
// word at the start of the scratch buffer and the CTA tears down normally.
#include "flash.cuh"
#include "per_device.hh"
#include "sm100.cuh"

namespace nb200 {
inline namespace NB200_ELEM_NS {

using namespace sm100;

namespace fwd {

// Optional cycle accounting of the roles (build with -DNB200_PROF): sums over all
// CTAs of the cycles one softmax thread and the MMA thread spend in each phase.
#ifdef NB200_PROF
__device__ unsigned long long g_prof[16];
#define PROF_T(var) const long long var = clock64()
#define PROF_ADD(slot, a, b) \
    do { if((threadIdx.x & 31) == 0) atomicAdd(&g_prof[slot], (unsigned long long)((b) - (a))); } while(0)
#else
#define PROF_T(var)
#define PROF_ADD(slot, a, b)
#endif

constexpr int BLK = 128;             // query rows per tile and keys per block
constexpr int THREADS = 384;         // 3 warpgroups: control, softmax 0, softmax 1
constexpr int KV_STAGES = 2;
constexpr int MAX_BLOCKS = 512;      // seq <= 65536
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr float LN2_F = 0.6931471805599453f;
constexpr float RESCALE_STEP = 8.0f;

// ------------------------------------------------------------ mask classifier
// grid (key block, query block), 256 threads; also clears the status word when one
// is given.
__global__ void __launch_bounds__(256)
mask_classify_kernel(int seq, int nblk, const elem_t *__restrict__ mask, uint8_t *cls,
        uint32_t *status)
{
    const int kb = blockIdx.x, qb = blockIdx.y;
    int zero = 1, ninf = 1, causal = 1;
#pragma unroll
    for(int i = 0; i < 8; ++i)
    {
        const int u = threadIdx.x + 256*i;
        const int row = u >> 4, c16 = u & 15;
        const uint4 v = *reinterpret_cast<const uint4 *>(
                mask + (size_t)(qb*BLK + row)*seq + kb*BLK + c16*8);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for(int e = 0; e < 8; ++e)
        {
            const uint32_t bits = (w[e >> 1] >> (16*(e & 1))) & 0xFFFFu;
            const bool is_zero = (bits & 0x7FFFu) == 0u, is_ninf = bits == ELEM_NINF_BITS;
            zero &= is_zero;
            ninf &= is_ninf;
            causal &= (c16*8 + e > row) ? is_ninf : is_zero;
        }
    }
    zero = __syncthreads_and(zero);
    ninf = __syncthreads_and(ninf);
    causal = __syncthreads_and(causal);
    if(threadIdx.x == 0)
    {
        cls[(size_t)qb*nblk + kb] =
                zero ? CLS_ZERO : ninf ? CLS_SKIP : causal ? CLS_CAUSAL : CLS_GENERIC;
        if(kb == 0 && qb == 0 && status != nullptr)
        {
            *status = 0u;
        }
    }
}

// ------------------------------------------------------------- shared storage
template<int D>
struct Smem
{
    static constexpr int TILE_BYTES = BLK*D*2;
    uint8_t q[2][TILE_BYTES];
    uint8_t k[KV_STAGES][TILE_BYTES];
    uint8_t v[KV_STAGES][TILE_BYTES];
    uint64_t q_full[2];
    uint64_t k_full[KV_STAGES], k_empty[KV_STAGES];
    uint64_t v_full[KV_STAGES], v_empty[KV_STAGES];
    uint64_t s_full[2], p_full[2], o_full[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    int nproc;
    int nact[2];
    uint16_t list[MAX_BLOCKS];       // key blocks to walk, in order
    uint8_t cls[2][MAX_BLOCKS];      // class of list[it] for tile 0 / tile 1
};

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

// S_t = Q_t K^T: D/16 k-steps, both operands K-major in 64-column panels.  The
// issuing thread passes the low descriptor words of the two tiles; every step
// only adds a constant to them.
template<int D>
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_lo, uint32_t k_lo)
{
    constexpr uint32_t idesc = idesc_16(BLK, BLK, 0, 0, ELEM_MMA_FORMAT);
    constexpr uint32_t hi = smem_desc_hi(1024);
#pragma unroll
    for(int ks = 0; ks < D/16; ++ks)
    {
        const uint32_t off = (uint32_t)(((ks >> 2)*(BLK*128) + (ks & 3)*32) >> 4);
        if(ks == 0)
        {
            mma_ss_c<false>(d_tmem, smem_desc_join(q_lo + off, hi), smem_desc_join(k_lo + off, hi),
                    idesc);
        }
        else
        {
            mma_ss_c<true>(d_tmem, smem_desc_join(q_lo + off, hi), smem_desc_join(k_lo + off, hi),
                    idesc);
        }
    }
}

// O_t (+)= P_t V, half of the 8 k-steps of 16 keys: P from TMEM (8 columns per
// step), V MN-major: 16 key rows = 2048 bytes per step (the next 64 head columns,
// 16 KB away, are the leading offset inside v_lo).
template<int D, int HALF>
__device__ __forceinline__ void issue_pv(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_lo,
        bool accumulate)
{
    constexpr uint32_t idesc = idesc_16(BLK, D, 0, 1, ELEM_MMA_FORMAT);
    constexpr uint32_t hi = smem_desc_hi(1024);
#pragma unroll
    for(int k4 = 0; k4 < BLK/32; ++k4)
    {
        const int ks = 4*HALF + k4;
        const uint64_t vd = smem_desc_join(v_lo + (uint32_t)((ks*2048) >> 4), hi);
        if(HALF == 0 && k4 == 0)
        {
            if(accumulate)
            {
                mma_ts_c<true>(d_tmem, p_tmem + 8*ks, vd, idesc);
            }
            else
            {
                mma_ts_c<false>(d_tmem, p_tmem + 8*ks, vd, idesc);
            }
        }
        else
        {
            mma_ts_c<true>(d_tmem, p_tmem + 8*ks, vd, idesc);
        }
    }
}

// TEST = the instantiation behind nntile_b200_test_arm_wait_timeout: waits give up
// after WAIT_LIMIT_TEST_NS and the producer withholds its first K copy, so that one
// wait runs out and the failure report can be checked.  Never launched otherwise.
template<int D, bool TEST>
__global__ void __launch_bounds__(THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
        const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
        const __grid_constant__ CUtensorMap tmap_a,
        int seq, int batch, int gsz, int kv_group, int kv_batch, float scale_log2,
        const elem_t *__restrict__ mask, uint32_t *status, const uint8_t *__restrict__ cls_tab,
        float *__restrict__ lse, elem_t *__restrict__ A)
{
    extern __shared__ uint8_t smem_raw[];
    Smem<D> &sm = *reinterpret_cast<Smem<D> *>(
            (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblk = seq/BLK;
    const int npairs = (nblk + 1)/2;
    int unit, b;
    group_decode(blockIdx.x, npairs, batch, gsz, unit, b);
    const int pair = npairs - 1 - unit;                         // heavy (late) rows first
    const int qb0 = 2*pair, qb1 = 2*pair + 1;
    const bool has1 = qb1 < nblk;
    volatile uint32_t *abort_flag = &sm.abort_flag;
    constexpr uint64_t LIMIT = TEST ? WAIT_LIMIT_TEST_NS : WAIT_LIMIT_NS;

    // ---- set-up: barriers, TMEM, list of key blocks ---------------------------
    if(tid == 0)
    {
        for(int i = 0; i < 2; ++i)
        {
            mbar_init(&sm.q_full[i], 1);
            mbar_init(&sm.s_full[i], 1);
            mbar_init(&sm.p_full[i], 4);                // one arrival per softmax warp
            mbar_init(&sm.o_full[i], 1);
        }
        for(int i = 0; i < KV_STAGES; ++i)
        {
            mbar_init(&sm.k_full[i], 1);
            mbar_init(&sm.k_empty[i], 1);
            mbar_init(&sm.v_full[i], 1);
            mbar_init(&sm.v_empty[i], 1);
        }
        fence_mbar_init();
        // The two Q tiles are wanted whatever the class table says (a tile without
        // any unmasked block is rare): their copies start now, under the set-up of
        // the other warps, and the tear-down waits for them in any case.
        mbar_arrive_expect_tx(&sm.q_full[0], Smem<D>::TILE_BYTES);
        load_tile<D>(sm.q[0], &tmap_q, &sm.q_full[0], b*seq + qb0*BLK);
        if(has1)
        {
            mbar_arrive_expect_tx(&sm.q_full[1], Smem<D>::TILE_BYTES);
            load_tile<D>(sm.q[1], &tmap_q, &sm.q_full[1], b*seq + qb1*BLK);
        }
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
        prefetch_tensormap(&tmap_a);
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
        // compact the key blocks at least one tile needs (ballot compaction)
        int count = 0, n0 = 0, n1 = 0;
        for(int base = 0; base < nblk; base += 32)
        {
            const int kb = base + lane;
            uint8_t c0 = CLS_SKIP, c1 = CLS_SKIP;
            if(kb < nblk)
            {
                c0 = cls_tab[(size_t)qb0*nblk + kb];
                c1 = has1 ? cls_tab[(size_t)qb1*nblk + kb] : (uint8_t)CLS_SKIP;
            }
            const bool need = c0 != CLS_SKIP || c1 != CLS_SKIP;
            const uint32_t m = __ballot_sync(0xffffffffu, need);
            if(need)
            {
                const int pos = count + __popc(m & ((1u << lane) - 1u));
                sm.list[pos] = (uint16_t)kb;
                sm.cls[0][pos] = c0;
                sm.cls[1][pos] = c1;
            }
            count += __popc(m);
            n0 += __popc(__ballot_sync(0xffffffffu, c0 != CLS_SKIP));
            n1 += __popc(__ballot_sync(0xffffffffu, c1 != CLS_SKIP));
        }
        if(lane == 0)
        {
            sm.nproc = count;
            sm.nact[0] = n0;
            sm.nact[1] = n1;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;
    const int nproc = sm.abort_flag != 0u ? 0 : sm.nproc;
    constexpr uint32_t TILE_BYTES = Smem<D>::TILE_BYTES;
    const int row_base = b*seq;                   // first row of this batch entry
    // K and V may be shared by `kv_group` consecutive groups of `kv_batch` entries
    // (grouped-query attention on un-replicated K/V; 1 and `batch` otherwise)
    const int kv_row_base = ((b % kv_batch) + kv_batch*(b/(kv_batch*kv_group)))*seq;

    if(warp < 4)
    {
    // control warpgroup: give registers away, then producer / MMA issuer / idle.
    // An increase is only ever served from registers a warpgroup of this CTA gave
    // up, and waits for them without a bound, so released must equal requested:
    // launch 168 x 384 = control 72 x 128 + softmax 216 x 256 (at 56 the
    // issuing thread spills and at 208 the softmax rows do; both cost several percent).
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if(warp == 0)
    {
        // =============================== TMA producer ==========================
        if(lane == 0 && nproc > 0)
        {
            bool ok = true;
            for(int it = 0; it < nproc && ok; ++it)
            {
                const int st = it % KV_STAGES;
                const uint32_t ph = (uint32_t)(it/KV_STAGES) & 1u;
                const int krow = kv_row_base + (int)sm.list[it]*BLK;
                ok = mbar_wait<LIMIT>(&sm.k_empty[st], ph ^ 1u, abort_flag);
                if(!ok) break;
                if(!(TEST && it == 0))
                {
                    mbar_arrive_expect_tx(&sm.k_full[st], TILE_BYTES);
                    load_tile<D>(sm.k[st], &tmap_k, &sm.k_full[st], krow);
                }
                ok = mbar_wait<LIMIT>(&sm.v_empty[st], ph ^ 1u, abort_flag);
                if(!ok) break;
                mbar_arrive_expect_tx(&sm.v_full[st], TILE_BYTES);
                load_tile<D>(sm.v[st], &tmap_v, &sm.v_full[st], krow);
            }
            if(!ok)
            {
                atomicCAS(status, 0u, STATUS_FWD_PRODUCER);
            }
        }
    }
    else if(warp == 1)
    {
        // ================================ MMA issuer ===========================
        // (all 32 lanes: waits are warp-wide, the tcgen05 instructions go out from one
        // elected lane)
        if(nproc > 0)
        {
            bool ok = true;
            const uint32_t s_tm[2] = {tmem, tmem + 128};
            const uint32_t o_tm[2] = {tmem + 256, tmem + 256 + D};
            // low descriptor words of every operand tile (K-major: leading offset
            // unused; MN-major V: next 64 head columns one 16 KB panel away)
            const uint32_t q_lo[2] = {smem_desc_lo(smem_u32(sm.q[0]), 16),
                                      smem_desc_lo(smem_u32(sm.q[1]), 16)};
            // stage s of K / V: low word of stage 0 + s*STAGE_LO (no indexed local arrays:
            // everything this thread keeps must stay in registers)
            const uint32_t k_lo0 = smem_desc_lo(smem_u32(sm.k[0]), 16);
            const uint32_t v_lo0 = smem_desc_lo(smem_u32(sm.v[0]), BLK*128);
            constexpr uint32_t STAGE_LO = (uint32_t)(Smem<D>::TILE_BYTES >> 4);
            const int nact_r[2] = {sm.nact[0], sm.nact[1]};
            int qk_done[2] = {-1, -1};          // last iteration whose QK_t was issued
            int n_pv[2] = {0, 0};               // PV steps issued per tile
            int k_waited = -1, k_released = -1;
            uint32_t p_phase[2] = {0, 0};
#pragma unroll
            for(int t = 0; t < 2; ++t)
            {
                if(nact_r[t] > 0)
                {
                    ok = mbar_wait_warp<LIMIT>(&sm.q_full[t], 0, abort_flag);
                }
            }
            // cls_other: class of the same block for the other tile
            auto qk = [&](int t, int it, uint8_t cls_other) -> bool
            {
                const int st = it % KV_STAGES;
                if(it > k_waited)
                {
                    if(!mbar_wait_warp<LIMIT>(&sm.k_full[st], (uint32_t)(it/KV_STAGES) & 1u, abort_flag))
                    {
                        return false;
                    }
                    k_waited = it;
                    tc_fence_after_sync();
                }
                qk_done[t] = it;
                // release the K stage once every tile that needs this block has issued
                const int o = t ^ 1;
                const bool release = it > k_released && (cls_other == CLS_SKIP || qk_done[o] >= it);
                const uint32_t k_lo = k_lo0 + (uint32_t)st*STAGE_LO;
                if(elect_one())
                {
                    issue_qk<D>(s_tm[t], q_lo[t], k_lo);
                    tc_commit(&sm.s_full[t]);
                    if(release)
                    {
                        tc_commit(&sm.k_empty[st]);
                    }
                }
                __syncwarp();
                if(release)
                {
                    k_released = it;
                }
                return true;
            };
            // classes of the current and the next block, read once per block
            uint8_t cur[2] = {sm.cls[0][0], sm.cls[1][0]};
            for(int it = 0; it < nproc && ok; ++it)
            {
                const int st = it % KV_STAGES;
                uint8_t nxt[2] = {CLS_SKIP, CLS_SKIP};
                if(it + 1 < nproc)
                {
                    nxt[0] = sm.cls[0][it + 1];
                    nxt[1] = sm.cls[1][it + 1];
                }
    #pragma unroll
            for(int t = 0; t < 2; ++t)
                {
                    if(cur[t] != CLS_SKIP && qk_done[t] < it)
                    {
                        ok = qk(t, it, cur[t ^ 1]);
                    }
                }
                if(!ok) break;
                ok = mbar_wait_warp<LIMIT>(&sm.v_full[st], (uint32_t)(it/KV_STAGES) & 1u, abort_flag);
                const int last_t = cur[1] != CLS_SKIP ? 1 : 0;
                const uint32_t v_lo = v_lo0 + (uint32_t)st*STAGE_LO;
    #pragma unroll
            for(int t = 0; t < 2; ++t)
                {
                    if(cur[t] == CLS_SKIP)
                    {
                        continue;
                    }
                    PROF_T(mt2);
                    ok = mbar_wait_warp<LIMIT>(&sm.p_full[t], p_phase[t], abort_flag);
                    if(!ok) break;
                    p_phase[t] ^= 1u;
                    tc_fence_after_sync();
                    PROF_T(mt3);
                    ++n_pv[t];
                    const bool last_pv = n_pv[t] == nact_r[t];
                    if(elect_one())
                    {
                        issue_pv<D, 0>(o_tm[t], s_tm[t], v_lo, n_pv[t] > 1);
                        issue_pv<D, 1>(o_tm[t], s_tm[t], v_lo, true);
                        if(t == last_t)
                        {
                            tc_commit(&sm.v_empty[st]);
                        }
                        if(last_pv)
                        {
                            tc_commit(&sm.o_full[t]);
                        }
                    }
                    __syncwarp();
                    PROF_T(mt4);
                    PROF_ADD(10, mt2, mt3);     // issuing warp: wait for P
                    PROF_ADD(11, mt3, mt4);     // issue 8 PV steps
#ifdef NB200_PROF
                    if(lane == 0) atomicAdd(&g_prof[12], 1ull);
#endif
                    if(!last_pv && nxt[t] != CLS_SKIP)
                    {
                        ok = qk(t, it + 1, nxt[t ^ 1]);
                    }
                }
                cur[0] = nxt[0];
                cur[1] = nxt[1];
            }
            if(!ok && lane == 0)
            {
                atomicCAS(status, 0u, STATUS_FWD_MMA);
            }
        }
    }
    }
    else
    {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        // ============================= softmax groups ==========================
        const int t = (warp - 4) >> 2;                    // query tile of this group
        const int r = 32*(warp & 3) + lane;               // row inside the tile
        const uint32_t lane_sel = (uint32_t)(32*(warp & 3)) << 16;
        const uint32_t s_tm = tmem + 128*t + lane_sel;
        const uint32_t o_tm = tmem + 256 + D*t + lane_sel;
        const int qb = t == 0 ? qb0 : qb1;
        const int nact = sm.nact[t];
        float m_used = -CUDART_INF_F, l = 0.0f;
        int n = 0;
        bool ok = true;
        uint32_t s_phase = 0;
        // the stored lse of this row is only needed by the epilogue: fetch it now
        float lse_old = 0.0f;
        if(nact > 0)
        {
            lse_old = lse[(size_t)b*seq + (size_t)qb*BLK + r];
        }
        asm volatile("" : "+f"(lse_old));
        for(int it = 0; it < nproc && ok && n < nact; ++it)
        {
            const uint8_t c = sm.cls[t][it];
            if(c == CLS_SKIP)
            {
                continue;
            }
            PROF_T(pt0);
            ok = mbar_wait<LIMIT>(&sm.s_full[t], s_phase, abort_flag);
            if(!ok) break;
            s_phase ^= 1u;
            tc_fence_after_sync();
            PROF_T(pt1);
            uint32_t s[4][32];
            tmem_ld32(s_tm, s[0]);
            tmem_ld32(s_tm + 32, s[1]);
            tmem_ld32(s_tm + 64, s[2]);
            tmem_ld32(s_tm + 96, s[3]);
            tmem_ld_wait();
            PROF_T(pt2);
            // ---- bias; x = s*scale_log2 + bias*log2e is formed lazily below ------
            float top_raw;
            if(c == CLS_GENERIC)
            {
                top_raw = -CUDART_INF_F;
                const elem_t *mrow = mask + (size_t)(qb*BLK + r)*seq + (size_t)sm.list[it]*BLK;
#pragma unroll
                for(int g = 0; g < 16; ++g)
                {
                    const uint4 v = *reinterpret_cast<const uint4 *>(mrow + 8*g);
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for(int e = 0; e < 8; ++e)
                    {
                        const float bias = (e & 1) ? elem_hi(w[e >> 1]) : elem_lo(w[e >> 1]);
                        const float x = fmaf(__uint_as_float(s[g >> 2][8*(g & 3) + e]), scale_log2,
                                bias*LOG2E_F);
                        s[g >> 2][8*(g & 3) + e] = __float_as_uint(x);
                        top_raw = fmaxf(top_raw, x);
                    }
                }
            }
            else
            {
                if(c == CLS_CAUSAL)
                {
#pragma unroll
                    for(int j = 0; j < 128; ++j)
                    {
                        if(j > r)
                        {
                            s[j >> 5][j & 31] = __float_as_uint(-CUDART_INF_F);
                        }
                    }
                }
                // four independent chains of three-input max
                float t0 = -CUDART_INF_F, t1 = t0, t2 = t0, t3 = t0;
#pragma unroll
                for(int q4 = 0; q4 < 4; ++q4)
                {
#pragma unroll
                    for(int j = 0; j < 32; j += 8)
                    {
                        t0 = fmax3(t0, __uint_as_float(s[q4][j]), __uint_as_float(s[q4][j + 1]));
                        t1 = fmax3(t1, __uint_as_float(s[q4][j + 2]), __uint_as_float(s[q4][j + 3]));
                        t2 = fmax3(t2, __uint_as_float(s[q4][j + 4]), __uint_as_float(s[q4][j + 5]));
                        t3 = fmax3(t3, __uint_as_float(s[q4][j + 6]), __uint_as_float(s[q4][j + 7]));
                    }
                }
                top_raw = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
            }
            const float mul = c == CLS_GENERIC ? 1.0f : scale_log2;
            const float m_blk = top_raw*mul;               // -inf stays -inf
            PROF_T(pt3);
            // ---- lazy rescale ----------------------------------------------------
            const bool grow = m_blk > m_used + RESCALE_STEP;   // true on the first finite block
            const float m_new = grow ? m_blk : m_used;
            // (the exponential of the correction only where a row of the warp grows: the
            // MUFU queue is full of the other tile's work most of the time)
            float alpha = 1.0f;
            const bool any_grow = __any_sync(0xffffffffu, grow);
            if(any_grow)
            {
                alpha = grow ? ex2(m_used - m_new) : 1.0f;
            }
            if(n > 0 && any_grow)
            {
#pragma unroll
                for(int cc = 0; cc < D/32; ++cc)
                {
                    uint32_t o[32];
                    tmem_ld32(o_tm + 32*cc, o);
                    tmem_ld_wait();
#pragma unroll
                    for(int j = 0; j < 32; ++j)
                    {
                        o[j] = __float_as_uint(__uint_as_float(o[j])*alpha);
                    }
                    tmem_st32(o_tm + 32*cc, o);
                }
                tmem_st_wait();
            }
            l *= alpha;
            m_used = m_new;
            const float neg_ref = m_used == -CUDART_INF_F ? 0.0f : -m_used;
            PROF_T(pt4);
            // ---- P = exp2(x - m), row sum, elem_t pack, back into the S columns (in two
            // rounds of 64 values to bound the registers), then one hand-over ---------
            const uint64_t mul2 = pack_f32x2(mul, mul), ref2 = pack_f32x2(neg_ref, neg_ref);
            uint64_t sum_a = 0ull, sum_b = 0ull;          // two packed chains = four sums
#pragma unroll
            for(int h = 0; h < 2; ++h)
            {
                uint32_t pk[32];
#pragma unroll
                for(int j = 0; j < 32; j += 2)
                {
                    const uint32_t *src = &s[2*h + (j >> 4)][(2*j) & 31];
                    float xa0, xa1, xb0, xb1;
                    unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(src[0]), __uint_as_float(src[1])),
                            mul2, ref2), xa0, xa1);
                    unpack_f32x2(ffma2(pack_f32x2(__uint_as_float(src[2]), __uint_as_float(src[3])),
                            mul2, ref2), xb0, xb1);
                    const float pa0 = ex2(xa0), pa1 = ex2(xa1), pb0 = ex2(xb0), pb1 = ex2(xb1);
                    sum_a = fadd2(sum_a, pack_f32x2(pa0, pa1));
                    sum_b = fadd2(sum_b, pack_f32x2(pb0, pb1));
                    pk[j] = pack_elem2(pa0, pa1);
                    pk[j + 1] = pack_elem2(pb0, pb1);
                }
                tmem_st32(s_tm + 32*h, pk);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if(lane == 0)
            {
                mbar_arrive(&sm.p_full[t]);
            }
            {
                float a0, a1, b0, b1;
                unpack_f32x2(fadd2(sum_a, sum_b), a0, a1);
                b0 = a0 + a1;
                b1 = 0.0f;
                l += b0 + b1;
            }
#ifdef NB200_PROF
            if(r == 0 && t == 0)
            {
                PROF_T(pt5);
                PROF_ADD(0, pt0, pt1);      // wait for S
                PROF_ADD(1, pt1, pt2);      // tcgen05.ld of the row
                PROF_ADD(2, pt2, pt3);      // mask + max
                PROF_ADD(3, pt3, pt4);      // rescale decision (+ O round trip)
                PROF_ADD(4, pt4, pt5);      // exp2, pack, store, arrive
                atomicAdd(&g_prof[5], 1ull);
            }
#endif
            ++n;
        }
        // ---- epilogue: normalise, merge with the stored (lse, A), store ---------
        if(ok && nact > 0)
        {
            ok = mbar_wait<LIMIT>(&sm.o_full[t], 0, abort_flag);
        }
        ok = __all_sync(0xffffffffu, ok);     // the epilogue is warp-collective
        if(ok && nact > 0)
        {
            tc_fence_after_sync();
            const size_t R = (size_t)row_base + (size_t)qb*BLK + r;
            const float in = l > 0.0f ? (m_used + log2f(l))*LN2_F : -CUDART_INF_F;
            // rows with nothing to add stay untouched; the TMEM loads below are
            // warp-collective, so only the global accesses are predicated
            const bool live = isfinite(in);
            float w_dst = 0.0f, w_src = 0.0f;
            if(live)
            {
                const float old = lse_old;
                float e, big;
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
                lse[R] = big + logf(1.0f + e);
            }
            const float inv = live ? 1.0f/l : 0.0f;
            // The normalised tile result, rounded to storage as the reference's scratch
            // output is, goes into this warp's 32 rows of the Q tile (no MMA reads it
            // any more) as 64-column panels with 128-byte rows in the 128-byte swizzle
            // of the tensor map.  When every row of the warp simply replaces the stored
            // one (lse was -inf: first K/V tile of this Q tile), one lane hands the
            // panels to the TMA unit as a store; otherwise the warp merges row-major
            // (TMEM gives a thread one row, global memory wants a warp on consecutive
            // bytes: one row per lane would cost 32 L1 wavefronts per instruction).
            constexpr int PANELS = D/64;
            uint8_t *stage = sm.q[t] + (warp & 3)*(PANELS*4096);
#pragma unroll
            for(int p = 0; p < PANELS; ++p)
            {
                uint32_t o[2][32];
                tmem_ld32(o_tm + 64*p, o[0]);
                tmem_ld32(o_tm + 64*p + 32, o[1]);
                tmem_ld_wait();
                uint8_t *prow = stage + p*4096 + lane*128;
#pragma unroll
                for(int g8 = 0; g8 < 8; ++g8)
                {
                    uint32_t w[4];
#pragma unroll
                    for(int e2 = 0; e2 < 4; ++e2)
                    {
                        w[e2] = pack_elem2(__uint_as_float(o[g8 >> 2][8*(g8 & 3) + 2*e2])*inv,
                                __uint_as_float(o[g8 >> 2][8*(g8 & 3) + 2*e2 + 1])*inv);
                    }
                    *reinterpret_cast<uint4 *>(prow + ((g8 ^ (lane & 7)) << 4)) =
                            make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            const bool replace_all = __all_sync(0xffffffffu, live && w_dst == 0.0f);
            if(replace_all)
            {
                fence_proxy_async();
                __syncwarp();
                if(lane == 0)
                {
                    const int row0 = row_base + qb*BLK + 32*(warp & 3);
#pragma unroll
                    for(int p = 0; p < PANELS; ++p)
                    {
                        tma_store_2d(&tmap_a, stage + p*4096, 64*p, row0);
                    }
                    bulk_commit_group();
                    bulk_wait_read_all();
                }
            }
            else
            {
            __syncwarp();
            constexpr int LPR = D/8;                  // lanes (16-byte pieces) per row
            constexpr int RPI = 32/LPR;               // rows per warp instruction
            const int sub = lane/LPR, piece = lane % LPR;
            elem_t *out = A + ((size_t)row_base + (size_t)qb*BLK + 32*(warp & 3))*D;
#pragma unroll
            for(int base = 0; base < 32; base += 8*RPI)
            {
                uint4 prev[8];
                float wd[8], ws[8];
                bool lv[8];
#pragma unroll
                for(int j = 0; j < 8; ++j)
                {
                    const int row = base + j*RPI + sub;
                    wd[j] = __shfl_sync(0xffffffffu, w_dst, row);
                    ws[j] = __shfl_sync(0xffffffffu, w_src, row);
                    lv[j] = __shfl_sync(0xffffffffu, (int)live, row) != 0;
                    prev[j] = make_uint4(0u, 0u, 0u, 0u);
                    if(lv[j] && wd[j] != 0.0f)        // a weight of zero never reads the old row
                    {
                        prev[j] = *reinterpret_cast<const uint4 *>(out + (size_t)row*D + 8*piece);
                    }
                }
#pragma unroll
                for(int j = 0; j < 8; ++j)
                {
                    const int row = base + j*RPI + sub;
                    const uint4 g = *reinterpret_cast<const uint4 *>(stage + (piece >> 3)*4096
                            + row*128 + (((piece & 7) ^ (row & 7)) << 4));
                    const uint32_t pw[4] = {prev[j].x, prev[j].y, prev[j].z, prev[j].w};
                    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
                    uint32_t outw[4];
#pragma unroll
                    for(int e2 = 0; e2 < 4; ++e2)
                    {
                        outw[e2] = pack_elem2(
                                wd[j]*elem_lo(pw[e2]) + ws[j]*elem_lo(gw[e2]),
                                wd[j]*elem_hi(pw[e2]) + ws[j]*elem_hi(gw[e2]));
                    }
                    if(lv[j])
                    {
                        *reinterpret_cast<uint4 *>(out + (size_t)row*D + 8*piece) =
                                make_uint4(outw[0], outw[1], outw[2], outw[3]);
                    }
                }
            }
            }
        }
        if(!ok && lane == 0)
        {
            atomicCAS(status, 0u, STATUS_FWD_SOFTMAX);
        }
    }
    // ---- tear-down ---------------------------------------------------------------
    if(tid == 0)
    {
        // the Q copies issued at the start must have landed before the shared memory
        // goes away, also when nobody needed them
        mbar_wait<LIMIT>(&sm.q_full[0], 0, abort_flag);
        if(has1)
        {
            mbar_wait<LIMIT>(&sm.q_full[1], 0, abort_flag);
        }
    }
    if(*abort_flag != 0u && tid == 0)
    {
        // give copies still in flight time to land before the CTA's memory goes away
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
}

} // namespace fwd

#if defined(NB200_PROF) && !defined(NB200_FP16)
extern "C" void nntile_b200_debug_prof(unsigned long long *out16, int reset)
{
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out16, fwd::g_prof, sizeof(unsigned long long)*16);
    if(reset)
    {
        unsigned long long z[16] = {0};
        cudaMemcpyToSymbol(fwd::g_prof, z, sizeof(z));
    }
}
#endif

bool flash_fwd_sm100_supports(Index seq, Index head, Index batch)
{
    return (head == 64 || head == 128) && seq >= fwd::BLK && seq % fwd::BLK == 0
            && seq/fwd::BLK <= fwd::MAX_BLOCKS && batch >= 1
            && batch*seq < ((Index)1 << 31) && batch*((seq/fwd::BLK + 1)/2) < ((Index)1 << 31);
}

static std::atomic<uint32_t> g_wait_test_armed{0};

template<int D>
static int fwd_run(cudaStream_t s, Index seq, Index batch, Index kv_group, Index kv_batch,
        const elem_t *K, const elem_t *Q,
        const elem_t *mask, const elem_t *V, float *lse, elem_t *A, const FwdAux &aux)
{
    using namespace fwd;
    CUtensorMap tq, tk, tv, ta;
    const uint64_t rows = (uint64_t)batch*seq;
    const uint64_t kv_rows = rows/(uint64_t)kv_group;
    if(!make_tmap_16_sw128(&tq, Q, rows, D, BLK, ELEM_TMAP_TYPE)
            || !make_tmap_16_sw128(&tk, K, kv_rows, D, BLK, ELEM_TMAP_TYPE)
            || !make_tmap_16_sw128(&tv, V, kv_rows, D, BLK, ELEM_TMAP_TYPE)
            || !make_tmap_16_sw128(&ta, A, rows, D, 32, ELEM_TMAP_TYPE))
    {
        return NNTILE_B200_E_LAUNCH;
    }
    const int nblk = (int)(seq/BLK);
    if(aux.classify && launch_mask_classify(s, (int)seq, mask, aux.cls, aux.status) != NNTILE_B200_OK)
    {
        return NNTILE_B200_E_LAUNCH;
    }
    // The opt-in to more than 48 KB of dynamic shared memory belongs to the kernel
    // ON ONE DEVICE: a process that drives several GPUs needs it on each of them.
    constexpr size_t smem_bytes = sizeof(Smem<D>) + 1024;
    static PerDeviceOnce optin;
    int dev = -1;
    if(cudaGetDevice(&dev) != cudaSuccess || !optin.ensure(dev, []() {
            return cudaFuncSetAttribute(flash_fwd_kernel<D, false>,
                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) == cudaSuccess
                && cudaFuncSetAttribute(flash_fwd_kernel<D, true>,
                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) == cudaSuccess; }))
    {
        return NNTILE_B200_E_LAUNCH;
    }
    const unsigned grid = (unsigned)(((nblk + 1)/2)*batch);
    const float scale_log2 = LOG2E_F/sqrtf((float)D);
    // Q, K, V, A of one batch entry
    const int gsz = l2_group_size(batch, (size_t)seq*D*2*4);
    if(g_wait_test_armed.exchange(0u, std::memory_order_relaxed) != 0u)
    {
        flash_fwd_kernel<D, true><<<grid, THREADS, smem_bytes, s>>>(tq, tk, tv, ta, (int)seq,
                (int)batch, gsz, (int)kv_group, (int)kv_batch, scale_log2, mask, aux.status,
                aux.cls, lse, A);
        return launch_status();
    }
    flash_fwd_kernel<D, false><<<grid, THREADS, smem_bytes, s>>>(tq, tk, tv, ta, (int)seq,
            (int)batch, gsz, (int)kv_group, (int)kv_batch, scale_log2, mask, aux.status, aux.cls,
            lse, A);
    return launch_status();
}

int launch_mask_classify(cudaStream_t s, int seq, const elem_t *mask, uint8_t *cls,
        uint32_t *status)
{
    const int nblk = seq/fwd::BLK;
    fwd::mask_classify_kernel<<<dim3(nblk, nblk), 256, 0, s>>>(seq, nblk, mask, cls, status);
    return launch_status();
}

int flash_fwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *mask, const elem_t *V, float *lse, elem_t *A, const FwdAux &aux,
        Index kv_group, Index kv_batch)
{
    if(kv_group < 1 || kv_batch < 1 || batch % (kv_group*kv_batch) != 0 || !aux.status || !aux.cls)
    {
        return NNTILE_B200_E_BADARG;
    }
    return head == 128
            ? fwd_run<128>(s, seq, batch, kv_group, kv_batch, K, Q, mask, V, lse, A, aux)
            : fwd_run<64>(s, seq, batch, kv_group, kv_batch, K, Q, mask, V, lse, A, aux);
}

} // inline namespace
} // namespace nb200

#ifndef NB200_FP16
// Test support: arms the one-shot wait-timeout hook described in the header (the
// bfloat16 build's forward kernel).
extern "C" void nntile_b200_test_arm_wait_timeout(void)
{
    nb200::g_wait_test_armed.store(1u, std::memory_order_relaxed);
}
#endif
