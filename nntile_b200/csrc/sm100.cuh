// Blackwell (sm_100a) building blocks as inline PTX: mbarriers with BOUNDED
// waits, TMA tiled loads (every copy targets this CTA only), tensor-memory management and
// the tcgen05 MMA / load / store instructions with their descriptors.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nb200 {
namespace sm100 {

// ------------------------------------------------------------------ addresses
__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ------------------------------------------------------------------ mbarriers
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
            :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}

// Every wait in these kernels is bounded: it gives up after LIMIT_NS of wall time,
// or as soon as a sibling role has given up (`*abort_flag` set), and returns
// false; the caller records where it stopped and leaves its loop, and the CTA
// tears down normally.  A wait never spins forever and never traps.  The limit is
// a compile-time constant (the issuing threads have no register to spare for
// it); the test instantiation of the forward kernel uses WAIT_LIMIT_TEST_NS.
constexpr uint64_t WAIT_LIMIT_NS = 200ull*1000ull*1000ull;
constexpr uint64_t WAIT_LIMIT_TEST_NS = 1000ull*1000ull;

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template<uint64_t LIMIT_NS = WAIT_LIMIT_NS>
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity,
        volatile uint32_t *abort_flag)
{
    if(mbar_try_wait(bar, parity))
    {
        return true;
    }
    const uint64_t t0 = global_timer_ns();
    for(;;)
    {
#pragma unroll 1
        for(int spin = 0; spin < 128; ++spin)
        {
            if(mbar_try_wait(bar, parity))
            {
                return true;
            }
        }
        if(*abort_flag != 0u)
        {
            return false;
        }
        if(global_timer_ns() - t0 > LIMIT_NS)
        {
            *abort_flag = 1u;
            return false;
        }
    }
}

// The same wait for a converged warp: every lane polls, and all lanes get the same
// answer (a limit that ran out in one lane ends the wait for the warp).
template<uint64_t LIMIT_NS = WAIT_LIMIT_NS>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity,
        volatile uint32_t *abort_flag)
{
    return __all_sync(0xffffffffu, mbar_wait<LIMIT_NS>(bar, parity, abort_flag));
}

// ------------------------------------------------------------------------ TMA
// 2-D tiled load global -> this CTA's shared memory, completion on an mbarrier.
// x is the innermost (contiguous) coordinate: x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map,
        uint64_t *bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)),
           "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// Untiled bulk copy global -> this CTA's shared memory, completion on an mbarrier;
// both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(void *smem_dst, const void *gmem_src,
        uint32_t bytes, uint64_t *bar)
{
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        :: "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes),
           "r"(smem_u32(bar)) : "memory");
}

// 2-D tiled store / element-wise add shared memory -> global through the TMA unit
// (bulk async-group completion).  The tile in shared memory has the layout the
// tensor map describes (here: 128-byte rows, 128-byte swizzle); x is the innermost
// coordinate and must be a multiple of 16 bytes / element size.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, const void *smem_src,
        int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
            :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
            : "memory");
}

__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, const void *smem_src,
        int32_t x, int32_t y)
{
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
            :: "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
            : "memory");
}

__device__ __forceinline__ void bulk_commit_group()
{
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// all committed bulk groups of this thread have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all()
{
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void prefetch_l2(const void *p)
{
    asm volatile("prefetch.global.L2 [%0];" :: "l"(p) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" :: "l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// -------------------------------------------------------------- tensor memory
// Allocate `ncols` (power of two, 32..512) TMEM columns; one full warp executes
// this, the base address lands in *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
            :: "r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
            :: "r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// mbarrier arrive (count 1) once every tcgen05 operation this thread has issued
// so far has completed.
__device__ __forceinline__ void tc_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
            :: "r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory operand descriptor, 128-byte swizzle, version 1 (Blackwell):
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 version = 1
//   bits 61-63 layout = 2 (SWIZZLE_128B)
// K-major operand stored as rows of 128 bytes (64 bf16 of the contraction
// dimension per row): 8-row groups are `sbo` bytes apart (1024 when rows are
// packed); the leading offset is unused.
// MN-major operand stored as rows of 128 bytes (64 bf16 of the M/N dimension per
// row, one row per contraction index): 8-row groups `sbo` bytes apart, the next
// 64 elements of M/N `lbo` bytes away.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes,
        uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// The same descriptor split into its two 32-bit words so that the issuing thread
// can keep one low word per tile and step through k by adding a constant: the
// high word depends only on the stride offset, the low word is
// (address >> 4) | (leading offset >> 4) << 16.  Adding (bytes >> 4) to the low word
// moves the start address as long as the tile stays below 256 KB of shared memory.
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes)
{
    return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}

__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr, uint32_t lbo_bytes)
{
    return ((saddr >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}

__device__ __forceinline__ uint64_t smem_desc_join(uint32_t lo, uint32_t hi)
{
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and fp32 accumulate:
//   bits 4-5 D format (1 = f32)   bits 7-9 A format (1 = bf16)   bits 10-12 B format
//   bit 15 A major (0 = K, 1 = MN)   bit 16 B major   bits 17-22 N>>3   bits 24-28 M>>4
// `fmt` is the format of both operands: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t idesc_16(int M, int N, int a_mn_major, int b_mn_major,
        uint32_t fmt)
{
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn_major << 15)
            | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17)
            | ((uint32_t)(M >> 4) << 24);
}

__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn_major, int b_mn_major)
{
    return idesc_16(M, N, a_mn_major, b_mn_major, 1u);
}

// ------------------------------------------------------------------------ MMA
// D[tmem] (+)= A[smem] * B[smem]; one thread issues.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A is 128 lanes x (K/2) columns of packed bf16.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
        uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Variants whose accumulate flag is a compile-time constant (no setp on a register).
template<bool ACC>
__device__ __forceinline__ void mma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
        uint32_t idesc)
{
    if(ACC)
    {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
    }
    else
    {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, 0, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
    }
}

template<bool ACC>
__device__ __forceinline__ void mma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
        uint32_t idesc)
{
    if(ACC)
    {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc) : "memory");
    }
    else
    {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, 0, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
            :: "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc) : "memory");
    }
}

// ------------------------------------------------------- TMEM <-> registers
// 32 lanes x 32 columns of 32 bits: thread i of the warp gets lane (base + i),
// register j gets column (base column + j).  A warp may only touch the lane
// quarter 32*(warp_id % 4).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_ld_wait()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
           "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
           "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
           "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
           "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 32 lanes x 16 columns variants.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]),
           "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
           "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Barrier among `nthreads` threads of the CTA (ids 1..15; 0 is __syncthreads).
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ void red_add_f32(float *addr, float a)
{
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(addr), "f"(a) : "memory");
}

__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
            :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void tmem_st_wait()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Three-input max and two-wide packed fp32 arithmetic (one instruction for two
// lanes of a 64-bit register pair), both new with sm_100.
__device__ __forceinline__ float fmax3(float a, float b, float c)
{
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("mul.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

} // namespace sm100

// ----------------------------------------------------------- host: tensor maps
// cuTensorMapEncodeTiled is reached through the runtime's driver entry point
// lookup, so the library links against nothing but cudart.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
        const cuuint64_t *, const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
        CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
        CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q)
                != cudaSuccess || q != cudaDriverEntryPointSuccess)
        {
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Row-major matrix of 16-bit elements [rows][cols] (cols contiguous) cut into boxes
// of box_rows x 64 columns (128 bytes), written to shared memory with the 128-byte
// swizzle that the MMA descriptors above expect.
inline bool make_tmap_16_sw128(CUtensorMap *map, const void *base, uint64_t rows,
        uint64_t cols, uint32_t box_rows, CUtensorMapDataType type)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if(!fn)
    {
        return false;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols*2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, type, 2, const_cast<void *>(base), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
            == CUDA_SUCCESS;
}

} // namespace nb200
