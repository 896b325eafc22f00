// Internal interface between the C entry points of the fused SDPA tile tasks
// and the kernels that implement them.
#pragma once
#include "common.cuh"

namespace nb200 {

// Generic CUDA-core kernels (flash_generic.cu): any seq, head <= 256.
int flash_fwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const bf16 *K,
        const bf16 *Q, const bf16 *mask, const bf16 *V, float *lse, bf16 *A);
int flash_bwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const bf16 *K,
        const bf16 *Q, const bf16 *V, const bf16 *A, const bf16 *dA, const bf16 *mask,
        const float *lse, float *delta, bf16 *dK, bf16 *dQ, bf16 *dV);
int flash_bwd_delta(cudaStream_t s, Index head, Index rows, const bf16 *A, const bf16 *dA,
        float *delta);

// tcgen05 / TMEM / TMA kernels (flash_fwd_sm100.cu, flash_bwd_sm100.cu):
// head in {64, 128}, seq a multiple of 128.
bool flash_fwd_sm100_supports(Index seq, Index head, Index batch);
// K, V (and dK, dV) may be shared by `kv_group` consecutive groups of `kv_batch`
// batch entries: entry b uses K/V entry (b % kv_batch) + kv_batch*(b/(kv_batch*kv_group)).
// kv_group = 1, kv_batch = batch is the plain one-to-one case.
int flash_fwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const bf16 *K,
        const bf16 *Q, const bf16 *mask, const bf16 *V, float *lse, bf16 *A,
        void *scratch, size_t scratch_bytes, Index kv_group, Index kv_batch);
bool flash_bwd_sm100_supports(Index seq, Index head, Index batch);
int flash_bwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const bf16 *K,
        const bf16 *Q, const bf16 *V, const bf16 *A, const bf16 *dA, const bf16 *mask,
        const float *lse, void *scratch_dK, void *scratch_dQ, void *scratch_dV,
        bf16 *dK, bf16 *dQ, bf16 *dV, Index kv_group, Index kv_batch);

// Classes of a 128x128 block of the additive mask [seq_q][seq_k].
enum : uint8_t
{
    CLS_ZERO = 0,     // every entry 0: the mask is not read
    CLS_SKIP = 1,     // every entry -inf: the block is never loaded or multiplied
    CLS_GENERIC = 2,  // anything else: the bias is read from global memory
    CLS_CAUSAL = 3    // exactly 0 where key <= query and -inf above the diagonal
};

// Layout of the scratch buffer the tcgen05 kernels use: a 32-bit status word at
// offset 0 (0 = every bounded wait completed), the class table
// [query block][key block] at CLS_OFFSET.
constexpr size_t CLS_OFFSET = 256;

// CTA numbering shared by the two tcgen05 kernels.  CTAs are numbered group by
// group; a group is `gsz` consecutive batch entries whose tensors (and, in the
// backward, fp32 dQ accumulator) fit the L2 cache together, so the CTAs that are
// resident at the same time re-read each other's K/V (forward) or Q/dO and
// accumulator lines (backward) from L2 instead of DRAM.  Inside a group the
// numbering is unit-major (unit = key block or query-tile pair), so the caller
// can put heavy units first.
constexpr size_t L2_GROUP_BYTES = (size_t)64 << 20;

inline int l2_group_size(Index batch, size_t bytes_per_entry)
{
    size_t budget = L2_GROUP_BYTES;
#ifdef NB200_EXP_ENV
    if(const char *e = getenv("NB200_L2_GROUP_MB")) budget = (size_t)atoi(e) << 20;
#endif
    const size_t g = budget/(bytes_per_entry > 0 ? bytes_per_entry : 1);
    return (int)(g < 1 ? 1 : (g > (size_t)batch ? (size_t)batch : g));
}

__device__ __forceinline__ void group_decode(unsigned cta, int nunits, int batch, int gsz,
        int &unit, int &b)
{
    const unsigned per = (unsigned)gsz*(unsigned)nunits;
    const unsigned g = cta/per, rem = cta - g*per;
    const int left = batch - (int)g*gsz;
    const unsigned cur = (unsigned)(left < gsz ? left : gsz);
    unit = (int)(rem/cur);
    b = (int)g*gsz + (int)(rem - (unsigned)unit*cur);
}

// Classify every block of `mask` into scratch + CLS_OFFSET and clear the status
// word (flash_fwd_sm100.cu).
int launch_mask_classify(cudaStream_t s, int seq, const bf16 *mask, uint8_t *scratch);

} // namespace nb200
