// Internal interface between the C entry points of the fused SDPA tile tasks
// and the kernels that implement them.
#pragma once
#include "common.cuh"
#include "elem.cuh"

namespace nb200 {
inline namespace NB200_ELEM_NS {

// Generic CUDA-core kernels (flash_generic.cu): any seq, head <= 256.
int flash_fwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *mask, const elem_t *V, float *lse, elem_t *A);
int flash_bwd_generic(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *V, const elem_t *A, const elem_t *dA, const elem_t *mask,
        const float *lse, float *delta, elem_t *dK, elem_t *dQ, elem_t *dV);
int flash_bwd_delta(cudaStream_t s, Index head, Index rows, const elem_t *A, const elem_t *dA,
        float *delta);

// tcgen05 / TMEM / TMA kernels (flash_fwd_sm100.cu, flash_bwd_sm100.cu):
// head in {64, 128}, seq a multiple of 128.
//
// Bookkeeping of a tile task in device memory.  `status` is the 32-bit status
// word (0 = every bounded wait completed; see STATUS_* below), `cls` the class
// table [query block][key block] of the task's mask tile.  A tile-level call
// carves both out of the scratch buffer of the task (status at offset 0, table
// at CLS_OFFSET), classifies the mask and clears the word itself; the
// tensor-level loops classify every distinct mask buffer once per call, keep one
// status word for the whole call that no task clears, and pass `classify = false`.
struct FwdAux
{
    uint32_t *status;
    uint8_t *cls;
    bool classify;
};

// Backward bookkeeping: besides the two above, delta = -rowsum(A o dA) and
// lse2 = -lse*log2(e) (rows floats each) and the fp32 dQ accumulator, split at
// `half_rows` over two buffers.  `phases` selects what a call enqueues, so that
// the tensor-level loops can prepare and finish a Q tile once for all its K/V
// tiles instead of once per pair.
enum : int
{
    BWD_CLASSIFY = 1,   // classify the mask into `cls`, clear `status`
    BWD_PREP = 2,       // delta, lse2, clear the accumulator
    BWD_MAIN = 4,       // the tcgen05 kernel: dK, dV += ..., accumulator += dQ
    BWD_FINISH = 8,     // dQ += elem_t(scale * accumulator)
    BWD_ALL = 15
};

struct BwdAux
{
    uint32_t *status;
    uint8_t *cls;
    float *delta, *lse2;
    float *acc_lo, *acc_hi;
    Index half_rows;
    int phases;
};

bool flash_fwd_sm100_supports(Index seq, Index head, Index batch);
// K, V (and dK, dV) may be shared by `kv_group` consecutive groups of `kv_batch`
// batch entries: entry b uses K/V entry (b % kv_batch) + kv_batch*(b/(kv_batch*kv_group)).
// kv_group = 1, kv_batch = batch is the plain one-to-one case.
int flash_fwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *mask, const elem_t *V, float *lse, elem_t *A,
        const FwdAux &aux, Index kv_group, Index kv_batch);
bool flash_bwd_sm100_supports(Index seq, Index head, Index batch);
int flash_bwd_sm100(cudaStream_t s, Index seq, Index head, Index batch, const elem_t *K,
        const elem_t *Q, const elem_t *V, const elem_t *A, const elem_t *dA, const elem_t *mask,
        const float *lse, const BwdAux &aux, elem_t *dK, elem_t *dQ, elem_t *dV, Index kv_group,
        Index kv_batch);
// Layout the tile-level entry points give the three scratch buffers of a backward
// task (status + class table + delta + lse2 in scratch_dV, the accumulator halves
// in scratch_dQ and scratch_dK).
BwdAux bwd_aux_from_scratch(Index seq, Index batch, void *scratch_dK, void *scratch_dQ,
        void *scratch_dV);
// Bytes of scratch_dV the layout above needs.
size_t bwd_aux_bytes(Index seq, Index batch);

// Entry points shared by the C wrappers (flash_api.cu) and the tensor-level
// loops (host_tensor.cu): argument checks and the choice between the tcgen05
// and the generic kernels.  `fwd_aux` / `bwd_aux` may be null: the bookkeeping
// is then carved out of the scratch buffers as the tile-level C ABI documents.
int flash_fwd_task(cudaStream_t s, Index seq, Index head, Index batch, const void *K,
        const void *Q, const void *mask, const void *V, void *scratch_A, float *lse, void *A,
        const FwdAux *fwd_aux);
int flash_bwd_task(cudaStream_t s, Index seq, Index head, Index batch, const void *K,
        const void *Q, const void *V, const void *A, const void *dA, const void *mask,
        const float *lse, void *scratch_dK, void *scratch_dQ, void *scratch_dV, void *dK,
        void *dQ, void *dV, const BwdAux *bwd_aux);

// Values of the status word: which role of which kernel gave up first.
enum : uint32_t
{
    STATUS_OK = 0,
    STATUS_FWD_PRODUCER = 1, STATUS_FWD_MMA = 2, STATUS_FWD_SOFTMAX = 3,
    STATUS_BWD_PRODUCER = 11, STATUS_BWD_MMA = 12, STATUS_BWD_DRAIN = 13,
    STATUS_BWD_SOFTMAX = 14, STATUS_BWD_SMEM_ALIGN = 20
};

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
    const size_t g = L2_GROUP_BYTES/(bytes_per_entry > 0 ? bytes_per_entry : 1);
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

// Classify every block of `mask` into `cls` and, when `status` is not null, clear
// that status word (flash_fwd_sm100.cu).
int launch_mask_classify(cudaStream_t s, int seq, const elem_t *mask, uint8_t *cls,
        uint32_t *status);

} // inline namespace
} // namespace nb200
