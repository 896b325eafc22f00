#include "flash.cuh"
namespace nb200 {
bool flash_bwd_sm100_supports(Index, Index, Index) { return false; }
int flash_bwd_sm100(cudaStream_t, Index, Index, Index, const bf16 *, const bf16 *, const bf16 *,
        const bf16 *, const bf16 *, const bf16 *, const float *, void *, void *, void *,
        bf16 *, bf16 *, bf16 *) { return NNTILE_B200_E_SHAPE; }
}
