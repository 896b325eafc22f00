#include "flash.cuh"
namespace nb200 {
bool flash_fwd_sm100_supports(Index, Index, Index) { return false; }
int flash_fwd_sm100(cudaStream_t, Index, Index, Index, const bf16 *, const bf16 *, const bf16 *,
        const bf16 *, float *, bf16 *, void *, size_t) { return NNTILE_B200_E_SHAPE; }
}
