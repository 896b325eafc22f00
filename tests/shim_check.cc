#define NNTILE_B200_STANDALONE_TYPES
#include <nntile_b200/kernel_shims.hh>
using namespace nntile;
int main()
{
    cudaStream_t s = nullptr;
    kernel::maxsumexp::cuda<fp32_t>(s, 1, 1, 1, nullptr, nullptr);
    kernel::maxsumexp::cuda<bf16_t>(s, 1, 1, 1, nullptr, nullptr);
    kernel::softmax_inplace::cuda<bf16_t>(s, 1, 1, 1, nullptr, 1.0f, nullptr);
    kernel::sumprod_slice::cuda<fp32_t>(s, 1, 1, 1, 1.0f, nullptr, nullptr, 0.0f, nullptr);
    kernel::mask_scalar::cuda<bf16_t>(s, 1, 1, nullptr, 0.0f, nullptr);
    kernel::add_slice_inplace::cuda<fp32_t>(s, 1, 1, 1, 1.0f, nullptr, 1.0f, nullptr);
    kernel::multiply_inplace::cuda<bf16_t>(s, 1, 1.0f, nullptr, nullptr);
    kernel::add_inplace::cuda<fp32_t>(s, 1, 1.0f, nullptr, 1.0f, nullptr);
    kernel::accumulate_attn_output::cuda<bf16_t>(s, 1, 1, 1, nullptr, nullptr, nullptr, nullptr);
    kernel::cublas::gemm<fp32_t>(nullptr, TransOp(TransOp::Trans), TransOp(TransOp::NoTrans), 4, 4, 4, 1, 1.0f, nullptr, nullptr, 0.0f, nullptr);
    if(nntile_b200::last_status() != NNTILE_B200_E_BADARG) return 2;
    kernel::cublas::gemm<bf16_t>(nullptr, TransOp(TransOp::NoTrans), TransOp(TransOp::Trans), 4, 4, 4, 1, 1.0f, nullptr, nullptr, 1.0f, nullptr);
    if(nntile_b200::last_status() != NNTILE_B200_E_BADARG) return 3;
    kernel::flash_sdpa_fwd::cuda<bf16_t>(s, 128, 64, 1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    kernel::flash_sdpa_bwd::cuda<bf16_t>(s, 128, 64, 1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    if(nntile_b200::last_status() != NNTILE_B200_E_BADARG) return 1;
    kernel::flash_sdpa_fwd::cuda<fp16_t>(s, 128, 64, 1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    if(nntile_b200::last_status() != NNTILE_B200_E_BADARG) return 4;
    kernel::flash_sdpa_bwd::cuda<fp16_t>(s, 128, 64, 1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    return nntile_b200::last_status() == NNTILE_B200_E_BADARG ? 0 : 5;
}
