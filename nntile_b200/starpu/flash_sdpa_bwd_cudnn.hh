// Replacement for include/nntile/starpu/flash_sdpa_bwd_cudnn.hh of the reference:
// the StarPU codelet of the fused backward tile task without cuDNN.  Class name,
// codelet name, args_t, footprint, the order of the thirteen buffers and the
// signature of submit() are the reference's (its header :36-170), so
// src/tile/flash_sdpa_bwd_cudnn.cc:90-136 compiles against this file unchanged.
// Gone: the per-worker graph cache and the cudaMalloc'ed cuDNN workspace it owned
// - the three scratch handles the tile layer registers hold everything the
// sm_100a kernels need (fp32 dQ accumulator, delta, lse*log2e, mask classes).
// Thirteen buffers still need StarPU built with --enable-maxbuffers=16, as the
// reference's Dockerfile does.
#pragma once

#include <nntile/defs.h>
#include <tuple>
#include <nntile/starpu/codelet.hh>
#include <nntile/starpu/handle.hh>

namespace nntile::starpu
{

template<typename T>
class FlashSdpaBwdCudnn;

template<typename T>
class FlashSdpaBwdCudnn<std::tuple<T>>
{
public:
    CodeletTyped<T> codelet;

    FlashSdpaBwdCudnn();

    struct args_t
    {
        FlashSdpaBwdCudnn<std::tuple<T>> *owner;
        Index seq = 0;
        Index head = 0;
        Index batch = 0;
    };

    static uint32_t hash_parameters(Index seq, Index head, Index batch);
    static uint32_t footprint(struct starpu_task *task);

    static constexpr func_array cpu_funcs = {};

#ifdef NNTILE_USE_CUDA
    static void cuda(void *buffers[], void *cl_args) noexcept;
    static constexpr func_array cuda_funcs = {
        cuda
    };
#else
    static constexpr func_array cuda_funcs = {};
#endif

    void submit(
        Index seq,
        Index head,
        Index batch,
        Handle K,
        Handle Q,
        Handle V,
        Handle A,
        Handle dA,
        Handle mask,
        Handle logsumexp,
        Handle dK,
        Handle dQ,
        Handle dV,
        Handle scratch_dK,
        Handle scratch_dQ,
        Handle scratch_dV
    );
};

using flash_sdpa_bwd_cudnn_pack_t = OperationPack<
    FlashSdpaBwdCudnn,
    std::tuple<nntile::bf16_t>,
    std::tuple<nntile::fp16_t>
>;

extern flash_sdpa_bwd_cudnn_pack_t flash_sdpa_bwd_cudnn;

} // namespace nntile::starpu
