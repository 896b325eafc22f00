// Replacement for include/nntile/starpu/flash_sdpa_fwd_cudnn.hh of the reference:
// the StarPU codelet of the fused forward tile task with the cuDNN graph machinery
// taken out.  Class name, codelet name, args_t, footprint, buffer order and the
// signature of submit() are those of the reference (its header :44-156), so the
// tile layer (src/tile/flash_sdpa_fwd_cudnn.cc:161-196) compiles against this file
// unchanged.  What is gone: the per-worker graph cache (CacheEntry, WorkerCache,
// the once-flags) and the include of the cuDNN kernel header.
//
// Drop this file and flash_sdpa_fwd_cudnn.cc over the reference's two files and
// link libnntile_b200.so.
#pragma once

#include <nntile/defs.h>
#include <tuple>
#include <nntile/starpu/codelet.hh>
#include <nntile/starpu/handle.hh>

namespace nntile::starpu
{

template<typename T>
class FlashSdpaFwdCudnn;

template<typename T>
class FlashSdpaFwdCudnn<std::tuple<T>>
{
public:
    //! Codelet for the current operation
    CodeletTyped<T> codelet;

    FlashSdpaFwdCudnn();

    //! Arguments of one task; `owner` is kept so that args_t stays layout-
    //! compatible with the reference's, nothing reads it any more
    struct args_t
    {
        FlashSdpaFwdCudnn<std::tuple<T>> *owner;
        Index seq;
        Index head;
        Index batch;
    };

    static uint32_t hash_parameters(Index seq, Index head, Index batch);

    static uint32_t footprint(struct starpu_task *task);

    //! No CPU implementations, as in the reference
    static constexpr func_array cpu_funcs = {};

#ifdef NNTILE_USE_CUDA
    //! Body run by a StarPU CUDA worker: one call into libnntile_b200.so
    static void cuda(void *buffers[], void *cl_args) noexcept;

    static constexpr func_array cuda_funcs = {
        cuda
    };
#else // NNTILE_USE_CUDA
    static constexpr func_array cuda_funcs = {};
#endif // NNTILE_USE_CUDA

    //! Buffers in the reference's order: K, Q, mask, logsumexp, V, A and the two
    //! scratch handles of the tile layer
    void submit(
        Index seq,
        Index head,
        Index batch,
        Handle K,
        Handle Q,
        Handle mask,
        Handle logsumexp,
        Handle V,
        Handle A,
        Handle scratch_logsumexp,
        Handle scratch_A
    );
};

//! bf16 and fp16, as in the reference
using flash_sdpa_fwd_cudnn_pack_t = OperationPack<
    FlashSdpaFwdCudnn,
    std::tuple<nntile::bf16_t>,
    std::tuple<nntile::fp16_t>
>;

extern flash_sdpa_fwd_cudnn_pack_t flash_sdpa_fwd_cudnn;

} // namespace nntile::starpu
