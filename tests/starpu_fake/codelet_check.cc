// C doors onto the replacement codelets, for the Python tests.  TEST
// INFRASTRUCTURE ONLY.  Each call wraps the given pointers in the reference's
// VariableHandle (user-owned memory), submits one task through
// nntile::starpu::flash_sdpa_{fwd,bwd}_cudnn exactly as the reference's tile layer
// does (src/tile/flash_sdpa_fwd_cudnn.cc:175-190, src/tile/flash_sdpa_bwd_cudnn.cc:
// 104-130), and returns what the fake runtime recorded.
#include <cstdint>

#include <nntile/starpu/flash_sdpa_bwd_cudnn.hh>
#include <nntile/starpu/flash_sdpa_fwd_cudnn.hh>

namespace ns = nntile::starpu;
using nntile::bf16_t;
using nntile::fp16_t;
using nntile::Index;

static ns::Handle wrap(void *ptr, std::size_t bytes)
{
    return ns::VariableHandle(ptr, bytes);
}

template<typename T>
static int check_fwd(void *stream, int64_t seq, int64_t head, int64_t batch,
        void *K, void *Q, void *mask, void *lse, void *V, void *A, void *scratch_lse,
        void *scratch_A)
{
    starpu_fake_set_stream(stream);
    const std::size_t t = (std::size_t)seq*head*batch*2, l = (std::size_t)seq*batch*4;
    try
    {
        ns::flash_sdpa_fwd_cudnn.submit<std::tuple<T>>(seq, head, batch, wrap(K, t),
                wrap(Q, t), wrap(mask, (std::size_t)seq*seq*2), wrap(lse, l), wrap(V, t),
                wrap(A, t), wrap(scratch_lse, l), wrap(scratch_A, t));
    }
    catch(...)
    {
        return -100;
    }
    return starpu_fake_last_nbuffers();
}

template<typename T>
static int check_bwd(void *stream, int64_t seq, int64_t head, int64_t batch,
        void *K, void *Q, void *V, void *A, void *dA, void *mask, void *lse, void *dK,
        void *dQ, void *dV, void *scratch_dK, void *scratch_dQ, void *scratch_dV)
{
    starpu_fake_set_stream(stream);
    const std::size_t t = (std::size_t)seq*head*batch*2, l = (std::size_t)seq*batch*4;
    try
    {
        ns::flash_sdpa_bwd_cudnn.submit<std::tuple<T>>(seq, head, batch, wrap(K, t),
                wrap(Q, t), wrap(V, t), wrap(A, t), wrap(dA, t),
                wrap(mask, (std::size_t)seq*seq*2), wrap(lse, l), wrap(dK, t), wrap(dQ, t),
                wrap(dV, t), wrap(scratch_dK, t), wrap(scratch_dQ, t), wrap(scratch_dV, t));
    }
    catch(...)
    {
        return -100;
    }
    return starpu_fake_last_nbuffers();
}

// `fp16` selects the codelet instance for nntile::fp16_t instead of nntile::bf16_t
extern "C" int codelet_check_fwd(void *stream, int fp16, int64_t seq, int64_t head,
        int64_t batch, void *K, void *Q, void *mask, void *lse, void *V, void *A,
        void *scratch_lse, void *scratch_A)
{
    return fp16 ? check_fwd<fp16_t>(stream, seq, head, batch, K, Q, mask, lse, V, A, scratch_lse,
                          scratch_A)
                : check_fwd<bf16_t>(stream, seq, head, batch, K, Q, mask, lse, V, A, scratch_lse,
                          scratch_A);
}

extern "C" int codelet_check_bwd(void *stream, int fp16, int64_t seq, int64_t head,
        int64_t batch, void *K, void *Q, void *V, void *A, void *dA, void *mask, void *lse,
        void *dK, void *dQ, void *dV, void *scratch_dK, void *scratch_dQ, void *scratch_dV)
{
    return fp16 ? check_bwd<fp16_t>(stream, seq, head, batch, K, Q, V, A, dA, mask, lse, dK, dQ,
                          dV, scratch_dK, scratch_dQ, scratch_dV)
                : check_bwd<bf16_t>(stream, seq, head, batch, K, Q, V, A, dA, mask, lse, dK, dQ,
                          dV, scratch_dK, scratch_dQ, scratch_dV);
}

extern "C" uint32_t codelet_check_footprint(int fwd, int64_t seq, int64_t head, int64_t batch)
{
    return fwd ? ns::FlashSdpaFwdCudnn<std::tuple<bf16_t>>::hash_parameters(seq, head, batch)
               : ns::FlashSdpaBwdCudnn<std::tuple<bf16_t>>::hash_parameters(seq, head, batch);
}

extern "C" const char *codelet_check_name(int fwd, int fp16)
{
    if(fp16)
    {
        return fwd ? static_cast<ns::FlashSdpaFwdCudnn<std::tuple<fp16_t>> &>(
                             ns::flash_sdpa_fwd_cudnn).codelet.name
                   : static_cast<ns::FlashSdpaBwdCudnn<std::tuple<fp16_t>> &>(
                             ns::flash_sdpa_bwd_cudnn).codelet.name;
    }
    return fwd ? static_cast<ns::FlashSdpaFwdCudnn<std::tuple<bf16_t>> &>(
                         ns::flash_sdpa_fwd_cudnn).codelet.name
               : static_cast<ns::FlashSdpaBwdCudnn<std::tuple<bf16_t>> &>(
                         ns::flash_sdpa_bwd_cudnn).codelet.name;
}
