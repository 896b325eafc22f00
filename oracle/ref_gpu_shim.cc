// C-callable doors onto the reference's own GPU wrappers of the fused pair.
//
// TEST INFRASTRUCTURE ONLY.  Compiled by oracle/build.py together with the
// reference's src/kernel/flash_sdpa_{fwd,bwd}_cudnn/cuda.cc,
// src/kernel/accumulate_attn_output/cuda.cu and src/kernel/add_inplace/cuda.cu,
// taken from the reference checkout where they lie (nothing is copied), against
// the installed cuDNN and cudnn_frontend headers, into
// oracle/_ref_gpu/libnntile_ref_gpu.so.  It is the second parity witness of the
// fused pair (the reference's actual GPU arithmetic: cuDNN graph into scratch,
// then the merge / the three add_inplace passes) and the timing comparator of
// bench.py.  The shipped library never sees it.
//
// Graph handling follows the reference's codelets (src/starpu/
// flash_sdpa_fwd_cudnn.cc:74-125, flash_sdpa_bwd_cudnn.cc:80-105, 273-288): one
// graph per (seq, head, batch), prepared on first use and kept; the backward
// graph's workspace is allocated once with cudaMalloc and kept with it.
#include <cstdint>
#include <map>
#include <tuple>

#include <nntile/defs.h>
#include <nntile/base_types.hh>
#include <nntile/kernel/flash_sdpa_bwd_cudnn/cuda.hh>
#include <nntile/kernel/flash_sdpa_fwd_cudnn/cuda.hh>

namespace nk = nntile::kernel;
using nntile::bf16_t;
using nntile::fp32_t;
typedef std::int64_t i64;

typedef std::tuple<int, i64, i64, i64> Key;       // (fp16?, seq, head, batch)

struct BwdEntry
{
    nk::flash_sdpa_bwd_cudnn::FlashSdpaBwdGraph graph;
    void *workspace = nullptr;
};

static cudnnHandle_t g_handle = nullptr;
static std::map<Key, nk::flash_sdpa_fwd_cudnn::FlashSdpaFwdGraph> g_fwd;
static std::map<Key, BwdEntry> g_bwd;

static bool ensure_handle(void *stream)
{
    if(!g_handle && cudnnCreate(&g_handle) != CUDNN_STATUS_SUCCESS)
    {
        g_handle = nullptr;
        return false;
    }
    return cudnnSetStream(g_handle, static_cast<cudaStream_t>(stream)) == CUDNN_STATUS_SUCCESS;
}

// 0 = enqueued, 1 = no cuDNN handle, 2 = prepare_graph returned null
template<typename T>
static int run_fwd(int fp16, void *stream, i64 seq, i64 head, i64 batch,
        const void *K, const void *Q, const void *mask, void *scratch_lse, const void *V,
        void *scratch_A, void *lse, void *A)
{
    if(!ensure_handle(stream)) return 1;
    const Key key(fp16, seq, head, batch);
    auto it = g_fwd.find(key);
    if(it == g_fwd.end())
    {
        auto graph = nk::flash_sdpa_fwd_cudnn::prepare_graph<T>(g_handle, seq, head, batch);
        if(!graph) return 2;
        it = g_fwd.emplace(key, graph).first;
    }
    nk::flash_sdpa_fwd_cudnn::execute_graph<T>(g_handle, it->second, seq, head, batch,
            static_cast<const T *>(K), static_cast<const T *>(Q),
            static_cast<const T *>(mask), static_cast<fp32_t *>(scratch_lse),
            static_cast<const T *>(V), static_cast<T *>(scratch_A),
            static_cast<fp32_t *>(lse), static_cast<T *>(A));
    return 0;
}

template<typename T>
static int run_bwd(int fp16, void *stream, i64 seq, i64 head, i64 batch,
        const void *K, const void *Q, const void *V, const void *A, const void *dA,
        const void *mask, const void *lse, void *scratch_dK, void *scratch_dQ,
        void *scratch_dV, void *dK, void *dQ, void *dV)
{
    if(!ensure_handle(stream)) return 1;
    const Key key(fp16, seq, head, batch);
    auto it = g_bwd.find(key);
    if(it == g_bwd.end())
    {
        BwdEntry e;
        e.graph = nk::flash_sdpa_bwd_cudnn::prepare_graph<T>(g_handle, seq, head, batch);
        if(!e.graph) return 2;
        ::int64_t ws = 0;
        if(!e.graph->get_workspace_size(ws).is_good()) return 3;
        if(ws > 0 && cudaMalloc(&e.workspace, (size_t)ws) != cudaSuccess) return 3;
        it = g_bwd.emplace(key, e).first;
    }
    nk::flash_sdpa_bwd_cudnn::execute_graph<T>(g_handle, it->second.graph, seq, head,
            batch, static_cast<const T *>(K), static_cast<const T *>(Q),
            static_cast<const T *>(V), static_cast<const T *>(A),
            static_cast<const T *>(dA), static_cast<const T *>(mask),
            static_cast<const fp32_t *>(lse), static_cast<T *>(scratch_dK),
            static_cast<T *>(scratch_dQ), static_cast<T *>(scratch_dV),
            static_cast<T *>(dK), static_cast<T *>(dQ), static_cast<T *>(dV),
            it->second.workspace);
    return 0;
}

#define REFGPU(suffix, TYPE, FLAG) \
extern "C" int refgpu_flash_sdpa_fwd_##suffix(void *stream, i64 seq, i64 head, i64 batch, \
        const void *K, const void *Q, const void *mask, void *scratch_lse, const void *V, \
        void *scratch_A, void *lse, void *A) \
{ \
    return run_fwd<TYPE>(FLAG, stream, seq, head, batch, K, Q, mask, scratch_lse, V, scratch_A, \
            lse, A); \
} \
extern "C" int refgpu_flash_sdpa_bwd_##suffix(void *stream, i64 seq, i64 head, i64 batch, \
        const void *K, const void *Q, const void *V, const void *A, const void *dA, \
        const void *mask, const void *lse, void *scratch_dK, void *scratch_dQ, \
        void *scratch_dV, void *dK, void *dQ, void *dV) \
{ \
    return run_bwd<TYPE>(FLAG, stream, seq, head, batch, K, Q, V, A, dA, mask, lse, scratch_dK, \
            scratch_dQ, scratch_dV, dK, dQ, dV); \
}

REFGPU(bf16, bf16_t, 0)
REFGPU(fp16, nntile::fp16_t, 1)
