// Host-side tile loops of the fused path: the part of the reference's tensor
// layer that turns one call on tiled tensors into (Q tile, K/V tile) tasks.
// No device code here.
//
// Follows src/tensor/flash_sdpa_fwd_cudnn.cc:148-274 (checks and loops),
// src/tile/flash_sdpa_fwd_cudnn.cc:170-173 (batch = product of the three batch
// extents of the tile) and src/tensor/flash_sdpa_bwd_cudnn.cc:172-246.
//
// The reference hands every pair to StarPU as one task and lets the runtime
// overlap tasks that touch different output tiles.  Here the same dependency
// structure is laid on CUDA streams: the caller's stream forks into a small
// per-device pool of helper streams and joins again before the call returns, so
// from outside everything is still "enqueued on the caller's stream".
//   forward   tasks of one Q tile run in K/V-tile order on one helper stream (they
//             merge into the same (lse, A)); different Q tiles run side by side.
//   backward  tasks that add into the same dK/dV tile run in Q-tile order on one
//             helper stream, so the elem_t "+=" into dK, dV happens in the reference's
//             order; dQ of a Q tile is summed in fp32 over all its K/V tiles
//             (red.add, any order) and rounded into dQ once, after the join.
// Work shared by the tasks of a call is done once: every distinct mask buffer is
// classified once, delta / lse*log2e of a Q tile are computed once.
// Tile shapes the tcgen05 kernels do not take run the generic kernels task by
// task on the caller's stream.
#include <mutex>
#include <vector>

#include "flash.cuh"
#include "per_device.hh"

namespace nb200 {
inline namespace NB200_ELEM_NS {

struct Grid5
{
    Index shape[5], tile[5], grid[5];
    Index ntiles;
};

static bool make_grid(const int64_t *shape, const int64_t *basetile, Grid5 &g)
{
    g.ntiles = 1;
    for(int d = 0; d < 5; ++d)
    {
        if(shape[d] <= 0 || basetile[d] <= 0 || basetile[d] > shape[d]) return false;
        g.shape[d] = shape[d];
        g.tile[d] = basetile[d];
        g.grid[d] = (shape[d] + basetile[d] - 1)/basetile[d];
        g.ntiles *= g.grid[d];
    }
    return true;
}

// extent of tile `idx` along dimension d (ragged at the upper edge)
static Index extent(const Grid5 &g, int d, Index idx)
{
    const Index lo = idx*g.tile[d];
    return (lo + g.tile[d] <= g.shape[d]) ? g.tile[d] : g.shape[d] - lo;
}

static void unravel(const Grid5 &g, Index a, Index idx[5])
{
    for(int d = 0; d < 5; ++d)
    {
        idx[d] = a % g.grid[d];
        a /= g.grid[d];
    }
}

// Linear index of the K/V tile that output tile `idx` meets at sequence tile ki.
// Plain form: K, V are tiled like Q.  Grouped-query form: K, V are
// [head, seq, batch, kv_heads] tensors tiled [head, seq_tile, batch_tile, kv_tile].
static Index kv_tile_index(const Grid5 &g, const Index idx[5], Index ki, bool gqa)
{
    if(gqa)
    {
        return ki + g.grid[1]*(idx[2] + g.grid[2]*idx[4]);
    }
    return ki + g.grid[1]*(idx[2] + g.grid[2]*(idx[3] + g.grid[3]*idx[4]));
}

// ------------------------------------------------------------- scratch layout
constexpr size_t HDR_BYTES = 4096;          // sticky status word at offset 0

static size_t align256(size_t x)
{
    return (x + 255) & ~(size_t)255;
}

struct Layout
{
    size_t cls_off, cls_slot, stats_off, acc_off, total;
    size_t generic_total;
};

static Layout make_layout(const Grid5 &g)
{
    Layout L;
    const size_t nblk_t = (size_t)((g.tile[1] + 127)/128);
    L.cls_slot = nblk_t*nblk_t;
    L.cls_off = HDR_BYTES;
    const size_t nseq = (size_t)g.grid[1];
    L.stats_off = L.cls_off + align256(L.cls_slot*nseq*nseq);
    const size_t rows = (size_t)g.shape[1]*g.shape[2]*g.shape[3]*g.shape[4];
    L.acc_off = L.stats_off + align256(rows*8);
    L.total = L.acc_off + align256(rows*(size_t)g.shape[0]*4);
    const size_t tile_bytes =
            align256((size_t)g.tile[0]*g.tile[1]*g.tile[2]*g.tile[3]*g.tile[4]*2);
    L.generic_total = HDR_BYTES + 3*tile_bytes;
    if(L.total < L.generic_total) L.total = L.generic_total;
    return L;
}

// --------------------------------------------------------- helper stream pool
constexpr int POOL_STREAMS = 8;

struct StreamPool
{
    cudaStream_t stream[POOL_STREAMS];
    cudaEvent_t fork, join[POOL_STREAMS];
    std::mutex lock;            // one enqueueing host thread per device at a time
};

static StreamPool g_pools[PerDeviceOnce::MAX_DEVICES];
static PerDeviceOnce g_pool_once;

// Helper streams and events of the current device, created on first use.
static StreamPool *pool_for_current_device()
{
    int dev = -1;
    if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PerDeviceOnce::MAX_DEVICES)
    {
        return nullptr;
    }
    static std::mutex create_lock;
    std::lock_guard<std::mutex> guard(create_lock);
    const bool ok = g_pool_once.ensure(dev, [dev]() {
        StreamPool &p = g_pools[dev];
        if(cudaEventCreateWithFlags(&p.fork, cudaEventDisableTiming) != cudaSuccess) return false;
        for(int i = 0; i < POOL_STREAMS; ++i)
        {
            if(cudaStreamCreateWithFlags(&p.stream[i], cudaStreamNonBlocking) != cudaSuccess
                    || cudaEventCreateWithFlags(&p.join[i], cudaEventDisableTiming) != cudaSuccess)
            {
                return false;
            }
        }
        return true;
    });
    return ok ? &g_pools[dev] : nullptr;
}

// Fork the caller's stream into the pool, run `body(stream_of)`, join again.
class ForkJoin
{
public:
    ForkJoin(cudaStream_t caller, bool parallel): caller_(caller), pool_(nullptr), used_(0)
    {
        if(parallel)
        {
            pool_ = pool_for_current_device();
        }
        if(pool_)
        {
            pool_->lock.lock();
            if(cudaEventRecord(pool_->fork, caller_) != cudaSuccess)
            {
                pool_->lock.unlock();
                pool_ = nullptr;
            }
        }
    }
    // stream on which work of lane `key` is enqueued
    cudaStream_t lane(Index key)
    {
        if(!pool_) return caller_;
        const int i = (int)(key % POOL_STREAMS);
        if(!(used_ & (1u << i)))
        {
            cudaStreamWaitEvent(pool_->stream[i], pool_->fork, 0);
            used_ |= 1u << i;
        }
        return pool_->stream[i];
    }
    // every lane's work precedes whatever the caller enqueues next
    void join()
    {
        if(!pool_) return;
        for(int i = 0; i < POOL_STREAMS; ++i)
        {
            if(used_ & (1u << i))
            {
                cudaEventRecord(pool_->join[i], pool_->stream[i]);
                cudaStreamWaitEvent(caller_, pool_->join[i], 0);
            }
        }
        used_ = 0;
        pool_->lock.unlock();
        pool_ = nullptr;
    }
    ~ForkJoin() { join(); }

private:
    cudaStream_t caller_;
    StreamPool *pool_;
    unsigned used_;
};

// Classify every distinct mask buffer once; slot_of[pair] = class table of the pair.
static int classify_masks(cudaStream_t s, const Grid5 &g, const void *const *mask_tiles,
        uint8_t *cls_base, size_t cls_slot, std::vector<uint8_t *> &slot_of)
{
    const Index nseq = g.grid[1];
    slot_of.assign((size_t)(nseq*nseq), nullptr);
    std::vector<std::pair<const void *, uint8_t *>> seen;
    for(Index p = 0; p < nseq*nseq; ++p)
    {
        const void *m = mask_tiles[p];
        if(!m) continue;
        uint8_t *slot = nullptr;
        for(const auto &e : seen)
        {
            if(e.first == m)
            {
                slot = e.second;
                break;
            }
        }
        if(!slot)
        {
            if(!aligned16(m)) return NNTILE_B200_E_ALIGN;
            slot = cls_base + (size_t)p*cls_slot;
            const int st = launch_mask_classify(s, (int)g.tile[1], (const elem_t *)m, slot, nullptr);
            if(st != NNTILE_B200_OK) return st;
            seen.emplace_back(m, slot);
        }
        slot_of[(size_t)p] = slot;
    }
    return NNTILE_B200_OK;
}

// All sequence tiles must have the same length (the reference rejects a pair whose
// K tile and Q tile differ, src/tensor/flash_sdpa_fwd_cudnn.cc:258-261) for the
// batched path; a ragged last tile goes task by task and is rejected there.
static bool uniform_seq(const Grid5 &g)
{
    return g.shape[1] % g.tile[1] == 0;
}

static int tensor_fwd(cudaStream_t stream, const int64_t *shape, const int64_t *basetile,
        const void *const *K_tiles, const void *const *Q_tiles, const void *const *mask_tiles,
        float *const *lse_tiles, const void *const *V_tiles, void *const *A_tiles,
        void *scratch, size_t scratch_bytes, bool gqa)
{
    Grid5 g;
    if(!shape || !basetile || !K_tiles || !Q_tiles || !mask_tiles || !lse_tiles
            || !V_tiles || !A_tiles || !make_grid(shape, basetile, g))
    {
        return NNTILE_B200_E_BADARG;
    }
    // head dimension must not be tiled (src/tensor/flash_sdpa_fwd_cudnn.cc:194-199)
    if(g.grid[0] != 1) return NNTILE_B200_E_SHAPE;
    const Layout L = make_layout(g);
    if(!scratch || scratch_bytes < L.total) return NNTILE_B200_E_SCRATCH;
    if((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return NNTILE_B200_E_ALIGN;
    const Index nseq = g.grid[1];
    uint8_t *base = static_cast<uint8_t *>(scratch);
    const Index full_batch = g.tile[2]*g.tile[3]*g.tile[4];
    const bool fast = uniform_seq(g) && flash_fwd_sm100_supports(g.tile[1], g.shape[0], full_batch);
    if(gqa && !fast) return NNTILE_B200_E_SHAPE;
    std::vector<uint8_t *> slot_of;
    if(fast)
    {
        if(cudaMemsetAsync(base, 0, 256, stream) != cudaSuccess) return NNTILE_B200_E_LAUNCH;
        const int st = classify_masks(stream, g, mask_tiles, base + L.cls_off, L.cls_slot, slot_of);
        if(st != NNTILE_B200_OK) return st;
    }
    ForkJoin fj(stream, fast && g.ntiles > 1);
    float *scratch_lse = reinterpret_cast<float *>(base + HDR_BYTES);   // generic path only
    void *scratch_A = base + HDR_BYTES;
    for(Index a = 0; a < g.ntiles; ++a)
    {
        Index idx[5];
        unravel(g, a, idx);           // Fortran order of the tile grid: index 0 fastest
        const Index qi = idx[1];
        const Index seq_q = extent(g, 1, qi);
        const Index bt = extent(g, 2, idx[2]), gt = extent(g, 3, idx[3]), ht = extent(g, 4, idx[4]);
        const Index batch = bt*gt*ht;
        // the lse tile grid is the A grid without the head axis: same linear index
        cudaStream_t s = fj.lane(a);
        for(Index ki = 0; ki < nseq; ++ki)
        {
            if(extent(g, 1, ki) != seq_q)
            {
                return NNTILE_B200_E_SHAPE;   // "K tile sequence length mismatches Q tile"
            }
            const void *m = mask_tiles[ki + qi*nseq];
            if(!m)
            {
                continue;   // the caller marked this pair as fully masked: no task
            }
            const Index kv = kv_tile_index(g, idx, ki, gqa);
            int st;
            if(fast)
            {
                if(!K_tiles[kv] || !Q_tiles[a] || !V_tiles[kv] || !lse_tiles[a] || !A_tiles[a])
                {
                    return NNTILE_B200_E_BADARG;
                }
                if(!aligned16(K_tiles[kv]) || !aligned16(Q_tiles[a]) || !aligned16(V_tiles[kv])
                        || !aligned16(A_tiles[a]))
                {
                    return NNTILE_B200_E_ALIGN;
                }
                const FwdAux aux = {reinterpret_cast<uint32_t *>(base),
                        slot_of[(size_t)(ki + qi*nseq)], false};
                st = flash_fwd_sm100(s, seq_q, g.shape[0], batch, (const elem_t *)K_tiles[kv],
                        (const elem_t *)Q_tiles[a], (const elem_t *)m, (const elem_t *)V_tiles[kv],
                        lse_tiles[a], (elem_t *)A_tiles[a], aux, gqa ? gt : 1, gqa ? bt : batch);
            }
            else
            {
                st = flash_fwd_task(s, seq_q, g.shape[0], batch, K_tiles[kv], Q_tiles[a], m,
                        V_tiles[kv], scratch_A, lse_tiles[a], A_tiles[a], nullptr);
                (void)scratch_lse;
            }
            if(st != NNTILE_B200_OK) return st;
        }
    }
    fj.join();
    return NNTILE_B200_OK;
}

static int tensor_bwd(cudaStream_t stream, const int64_t *shape, const int64_t *basetile,
        const void *const *K_tiles, const void *const *Q_tiles, const void *const *V_tiles,
        const void *const *A_tiles, const void *const *dA_tiles, const void *const *mask_tiles,
        const float *const *lse_tiles, void *const *dK_tiles, void *const *dQ_tiles,
        void *const *dV_tiles, void *scratch, size_t scratch_bytes, bool gqa)
{
    Grid5 g;
    if(!shape || !basetile || !K_tiles || !Q_tiles || !V_tiles || !A_tiles || !dA_tiles
            || !mask_tiles || !lse_tiles || !dK_tiles || !dQ_tiles || !dV_tiles
            || !make_grid(shape, basetile, g))
    {
        return NNTILE_B200_E_BADARG;
    }
    if(g.grid[0] != 1) return NNTILE_B200_E_SHAPE;
    const Layout L = make_layout(g);
    if(!scratch || scratch_bytes < L.total) return NNTILE_B200_E_SCRATCH;
    if((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return NNTILE_B200_E_ALIGN;
    const Index nseq = g.grid[1];
    uint8_t *base = static_cast<uint8_t *>(scratch);
    const Index full_batch = g.tile[2]*g.tile[3]*g.tile[4];
    const Index D = g.shape[0];
    const bool fast = uniform_seq(g) && flash_bwd_sm100_supports(g.tile[1], D, full_batch);
    if(gqa && !fast) return NNTILE_B200_E_SHAPE;
    if(!fast)
    {
        // generic kernels, one whole task after the other on the caller's stream
        const size_t tile_bytes = (L.generic_total - HDR_BYTES)/3;
        for(Index a = 0; a < g.ntiles; ++a)
        {
            Index idx[5];
            unravel(g, a, idx);
            const Index qi = idx[1];
            const Index seq_q = extent(g, 1, qi);
            const Index batch = extent(g, 2, idx[2])*extent(g, 3, idx[3])*extent(g, 4, idx[4]);
            for(Index ki = 0; ki < nseq; ++ki)
            {
                if(extent(g, 1, ki) != seq_q) return NNTILE_B200_E_SHAPE;
                const void *m = mask_tiles[ki + qi*nseq];
                if(!m)
                {
                    continue;   // fully masked pair: contributes nothing to any gradient
                }
                const Index kv = kv_tile_index(g, idx, ki, false);
                const int st = flash_bwd_task(stream, seq_q, D, batch, K_tiles[kv], Q_tiles[a],
                        V_tiles[kv], A_tiles[a], dA_tiles[a], m, lse_tiles[a],
                        base + HDR_BYTES, base + HDR_BYTES + tile_bytes,
                        base + HDR_BYTES + 2*tile_bytes, dK_tiles[kv], dQ_tiles[a], dV_tiles[kv],
                        nullptr);
                if(st != NNTILE_B200_OK) return st;
            }
        }
        return NNTILE_B200_OK;
    }
    if(cudaMemsetAsync(base, 0, 256, stream) != cudaSuccess) return NNTILE_B200_E_LAUNCH;
    std::vector<uint8_t *> slot_of;
    int st = classify_masks(stream, g, mask_tiles, base + L.cls_off, L.cls_slot, slot_of);
    if(st != NNTILE_B200_OK) return st;
    // per output tile: its rows of delta / lse2 and of the fp32 dQ accumulator
    std::vector<BwdAux> aux((size_t)g.ntiles);
    std::vector<char> live((size_t)g.ntiles, 0);
    float *stats = reinterpret_cast<float *>(base + L.stats_off);
    float *acc = reinterpret_cast<float *>(base + L.acc_off);
    size_t row_off = 0;
    for(Index a = 0; a < g.ntiles; ++a)
    {
        Index idx[5];
        unravel(g, a, idx);
        const Index qi = idx[1];
        const Index seq_q = extent(g, 1, qi);
        const Index batch = extent(g, 2, idx[2])*extent(g, 3, idx[3])*extent(g, 4, idx[4]);
        const size_t rows = (size_t)seq_q*batch;
        BwdAux &x = aux[(size_t)a];
        x.status = reinterpret_cast<uint32_t *>(base);
        x.cls = base + L.cls_off;                       // per pair, set below
        x.delta = stats + 2*row_off;
        x.lse2 = x.delta + rows;
        x.acc_lo = acc + row_off*(size_t)D;
        x.acc_hi = x.acc_lo;
        x.half_rows = (Index)rows;                      // the whole tile in one buffer
        x.phases = BWD_PREP;
        row_off += rows;
        for(Index ki = 0; ki < nseq; ++ki)
        {
            if(mask_tiles[ki + qi*nseq]) live[(size_t)a] = 1;
        }
        if(!live[(size_t)a]) continue;                  // nothing reaches this Q tile
        if(!Q_tiles[a] || !A_tiles[a] || !dA_tiles[a] || !lse_tiles[a] || !dQ_tiles[a])
        {
            return NNTILE_B200_E_BADARG;
        }
        if(!aligned16(Q_tiles[a]) || !aligned16(A_tiles[a]) || !aligned16(dA_tiles[a])
                || !aligned16(dQ_tiles[a]))
        {
            return NNTILE_B200_E_ALIGN;
        }
        // K, V, mask are not touched by this phase
        st = flash_bwd_sm100(stream, seq_q, D, batch, (const elem_t *)Q_tiles[a],
                (const elem_t *)Q_tiles[a], (const elem_t *)Q_tiles[a], (const elem_t *)A_tiles[a],
                (const elem_t *)dA_tiles[a], (const elem_t *)Q_tiles[a], lse_tiles[a], x,
                (elem_t *)dQ_tiles[a], (elem_t *)dQ_tiles[a], (elem_t *)dQ_tiles[a], 1, batch);
        if(st != NNTILE_B200_OK) return st;
    }
    {
        ForkJoin fj(stream, true);
        for(Index a = 0; a < g.ntiles; ++a)
        {
            if(!live[(size_t)a]) continue;
            Index idx[5];
            unravel(g, a, idx);
            const Index qi = idx[1];
            const Index seq_q = extent(g, 1, qi);
            const Index bt = extent(g, 2, idx[2]), gt = extent(g, 3, idx[3]);
            const Index batch = bt*gt*extent(g, 4, idx[4]);
            for(Index ki = 0; ki < nseq; ++ki)
            {
                if(extent(g, 1, ki) != seq_q) return NNTILE_B200_E_SHAPE;
                const void *m = mask_tiles[ki + qi*nseq];
                if(!m) continue;
                const Index kv = kv_tile_index(g, idx, ki, gqa);
                if(!K_tiles[kv] || !V_tiles[kv] || !dK_tiles[kv] || !dV_tiles[kv])
                {
                    return NNTILE_B200_E_BADARG;
                }
                if(!aligned16(K_tiles[kv]) || !aligned16(V_tiles[kv]) || !aligned16(dK_tiles[kv])
                        || !aligned16(dV_tiles[kv]))
                {
                    return NNTILE_B200_E_ALIGN;
                }
                BwdAux x = aux[(size_t)a];
                x.cls = slot_of[(size_t)(ki + qi*nseq)];
                x.phases = BWD_MAIN;
                st = flash_bwd_sm100(fj.lane(kv), seq_q, D, batch, (const elem_t *)K_tiles[kv],
                        (const elem_t *)Q_tiles[a], (const elem_t *)V_tiles[kv],
                        (const elem_t *)A_tiles[a], (const elem_t *)dA_tiles[a], (const elem_t *)m,
                        lse_tiles[a], x, (elem_t *)dK_tiles[kv], (elem_t *)dQ_tiles[a],
                        (elem_t *)dV_tiles[kv], gqa ? gt : 1, gqa ? bt : batch);
                if(st != NNTILE_B200_OK) return st;
            }
        }
        fj.join();
    }
    for(Index a = 0; a < g.ntiles; ++a)
    {
        if(!live[(size_t)a]) continue;
        Index idx[5];
        unravel(g, a, idx);
        const Index seq_q = extent(g, 1, idx[1]);
        const Index batch = extent(g, 2, idx[2])*extent(g, 3, idx[3])*extent(g, 4, idx[4]);
        BwdAux x = aux[(size_t)a];
        x.phases = BWD_FINISH;
        st = flash_bwd_sm100(stream, seq_q, D, batch, (const elem_t *)Q_tiles[a],
                (const elem_t *)Q_tiles[a], (const elem_t *)Q_tiles[a], (const elem_t *)A_tiles[a],
                (const elem_t *)dA_tiles[a], (const elem_t *)Q_tiles[a], lse_tiles[a], x,
                (elem_t *)dQ_tiles[a], (elem_t *)dQ_tiles[a], (elem_t *)dQ_tiles[a], 1, batch);
        if(st != NNTILE_B200_OK) return st;
    }
    return NNTILE_B200_OK;
}

} // inline namespace
} // namespace nb200

using namespace nb200;

extern "C" int NB200_SFX(nntile_b200_tensor_flash_sdpa_fwd)(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles, float *const *lse_tiles,
        const void *const *V_tiles, void *const *A_tiles, void *scratch,
        size_t scratch_bytes)
{
    return tensor_fwd(as_stream(stream), shape, basetile, K_tiles, Q_tiles, mask_tiles,
            lse_tiles, V_tiles, A_tiles, scratch, scratch_bytes, false);
}

extern "C" int NB200_SFX(nntile_b200_tensor_flash_sdpa_bwd)(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles, const void *const *A_tiles,
        const void *const *dA_tiles, const void *const *mask_tiles,
        const float *const *lse_tiles, void *const *dK_tiles, void *const *dQ_tiles,
        void *const *dV_tiles, void *scratch, size_t scratch_bytes)
{
    return tensor_bwd(as_stream(stream), shape, basetile, K_tiles, Q_tiles, V_tiles, A_tiles,
            dA_tiles, mask_tiles, lse_tiles, dK_tiles, dQ_tiles, dV_tiles, scratch,
            scratch_bytes, false);
}

extern "C" int NB200_SFX(nntile_b200_tensor_flash_sdpa_fwd_gqa)(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles, float *const *lse_tiles,
        const void *const *V_tiles, void *const *A_tiles, void *scratch,
        size_t scratch_bytes)
{
    return tensor_fwd(as_stream(stream), shape, basetile, K_tiles, Q_tiles, mask_tiles,
            lse_tiles, V_tiles, A_tiles, scratch, scratch_bytes, true);
}

extern "C" int NB200_SFX(nntile_b200_tensor_flash_sdpa_bwd_gqa)(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles, const void *const *A_tiles,
        const void *const *dA_tiles, const void *const *mask_tiles,
        const float *const *lse_tiles, void *const *dK_tiles, void *const *dQ_tiles,
        void *const *dV_tiles, void *scratch, size_t scratch_bytes)
{
    return tensor_bwd(as_stream(stream), shape, basetile, K_tiles, Q_tiles, V_tiles, A_tiles,
            dA_tiles, mask_tiles, lse_tiles, dK_tiles, dQ_tiles, dV_tiles, scratch,
            scratch_bytes, true);
}

#ifndef NB200_FP16
extern "C" size_t nntile_b200_tensor_flash_sdpa_scratch_bytes(const int64_t *shape,
        const int64_t *basetile)
{
    Grid5 g;
    if(!shape || !basetile || !make_grid(shape, basetile, g)) return 0;
    return make_layout(g).total;
}
#endif // NB200_FP16
