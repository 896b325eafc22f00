// Host-side tile loops of the fused path: the part of the reference's tensor
// layer that turns one call on tiled tensors into (Q tile, K/V tile) tasks.
// No device code here; every task is one call of the tile-level entry point on
// the caller's stream, so tasks that share an output tile run in submission
// order exactly as StarPU's read-write dependency on (lse, A) / (dK, dQ, dV)
// makes them in the reference.
//
// Follows src/tensor/flash_sdpa_fwd_cudnn.cc:148-274 (checks and loops),
// src/tile/flash_sdpa_fwd_cudnn.cc:170-173 (batch = product of the three batch
// extents of the tile) and src/tensor/flash_sdpa_bwd_cudnn.cc:172-246.
#include <vector>

#include "common.cuh"

namespace nb200 {

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

} // namespace nb200

using namespace nb200;

extern "C" int nntile_b200_tensor_flash_sdpa_fwd_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *mask_tiles, float *const *lse_tiles,
        const void *const *V_tiles, void *const *A_tiles, void *scratch,
        size_t scratch_bytes)
{
    Grid5 g;
    if(!shape || !basetile || !K_tiles || !Q_tiles || !mask_tiles || !lse_tiles
            || !V_tiles || !A_tiles || !make_grid(shape, basetile, g))
    {
        return NNTILE_B200_E_BADARG;
    }
    // head dimension must not be tiled (src/tensor/flash_sdpa_fwd_cudnn.cc:194-199)
    if(g.grid[0] != 1) return NNTILE_B200_E_SHAPE;
    const Index nseq = g.grid[1];
    const size_t tile_elems = (size_t)g.tile[0]*g.tile[1]*g.tile[2]*g.tile[3]*g.tile[4];
    const size_t lse_bytes = ((tile_elems/g.tile[0])*sizeof(float) + 255) & ~(size_t)255;
    if(!scratch || scratch_bytes < lse_bytes + tile_elems*2) return NNTILE_B200_E_SCRATCH;
    float *scratch_lse = static_cast<float *>(scratch);
    void *scratch_A = static_cast<char *>(scratch) + lse_bytes;
    for(Index a = 0; a < g.ntiles; ++a)
    {
        // Fortran order of the tile grid: index 0 fastest
        Index rem = a, idx[5];
        for(int d = 0; d < 5; ++d)
        {
            idx[d] = rem % g.grid[d];
            rem /= g.grid[d];
        }
        const Index qi = idx[1];
        const Index seq_q = extent(g, 1, qi);
        const Index batch = extent(g, 2, idx[2])*extent(g, 3, idx[3])*extent(g, 4, idx[4]);
        // lse tile grid is the A grid without the head axis
        const Index l = a;   // grid[0] == 1, so the linear indices coincide
        for(Index ki = 0; ki < nseq; ++ki)
        {
            if(extent(g, 1, ki) != seq_q)
            {
                return NNTILE_B200_E_SHAPE;   // "K tile sequence length mismatches Q tile"
            }
            if(!mask_tiles[ki + qi*nseq])
            {
                continue;   // the caller marked this pair as fully masked: no task
            }
            const Index kv = a + (ki - qi)*g.grid[0];
            const int st = nntile_b200_flash_sdpa_fwd_bf16(stream, seq_q, g.shape[0], batch,
                    K_tiles[kv], Q_tiles[a], mask_tiles[ki + qi*nseq], scratch_lse,
                    V_tiles[kv], scratch_A, lse_tiles[l], A_tiles[a]);
            if(st != NNTILE_B200_OK) return st;
        }
    }
    return NNTILE_B200_OK;
}

extern "C" int nntile_b200_tensor_flash_sdpa_bwd_bf16(nntile_b200_stream_t stream,
        const int64_t *shape, const int64_t *basetile, const void *const *K_tiles,
        const void *const *Q_tiles, const void *const *V_tiles, const void *const *A_tiles,
        const void *const *dA_tiles, const void *const *mask_tiles,
        const float *const *lse_tiles, void *const *dK_tiles, void *const *dQ_tiles,
        void *const *dV_tiles, void *scratch, size_t scratch_bytes)
{
    Grid5 g;
    if(!shape || !basetile || !K_tiles || !Q_tiles || !V_tiles || !A_tiles || !dA_tiles
            || !mask_tiles || !lse_tiles || !dK_tiles || !dQ_tiles || !dV_tiles
            || !make_grid(shape, basetile, g))
    {
        return NNTILE_B200_E_BADARG;
    }
    if(g.grid[0] != 1) return NNTILE_B200_E_SHAPE;
    const Index nseq = g.grid[1];
    const size_t tile_bytes =
            ((size_t)g.tile[0]*g.tile[1]*g.tile[2]*g.tile[3]*g.tile[4]*2 + 255) & ~(size_t)255;
    if(!scratch || scratch_bytes < 3*tile_bytes) return NNTILE_B200_E_SCRATCH;
    char *base = static_cast<char *>(scratch);
    for(Index a = 0; a < g.ntiles; ++a)
    {
        Index rem = a, idx[5];
        for(int d = 0; d < 5; ++d)
        {
            idx[d] = rem % g.grid[d];
            rem /= g.grid[d];
        }
        const Index qi = idx[1];
        const Index seq_q = extent(g, 1, qi);
        const Index batch = extent(g, 2, idx[2])*extent(g, 3, idx[3])*extent(g, 4, idx[4]);
        for(Index ki = 0; ki < nseq; ++ki)
        {
            if(extent(g, 1, ki) != seq_q) return NNTILE_B200_E_SHAPE;
            if(!mask_tiles[ki + qi*nseq])
            {
                continue;   // fully masked pair: contributes nothing to any gradient
            }
            const Index kv = a + (ki - qi)*g.grid[0];
            const int st = nntile_b200_flash_sdpa_bwd_bf16(stream, seq_q, g.shape[0], batch,
                    K_tiles[kv], Q_tiles[a], V_tiles[kv], A_tiles[a], dA_tiles[a],
                    mask_tiles[ki + qi*nseq], lse_tiles[a], base, base + tile_bytes,
                    base + 2*tile_bytes, dK_tiles[kv], dQ_tiles[a], dV_tiles[kv]);
            if(st != NNTILE_B200_OK) return st;
        }
    }
    return NNTILE_B200_OK;
}

extern "C" size_t nntile_b200_tensor_flash_sdpa_scratch_bytes(const int64_t *basetile)
{
    if(!basetile) return 0;
    size_t elems = 1;
    for(int d = 0; d < 5; ++d)
    {
        if(basetile[d] <= 0) return 0;
        elems *= (size_t)basetile[d];
    }
    const size_t tile_bytes = (elems*2 + 255) & ~(size_t)255;
    return 3*tile_bytes + 4096;
}
