"""Seeded sweep of shapes and mask structures through the tcgen05 tile tasks
against the oracle: odd numbers of 128-blocks, block-sparse masks (whole blocks
of -inf in arbitrary places, fully masked query tiles and key blocks), finite
biases, several batch sizes - the cases that exercise the block lists, the stage
hand-backs and the skip paths of the kernels.  bf16 bar 2e-2 as everywhere."""
import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import flash_sdpa_bwd_async, flash_sdpa_fwd_async, from_fortran, to_fortran

pytestmark = pytest.mark.gpu
F = np.asfortranarray
TOL = 2e-2


def block_sparse_mask(S, rng, kind):
    nb = S//128
    k, q = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")     # Fortran [k, q]
    m = np.zeros((S, S), np.float32)
    if kind in ("causal", "causal_sparse", "causal_bias"):
        m[k > q] = -np.inf
    if kind in ("sparse", "causal_sparse"):
        drop = rng.random((nb, nb)) < 0.35                            # [key block, query block]
        if kind == "causal_sparse":
            drop[np.arange(nb), np.arange(nb)] = False                # keep the diagonal
        m[np.kron(drop, np.ones((128, 128), bool))] = -np.inf
    if kind == "causal_bias":
        fin = np.isfinite(m)
        m[fin] = (rng.standard_normal((S, S)).astype(np.float32)*0.3)[fin]
    if kind == "dead_tiles":
        m[:, 128:256] = -np.inf                                       # query block 1 sees nothing
        m[0:128, :] = -np.inf                                         # key block 0 is seen by nobody
    return F(m)


CASES = [
    (128, 128, 1, "causal"), (128, 384, 2, "causal_sparse"), (128, 640, 1, "sparse"),
    (64, 384, 3, "causal_bias"), (64, 640, 2, "causal_sparse"), (128, 384, 1, "dead_tiles"),
    (64, 256, 5, "sparse"), (128, 256, 3, "causal_bias"),
]


@pytest.mark.parametrize("head,seq,batch,kind", CASES)
def test_block_structures_against_oracle(head, seq, batch, kind):
    rng = np.random.default_rng(1000 + head + seq + batch)
    shape = (head, seq, batch, 1, 1)
    assert ops.flash_sdpa_path(seq, head, batch) == 2                 # the tcgen05 kernels
    Q, K, V, dA = (O.to_bf16(F(rng.standard_normal(shape).astype(np.float32))) for _ in range(4))
    mask = O.to_bf16(block_sparse_mask(seq, rng, kind))
    wantA, wantL = O.flash_forward(Q, K, V, mask)
    q, k, v, m = (from_fortran(x) for x in (Q, K, V, mask))
    lse = torch.full((1, 1, batch, seq), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    flash_sdpa_fwd_async(k, q, m, lse, v, A)
    torch.cuda.synchronize()
    fin = np.isfinite(wantL)
    gl = to_fortran(lse)
    assert np.array_equal(np.isfinite(gl), fin)
    assert np.allclose(gl[fin], wantL[fin], rtol=1e-3, atol=1e-3)
    assert O.rel_err(O.from_bf16(to_fortran(A)), O.from_bf16(wantA)) <= TOL
    z = lambda: O.zeros(shape, np.uint16)
    lse_in = F(np.where(fin, wantL, 0.0).astype(np.float32))
    wq, wk, wv = O.flash_backward(Q, K, V, wantA, dA, mask, lse_in, z(), z(), z())
    dK, dQ, dV = (torch.zeros_like(q) for _ in range(3))
    flash_sdpa_bwd_async(k, q, v, from_fortran(wantA), from_fortran(dA), m, from_fortran(lse_in),
                         dK, dQ, dV)
    torch.cuda.synchronize()
    for got, w in ((dQ, wq), (dK, wk), (dV, wv)):
        wf = O.from_bf16(w)
        gf = O.from_bf16(to_fortran(got))
        if np.abs(wf).max() == 0.0:
            assert np.abs(gf).max() == 0.0
        else:
            assert O.rel_err(gf, wf) <= TOL
