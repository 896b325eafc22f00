"""Full BASELINE sizes on the GPU, checked through size-independent properties
(the CPU oracle would need minutes at these sizes):

forward   V = 1 gives A = 1 on every row that sees a key; A is linear in V;
          lse does not depend on V.
backward  sum(dQ o Q) = sum(dK o K) per slice (both equal sum dS o S);
          with dA constant along the sequence, sum_k dV[k, :] = sum_q dA[q, :];
          gradients are added to what dK, dQ, dV held.
decode    config 5 shape: constant V rows come back unchanged; doubling V doubles out.
A medium case (seq 1024, several waves of CTAs) is compared with the oracle itself.
"""
import math

import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import decode_sdpa, from_fortran, to_fortran

pytestmark = pytest.mark.gpu


def causal_mask(S):
    q = torch.arange(S, device="cuda")[:, None]
    k = torch.arange(S, device="cuda")[None, :]
    return torch.where(k > q, -math.inf, 0.0).to(torch.bfloat16)


def run_fwd(q, k, v, mask):
    nb, S, D = q.shape
    lse = torch.full((nb, S), -math.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    s_l, s_A = torch.empty_like(lse), torch.empty_like(A)
    ops.flash_sdpa_fwd(S, D, nb, k, q, mask, s_l, v, s_A, lse, A)
    torch.cuda.synchronize()
    assert int(s_A.view(torch.int32).flatten()[0].item()) == 0      # status word
    return A, lse


def run_bwd(q, k, v, A, dA, mask, lse, init=0.0):
    nb, S, D = q.shape
    dK, dQ, dV = (torch.full_like(q, init) for _ in range(3))
    s1, s2, s3 = (torch.empty_like(q) for _ in range(3))
    ops.flash_sdpa_bwd(S, D, nb, k, q, v, A, dA, mask, lse, s1, s2, s3, dK, dQ, dV)
    torch.cuda.synchronize()
    assert int(s3.view(torch.int32).flatten()[0].item()) == 0       # status word
    return dQ, dK, dV


@pytest.mark.parametrize("S,D,nb", [(4096, 128, 32), (1024, 64, 96), (2048, 128, 16)])
def test_forward_backward_properties_at_baseline_sizes(S, D, nb):
    g = torch.Generator(device="cuda").manual_seed(S + D)
    q, k, v, dA = (torch.randn((nb, S, D), generator=g, device="cuda").to(torch.bfloat16)
                   for _ in range(4))
    mask = causal_mask(S)
    assert ops.flash_sdpa_path(S, D, nb) == 2 and ops.flash_sdpa_path(S, D, nb, True) == 2
    A, lse = run_fwd(q, k, v, mask)
    ones = torch.ones_like(v)
    A1, lse1 = run_fwd(q, k, ones, mask)
    assert torch.all(A1.float() == 1.0)
    assert torch.equal(lse1, lse)
    A2, _ = run_fwd(q, k, (2*v.float()).to(torch.bfloat16), mask)
    assert torch.allclose(A2.float(), 2*A.float(), rtol=2e-2, atol=1e-2)
    assert torch.isfinite(lse).all()
    # lse against a direct fp32 evaluation on three slices (first, a middle one, last)
    for s in (0, nb//2, nb - 1):
        sc = (q[s].float() @ k[s].float().T)/math.sqrt(D) + mask.float()
        ref = torch.logsumexp(sc, dim=1)
        assert torch.allclose(lse[s], ref, rtol=1e-3, atol=1e-3)
        refA = torch.softmax(sc, dim=1) @ v[s].float()
        err = (A[s].float() - refA).norm()/refA.norm()
        assert err <= 2e-2
    dQ, dK, dV = run_bwd(q, k, v, A, dA, mask, lse)
    lhs = (dQ.float()*q.float()).sum(dim=(1, 2))
    rhs = (dK.float()*k.float()).sum(dim=(1, 2))
    scale = (dQ.float().abs()*q.float().abs()).sum(dim=(1, 2))
    assert torch.all((lhs - rhs).abs() <= 2e-2*scale)
    # gradients on three slices against autograd in fp32
    for s in (0, nb - 1):
        qs, ks, vs = (x[s].float().clone().requires_grad_(True) for x in (q, k, v))
        sc = (qs @ ks.T)/math.sqrt(D) + mask.float()
        out = torch.softmax(sc, dim=1) @ vs
        out.backward(dA[s].float())
        for got, want in ((dQ[s], qs.grad), (dK[s], ks.grad), (dV[s], vs.grad)):
            assert (got.float() - want).norm()/want.norm() <= 2e-2
    # dA constant along the sequence: column sums of dV equal column sums of dA
    dA_c = dA[:, :1, :].expand(-1, S, -1).contiguous()
    _, _, dVc = run_bwd(q, k, v, A, dA_c, mask, lse)
    got = dVc.float().sum(dim=1)
    want = dA_c.float().sum(dim=1)
    assert torch.allclose(got, want, rtol=2e-2, atol=2e-2*float(want.abs().max()))
    # += contract at full size
    dQi, dKi, dVi = run_bwd(q, k, v, A, dA, mask, lse, init=0.5)
    for a, b in ((dQi, dQ), (dKi, dK), (dVi, dV)):
        assert torch.allclose(a.float(), b.float() + 0.5, rtol=2e-2, atol=2e-2)


def test_medium_case_against_oracle():
    """seq 1024, head 128, 6 slices: several CTAs per SM-wave of both kernels."""
    rng = np.random.default_rng(77)
    shape = (128, 1024, 3, 2, 1)
    Q, K, V, dA = (O.to_bf16(rng.standard_normal(shape).astype(np.float32)) for _ in range(4))
    k, q = np.meshgrid(np.arange(1024), np.arange(1024), indexing="ij")
    mask = O.to_bf16(np.asfortranarray(np.where(k > q, -np.inf, 0.0).astype(np.float32)))
    wantA, wantL = O.flash_forward(Q, K, V, mask)
    qd, kd, vd, md = (from_fortran(x) for x in (Q, K, V, mask))
    A, lse = run_fwd(qd.view(6, 1024, 128), kd.view(6, 1024, 128), vd.view(6, 1024, 128), md)
    got = O.from_bf16(to_fortran(A.view(1, 2, 3, 1024, 128)))
    assert O.rel_err(got, O.from_bf16(wantA)) <= 2e-2
    assert np.allclose(to_fortran(lse.view(1, 2, 3, 1024)), wantL, rtol=1e-3, atol=1e-3)
    z = lambda: O.zeros(shape, np.uint16)
    wq, wk, wv = O.flash_backward(Q, K, V, wantA, dA, mask, wantL, z(), z(), z())
    dQ, dK, dV = run_bwd(qd.view(6, 1024, 128), kd.view(6, 1024, 128), vd.view(6, 1024, 128),
                         from_fortran(wantA).view(6, 1024, 128),
                         from_fortran(dA).view(6, 1024, 128), md,
                         from_fortran(wantL).view(6, 1024))
    for got_t, want in ((dQ, wq), (dK, wk), (dV, wv)):
        got = O.from_bf16(to_fortran(got_t.view(1, 2, 3, 1024, 128)))
        assert O.rel_err(got, O.from_bf16(want)) <= 2e-2


def test_decode_properties_at_config5_size():
    D, L, B, G, H = 128, 8192, 64, 4, 8
    g = torch.Generator(device="cuda").manual_seed(4)
    q = torch.randn((H, G, B, 1, D), generator=g, device="cuda").to(torch.bfloat16)
    Kc = torch.randn((H, B, L, D), generator=g, device="cuda").to(torch.bfloat16)
    Vc = torch.randn((H, B, L, D), generator=g, device="cuda").to(torch.bfloat16)
    lse = torch.empty((H, G, B), dtype=torch.float32, device="cuda")
    o1 = decode_sdpa(q, Kc, Vc, lse_out=lse).float()
    o2 = decode_sdpa(q, Kc, (2*Vc.float()).to(torch.bfloat16)).float()
    assert torch.allclose(o2, 2*o1, rtol=2e-2, atol=2e-3)
    row = torch.randn(D, generator=g, device="cuda").to(torch.bfloat16)
    oc = decode_sdpa(q, Kc, row.expand(H, B, L, D).contiguous()).float()
    assert torch.allclose(oc, row.float().expand_as(oc), rtol=1e-2, atol=1e-2)
    # direct fp32 evaluation of a few (batch, kv head) units
    for h, b in ((0, 0), (3, 17), (7, 63)):
        sc = (q[h, :, b, 0].float() @ Kc[h, b].float().T)/math.sqrt(D)       # [G, L]
        ref = torch.softmax(sc, dim=1) @ Vc[h, b].float()
        got = o1[h, :, b, 0]
        assert (got - ref).norm()/ref.norm() <= 2e-2
        assert torch.allclose(lse[h, :, b], torch.logsumexp(sc, dim=1), rtol=1e-3, atol=1e-3)
