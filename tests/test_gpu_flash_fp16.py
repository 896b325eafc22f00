"""GPU parity of the IEEE-half (fp16) forms of the fused pair, which the reference
instantiates next to bf16 (src/starpu/flash_sdpa_fwd_cudnn.cc:292-293): the same
kernels compiled for the other 16-bit format, against the oracle's fp16 storage
instantiation (fp32 accumulation, values rounded to half where the reference stores
them), the reference kernel tests' PRESET inputs and fp64 formulas (eps 1e-2,
tests/kernel/flash_sdpa_{fwd,bwd}_cudnn.cc), the tile loops, and the grouped-query
form.  Tolerance: 2e-2 relative, the path's bar for 16-bit storage (fp16 carries three
more mantissa bits than bf16, the errors seen are a few 1e-4)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import Sdpa, flash_sdpa_bwd_async, flash_sdpa_fwd_async, from_fortran, to_fortran

pytestmark = pytest.mark.gpu
F = np.asfortranarray
TOL = 2e-2
H16 = np.float16


def _mg():
    p = os.path.join(os.path.dirname(__file__), "golden", "make_golden.py")
    spec = importlib.util.spec_from_file_location("make_golden", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def half(x):
    return F(np.asarray(x, dtype=np.float32).astype(H16))


def f32(t):
    return to_fortran(t).astype(np.float32)


def mask_of(kind, S):
    k, q = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    if kind == "none":
        return half(np.zeros((S, S)))
    m = np.where(k > q, -np.inf, 0.0).astype(np.float32)
    if kind == "biased":
        rng = np.random.default_rng(5)
        m = np.where(np.isfinite(m), rng.standard_normal((S, S)).astype(np.float32)*0.5, m)
        m[:, 3] = -np.inf               # query 3 sees nothing at all
    return half(m)


@pytest.mark.parametrize("head,seq,batch,group,kvh,kind", [
    (128, 256, 2, 2, 1, "causal"),     # tcgen05 kernels, head 128
    (64, 384, 1, 1, 3, "causal"),      # tcgen05 kernels, head 64, odd block count
    (128, 128, 3, 1, 1, "none"),
    (128, 256, 1, 1, 2, "biased"),     # finite biases and a fully masked query row
    (32, 80, 2, 1, 1, "causal"),       # generic kernels
    (16, 16, 1, 1, 1, "none"),         # the reference's smallest test shape
])
def test_fwd_bwd_against_oracle(head, seq, batch, group, kvh, kind):
    rng = np.random.default_rng(head + seq)
    shape = (head, seq, batch, group, kvh)
    Q, K, V, dA = (half(rng.standard_normal(shape)) for _ in range(4))
    mask = mask_of(kind, seq)
    wantA, wantL = O.flash_forward(Q, K, V, mask)
    q, k, v, m = (from_fortran(x) for x in (Q, K, V, mask))
    assert q.dtype == torch.float16
    lse = torch.full((kvh, group, batch, seq), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    flash_sdpa_fwd_async(k, q, m, lse, v, A)
    torch.cuda.synchronize()
    assert O.rel_err(f32(A), O.as_f32(wantA)) <= TOL
    gl, fin = to_fortran(lse), np.isfinite(wantL)
    assert np.array_equal(np.isfinite(gl), fin)
    assert np.allclose(gl[fin], wantL[fin], rtol=1e-3, atol=1e-3)
    assert np.array_equal(to_fortran(q), Q) and np.array_equal(to_fortran(k), K)   # inputs untouched
    lse_in = F(np.where(fin, wantL, 0.0).astype(np.float32))
    z = lambda: O.zeros(shape, H16)
    wq, wk, wv = O.flash_backward(Q, K, V, wantA, dA, mask, lse_in, z(), z(), z())
    dK, dQ, dV = (torch.zeros_like(q) for _ in range(3))
    flash_sdpa_bwd_async(k, q, v, from_fortran(wantA), from_fortran(dA), m, from_fortran(lse_in),
                         dK, dQ, dV)
    torch.cuda.synchronize()
    for got, want in ((dQ, wq), (dK, wk), (dV, wv)):
        assert O.rel_err(f32(got), O.as_f32(want)) <= TOL


@pytest.mark.parametrize("seq,head,batch,causal", [(32, 64, 2, True), (16, 64, 1, False)])
def test_reference_kernel_test_formula_forward(seq, head, batch, causal):
    """PRESET inputs of tests/kernel/flash_sdpa_fwd_cudnn.cc:211-263 in fp16 against its
    fp64 formula, eps 1e-2 as there."""
    mg = _mg()
    Q, K, V, mask = mg.preset_fwd(seq, head, batch, causal)
    Qh, Kh, Vh = (half(mg._as5(x, head, seq, batch)) for x in (Q, K, V))
    mkq = half(np.asfortranarray(mask.T))
    a64, l64 = O.sdpa_fp64(O.as_f32(Qh), O.as_f32(Kh), O.as_f32(Vh), O.as_f32(mkq))
    q, k, v, m = (from_fortran(x) for x in (Qh, Kh, Vh, mkq))
    lse = torch.full((1, 1, batch, seq), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    flash_sdpa_fwd_async(k, q, m, lse, v, A)
    torch.cuda.synchronize()
    assert O.rel_err(f32(A), a64) <= 1e-2
    assert np.allclose(to_fortran(lse), l64, rtol=1e-3, atol=1e-3)


def test_tile_loops_and_merge_in_fp16():
    """Two K/V sequence tiles per Q tile: the second task merges into (lse, A), the
    gradients of both tasks add up; against the oracle's tile loops."""
    rng = np.random.default_rng(21)
    shape = (128, 256, 2, 1, 2)
    Q, K, V, dA = (half(rng.standard_normal(shape)*0.5) for _ in range(4))
    mask = mask_of("causal", 256)
    wantA, wantL = O.flash_forward(Q, K, V, mask, seq_tile=128, batch_tile=(1, 1, 2))
    q, k, v, m = (from_fortran(x) for x in (Q, K, V, mask))
    layer = Sdpa(q, k, v, mask=m, flash_attention=True, seq_tile=128, batch_tile=(1, 1, 2))
    y = layer.forward_async()
    torch.cuda.synchronize()
    assert O.rel_err(f32(y), O.as_f32(wantA)) <= TOL
    assert np.allclose(to_fortran(layer.flash_logsumexp), wantL, rtol=1e-3, atol=1e-3)
    z = lambda: O.zeros(shape, H16)
    wq, wk, wv = O.flash_backward(Q, K, V, wantA, dA, mask, wantL, z(), z(), z(),
                                  seq_tile=128, batch_tile=(1, 1, 2))
    dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
    layer.y.copy_(from_fortran(wantA))
    layer.flash_logsumexp.copy_(from_fortran(wantL))
    layer.backward_async(from_fortran(dA), dq, dk, dv)
    torch.cuda.synchronize()
    for got, want in ((dq, wq), (dk, wk), (dv, wv)):
        assert O.rel_err(f32(got), O.as_f32(want)) <= 3e-2     # dQ rounded once here, per task there


def test_grouped_query_fp16():
    rng = np.random.default_rng(31)
    D, S, B, G, H = 128, 256, 2, 4, 2
    Q, dA = (half(rng.standard_normal((D, S, B, G, H))) for _ in range(2))
    Kkv, Vkv = (half(rng.standard_normal((D, S, B, H))) for _ in range(2))
    Krep = F(np.repeat(Kkv[:, :, :, None, :], G, axis=3))
    Vrep = F(np.repeat(Vkv[:, :, :, None, :], G, axis=3))
    mask = mask_of("causal", S)
    wantA, wantL = O.flash_forward(Q, Krep, Vrep, mask)
    q, k, v, m = (from_fortran(x) for x in (Q, Kkv, Vkv, mask))
    lse = torch.full((H, G, B, S), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    scratch = torch.empty(ops.flash_sdpa_gqa_scratch_bytes(S, D, B, G, H), dtype=torch.uint8,
                          device="cuda")
    ops.flash_sdpa_fwd_gqa(S, D, B, G, H, k, q, m, v, lse, A, scratch)
    torch.cuda.synchronize()
    assert O.rel_err(f32(A), O.as_f32(wantA)) <= TOL
    z = lambda: O.zeros(Q.shape, H16)
    wq, wk, wv = O.flash_backward(Q, Krep, Vrep, wantA, dA, mask, wantL, z(), z(), z())
    dQ = torch.zeros_like(q)
    dK, dV = torch.zeros_like(k), torch.zeros_like(k)
    ops.flash_sdpa_bwd_gqa(S, D, B, G, H, k, q, v, from_fortran(wantA), from_fortran(dA), m,
                           from_fortran(wantL), dK, dQ, dV, scratch)
    torch.cuda.synchronize()
    assert ops.flash_sdpa_read_status(scratch) == 0
    assert O.rel_err(f32(dQ), O.as_f32(wq)) <= TOL
    assert O.rel_err(f32(dK), O.as_f32(wk).sum(axis=3)) <= TOL
    assert O.rel_err(f32(dV), O.as_f32(wv).sum(axis=3)) <= TOL


def test_bf16_buffers_are_not_taken_for_fp16():
    """The two builds are separate entry points: dtype picks one, fp32 is refused."""
    t = torch.zeros((1, 128, 128), dtype=torch.float32, device="cuda")
    with pytest.raises(TypeError):
        ops.flash_sdpa_fwd(128, 128, 1, t, t, t, t, t, t, t, t)
