"""GPU parity of the unfused chain: every kernel against the reference's own CPU
kernels' outputs (tests/golden/ref_kernels.npz) and against the oracle on fresh
seeded inputs; then the whole forward/backward chain of nntile.layer.Sdpa
against the reference-kernel chain (ref_chain.npz) and the oracle.

Tolerances: fp32 <= 1e-5 relative (the path's stated bar); bf16 kernels are
compared with the oracle's bf16 restatement, one rounding step apart at most
(2^-7 relative per element)."""
import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import Sdpa, from_fortran, to_fortran

pytestmark = pytest.mark.gpu
F = np.asfortranarray
FP32_TOL = 1e-5


def dev(a):
    return from_fortran(a)


def close32(got_t, want, tol=FP32_TOL):
    got = to_fortran(got_t)
    want = np.asarray(want)
    assert got.shape == want.shape
    fin = np.isfinite(want)
    assert np.array_equal(np.isfinite(got), fin)
    assert np.array_equal(got[~fin], want[~fin])
    scale = max(1.0, float(np.abs(want[fin]).max()))
    assert np.abs(got[fin].astype(np.float64) - want[fin]).max() <= tol*scale


@pytest.mark.parametrize("tag,m,n,k", [("m1", 1, 24, 37), ("m3", 3, 5, 11)])
def test_kernels_match_reference_outputs(golden, tag, m, n, k):
    g = golden("ref_kernels.npz")
    dst = dev(O.zeros((2, m, n), np.float32))
    ops.maxsumexp(m, n, k, dev(g[f"maxsumexp_{tag}_src"]), dst)
    close32(dst, g[f"maxsumexp_{tag}_first"])
    ops.maxsumexp(m, n, k, dev(g[f"maxsumexp_{tag}_src2"]), dst)
    close32(dst, g[f"maxsumexp_{tag}_second"])
    sm = dev(g[f"maxsumexp_{tag}_src"])
    ops.softmax_inplace(m, n, k, dev(g[f"maxsumexp_{tag}_first"]), 0.75, sm)
    close32(sm, g[f"softmax_{tag}_out"])
    d = dev(g[f"sumprod_{tag}_dst0"])
    ops.sumprod_slice(m, n, k, 1.5, dev(g[f"sumprod_{tag}_a"]), dev(g[f"sumprod_{tag}_b"]), -0.5, d)
    close32(d, g[f"sumprod_{tag}_out"])
    d = dev(g[f"sumprod_{tag}_dst0"])
    ops.sumprod_slice(m, n, k, 1.0, dev(g[f"sumprod_{tag}_a"]), dev(g[f"sumprod_{tag}_b"]), 0.0, d)
    close32(d, g[f"sumprod_{tag}_out_beta0"])
    t = dev(g[f"addslice_{tag}_dst0"])
    ops.add_slice_inplace(m, n, k, -1.0, dev(g[f"addslice_{tag}_src"]), 1.0, t)
    close32(t, g[f"addslice_{tag}_out"], 1e-7)


def test_elementwise_kernels_match_reference_outputs(golden):
    g = golden("ref_kernels.npz")
    d = dev(g["mask_dst0"])
    ops.mask_scalar(35, 6, dev(g["mask_mask"]), -np.inf, d)
    assert np.array_equal(to_fortran(d), g["mask_out"])
    y = dev(g["mul_dst0"])
    ops.multiply_inplace(301, 0.5, dev(g["mul_src"]), y)
    close32(y, g["mul_out"], 1e-7)
    y = dev(g["mul_dst0"])
    ops.add_inplace(301, 2.0, dev(g["mul_src"]), -1.0, y)
    close32(y, g["add_out"], 1e-7)
    C = dev(g["gemm_C0"])
    ops.gemm(True, False, 7, 5, 16, 3, 0.125, dev(g["gemm_A"]), dev(g["gemm_B"]), 1.0, C)
    close32(C, g["gemm_out"])


@pytest.mark.parametrize("head", [1, 3, 4, 8, 15, 16, 32, 64])
def test_accumulate_attn_output(head):
    """Head sizes of tests/kernel/accumulate_attn_output.cc:176-179, tol 1e-5."""
    rng = np.random.default_rng(head)
    seq, batch = 19, 3
    sl = rng.standard_normal(seq*batch).astype(np.float32)
    dl = rng.standard_normal(seq*batch).astype(np.float32)
    sl[[2, 11]] = -np.inf
    dl[[5, 11]] = -np.inf
    sl[7] = np.nan
    sa = F(rng.standard_normal((head, seq*batch)).astype(np.float32))
    da = F(rng.standard_normal((head, seq*batch)).astype(np.float32))
    want_l, want_a = dl.copy(), da.copy(order="F")
    O.accumulate_attn_output(head, seq, batch, sl, sa, want_l, want_a, cuda_rules=True)
    gl, ga = dev(dl), dev(da)
    ops.accumulate_attn_output(head, seq, batch, dev(sl), dev(sa), gl, ga)
    close32(gl, want_l)
    close32(ga, want_a)
    # bf16 storage
    sab, dab = O.to_bf16(sa), O.to_bf16(da)
    want_l, want_a = dl.copy(), dab.copy(order="F")
    O.accumulate_attn_output(head, seq, batch, sl, sab, want_l, want_a, cuda_rules=True)
    gl, ga = dev(dl), dev(dab)
    ops.accumulate_attn_output(head, seq, batch, dev(sl), dev(sab), gl, ga)
    close32(gl, want_l)
    assert O.rel_err(O.from_bf16(to_fortran(ga)), O.from_bf16(want_a)) <= 2.0**-7


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("m,n,k", [(1, 300, 257), (1, 64, 2048), (4, 33, 65), (1, 1, 1), (2, 0, 5)])
def test_kernels_against_oracle_on_fresh_inputs(dtype, m, n, k):
    rng = np.random.default_rng(m*1000 + n + k)
    cast = (lambda a: F(a.astype(np.float32))) if dtype == "fp32" else O.to_bf16
    npdt = np.float32 if dtype == "fp32" else np.uint16
    tol = FP32_TOL if dtype == "fp32" else 2.0**-6

    def cmp(got_t, want):
        got = to_fortran(got_t) if got_t.numel() else np.zeros(want.shape, want.dtype)
        if want.size == 0:
            return
        assert O.rel_err(O.as_f32(got), O.as_f32(want)) <= tol

    src = rng.standard_normal((m, k, n)).astype(np.float32)*3
    if src.size:
        src[:, ::7, :] = -np.inf
    src = cast(src)
    want = O.zeros((2, m, n), npdt)
    O.maxsumexp(m, n, k, src, want)
    got = dev(O.zeros((2, m, n), npdt))
    ops.maxsumexp(m, n, k, dev(src), got)
    cmp(got, want)
    want_s = src.copy(order="F")
    O.softmax_inplace(m, n, k, want, 1.0, want_s)
    got_s = dev(src)
    ops.softmax_inplace(m, n, k, dev(want), 1.0, got_s)
    cmp(got_s, want_s)
    a, b = cast(rng.standard_normal((m, k, n))), cast(rng.standard_normal((m, k, n)))
    d0 = cast(rng.standard_normal((m, n)))
    want_d = d0.copy(order="F")
    O.sumprod_slice(m, n, k, 0.5, a, b, 2.0, want_d)
    got_d = dev(d0)
    ops.sumprod_slice(m, n, k, 0.5, dev(a), dev(b), 2.0, got_d)
    cmp(got_d, want_d)
    t0 = cast(rng.standard_normal((m, k, n)))
    want_t = t0.copy(order="F")
    O.add_slice_inplace(m, n, k, -1.0, d0, 1.0, want_t)
    got_t = dev(t0)
    ops.add_slice_inplace(m, n, k, -1.0, dev(d0), 1.0, got_t)
    cmp(got_t, want_t)
    want_m = t0.copy(order="F")
    O.multiply_inplace(t0.size, 0.7, a, want_m)
    got_m = dev(t0)
    ops.multiply_inplace(t0.size, 0.7, dev(a), got_m)
    cmp(got_m, want_m)


def test_chain_matches_reference_kernels_chain(golden):
    """The forward+backward chain stored in ref_chain.npz was run by the
    reference's own CPU kernels; fp32, <= 1e-5 relative."""
    g = golden("ref_chain.npz")
    Q, K, V, dY = (g[k] for k in ("chain_Q", "chain_K", "chain_V", "chain_dY"))
    S = Q.shape[1]
    mask = F(np.triu(np.ones((S, S), dtype=bool)))
    layer = Sdpa(dev(Q), dev(K), dev(V), mask=dev(mask))
    y = layer.forward_async()
    assert O.rel_err(to_fortran(y), g["chain_Y"]) <= FP32_TOL
    dq, dk, dv = (torch.zeros_like(layer.q) for _ in range(3))
    layer.backward_async(dev(dY), dq, dk, dv)
    for got, key in ((dq, "chain_dQ"), (dk, "chain_dK"), (dv, "chain_dV")):
        assert O.rel_err(to_fortran(got), g[key]) <= FP32_TOL


def test_baseline_config1_forward_fp32():
    """BASELINE config 1: batch 4, heads 4, head_dim 64, seq 256, one tile,
    Q,K,V ~ N(0,1) seed 0, causal -inf mask; <= 1e-5 relative vs the oracle chain
    (the reference's kernels when oracle/_ref is present)."""
    rng = np.random.default_rng(0)
    shape = (64, 256, 4, 1, 4)
    Q, K, V = (F(rng.standard_normal(shape).astype(np.float32)) for _ in range(3))
    mask = F(np.triu(np.ones((256, 256), dtype=bool)))
    want, _, want_mse = O.vanilla_forward(Q, K, V, mask,
                                          backend="ref" if O.have_ref() else "port")
    layer = Sdpa(dev(Q), dev(K), dev(V), mask=dev(mask))
    y = layer.forward_async()
    assert O.rel_err(to_fortran(y), want) <= FP32_TOL
    assert O.rel_err(to_fortran(layer.attn_maxsumexp), want_mse) <= FP32_TOL


def test_chain_bf16_against_oracle():
    rng = np.random.default_rng(11)
    shape = (32, 96, 2, 2, 2)
    Q, K, V, dY = (O.to_bf16(rng.standard_normal(shape).astype(np.float32)) for _ in range(4))
    mask = F(np.triu(np.ones((96, 96), dtype=bool)))
    want, attn, _ = O.vanilla_forward(Q, K, V, mask)
    layer = Sdpa(dev(Q), dev(K), dev(V), mask=dev(mask))
    y = layer.forward_async()
    assert O.rel_err(O.from_bf16(to_fortran(y)), O.from_bf16(want)) <= 2e-2
    wq, wk, wv = (O.zeros(shape, np.uint16) for _ in range(3))
    O.vanilla_backward(Q, K, V, want, dY, attn, mask, wq, wk, wv)
    dq, dk, dv = (torch.zeros_like(layer.q) for _ in range(3))
    layer.backward_async(dev(dY), dq, dk, dv)
    for got, w in ((dq, wq), (dk, wk), (dv, wv)):
        assert O.rel_err(O.from_bf16(to_fortran(got)), O.from_bf16(w)) <= 2e-2
