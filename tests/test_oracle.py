"""The CPU oracle against the reference: (1) its C restatement reproduces the
outputs of the reference's own CPU kernels stored under tests/golden/
(ref_kernels.npz, ref_chain.npz were produced by oracle/_ref, i.e. the
reference sources compiled in place); (2) when oracle/_ref is present it is
compared live as well; (3) the fused-path restatement meets the reference
tests' fp64 formulas within the reference tests' own tolerances."""
import numpy as np
import pytest

import oracle as O

F = np.asfortranarray
TIGHT = 2e-6   # fp32, same formulas; differences come from libm/sum order only


def close(a, b, tol=TIGHT):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert a.shape == b.shape
    fin = np.isfinite(b)
    assert np.array_equal(np.isfinite(a), fin)
    assert np.array_equal(a[~fin], b[~fin]) or np.all(np.isnan(b[~fin]) == np.isnan(a[~fin]))
    scale = max(1.0, float(np.abs(b[fin]).max()) if fin.any() else 1.0)
    assert np.abs(a[fin] - b[fin]).max() <= tol * scale


@pytest.mark.parametrize("tag,m,n,k", [("m1", 1, 24, 37), ("m3", 3, 5, 11)])
def test_port_matches_reference_kernels(golden, tag, m, n, k):
    g = golden("ref_kernels.npz")
    dst = O.zeros((2, m, n), np.float32)
    O.maxsumexp(m, n, k, F(g[f"maxsumexp_{tag}_src"]), dst)
    close(dst, g[f"maxsumexp_{tag}_first"])
    O.maxsumexp(m, n, k, F(g[f"maxsumexp_{tag}_src2"]), dst)
    close(dst, g[f"maxsumexp_{tag}_second"])
    sm = F(g[f"maxsumexp_{tag}_src"].copy())
    O.softmax_inplace(m, n, k, F(g[f"maxsumexp_{tag}_first"]), 0.75, sm)
    # a fully masked fibre has (max,sum)=(0,0): the reference yields 0 there
    close(sm, g[f"softmax_{tag}_out"])
    d = F(g[f"sumprod_{tag}_dst0"].copy())
    O.sumprod_slice(m, n, k, 1.5, F(g[f"sumprod_{tag}_a"]), F(g[f"sumprod_{tag}_b"]), -0.5, d)
    close(d, g[f"sumprod_{tag}_out"])
    d = F(g[f"sumprod_{tag}_dst0"].copy())
    O.sumprod_slice(m, n, k, 1.0, F(g[f"sumprod_{tag}_a"]), F(g[f"sumprod_{tag}_b"]), 0.0, d)
    close(d, g[f"sumprod_{tag}_out_beta0"])
    t = F(g[f"addslice_{tag}_dst0"].copy())
    O.add_slice_inplace(m, n, k, -1.0, F(g[f"addslice_{tag}_src"]), 1.0, t)
    close(t, g[f"addslice_{tag}_out"], 0)


def test_port_matches_reference_elementwise(golden):
    g = golden("ref_kernels.npz")
    d = F(g["mask_dst0"].copy())
    O.mask_scalar(35, 6, g["mask_mask"], -np.inf, d)
    assert np.array_equal(d, g["mask_out"])
    y = g["mul_dst0"].copy()
    O.multiply_inplace(301, 0.5, g["mul_src"], y)
    assert np.array_equal(y, g["mul_out"])
    y = g["mul_dst0"].copy()
    O.add_inplace(301, 2.0, g["mul_src"], -1.0, y)
    close(y, g["add_out"], 1e-7)
    da, dl = F(g["acc_dst_attn0"].copy()), g["acc_dst_lse0"].copy()
    O.accumulate_attn_output(15, 9, 2, g["acc_src_lse"], F(g["acc_src_attn"]), dl, da,
                             cuda_rules=False)
    close(dl, g["acc_dst_lse"])
    close(da, g["acc_dst_attn"])
    C = F(g["gemm_C0"].copy())
    O.gemm(1, 0, 7, 5, 16, 3, 0.125, F(g["gemm_A"]), F(g["gemm_B"]), 1.0, C)
    close(C, g["gemm_out"])


def test_port_matches_reference_chain(golden):
    g = golden("ref_chain.npz")
    Q, K, V, dY = (F(g[k]) for k in ("chain_Q", "chain_K", "chain_V", "chain_dY"))
    S = Q.shape[1]
    mask = F(np.triu(np.ones((S, S), dtype=bool)))
    Y, attn, mse = O.vanilla_forward(Q, K, V, mask)
    assert O.rel_err(Y, g["chain_Y"]) <= 1e-6
    close(mse, g["chain_mse"], 1e-5)
    dQ, dK, dV = (O.zeros(Q.shape, np.float32) for _ in range(3))
    O.vanilla_backward(Q, K, V, Y, dY, attn, mask, dQ, dK, dV)
    for got, key in ((dQ, "chain_dQ"), (dK, "chain_dK"), (dV, "chain_dV")):
        assert O.rel_err(got, g[key]) <= 1e-6
    # the same answer whatever the tiling (tests/tensor/*: single vs multi tile)
    Yt, _, _ = O.vanilla_forward(Q, K, V, mask, q_tile=16, k_tile=16, batch_tile=(1, 1, 1))
    assert O.rel_err(Yt, g["chain_Y"]) <= 1e-6
    # and the reference tests' fp64 formula
    a64, _ = O.sdpa_fp64(Q, K, V, np.where(mask, 0, -np.inf).astype(np.float32))
    assert O.rel_err(Y, a64) <= 1e-5


@pytest.mark.skipif(not O.have_ref(), reason="oracle/_ref not built")
def test_port_matches_live_reference():
    rng = np.random.default_rng(7)
    D, S, B, G, H = 32, 96, 2, 2, 2
    Q, K, V = (F(rng.standard_normal((D, S, B, G, H)).astype(np.float32)) for _ in range(3))
    mask = F(np.triu(np.ones((S, S), dtype=bool)))
    Yp, ap, mp = O.vanilla_forward(Q, K, V, mask, backend="port")
    Yr, ar, mr = O.vanilla_forward(Q, K, V, mask, q_tile=32, k_tile=32, backend="ref")
    assert O.rel_err(Yp, Yr) <= 1e-6
    assert O.ref.ref_bf16_rounds_to_nearest() == 1
    # bf16 kernels of the reference build against the port's bf16 restatement
    x = O.to_bf16(rng.standard_normal((1, 40, 12)).astype(np.float32))
    d1, d2 = O.zeros((2, 1, 12), np.uint16), O.zeros((2, 1, 12), np.uint16)
    O.maxsumexp(1, 12, 40, x, d1, backend="port")
    O.maxsumexp(1, 12, 40, x, d2, backend="ref")
    assert np.array_equal(d1, d2)
    s1, s2 = x.copy(order="F"), x.copy(order="F")
    O.softmax_inplace(1, 12, 40, d1, 1.0, s1, backend="port")
    O.softmax_inplace(1, 12, 40, d2, 1.0, s2, backend="ref")
    assert np.array_equal(s1, s2)


def test_bf16_conversion_rounds_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, np.inf, -np.inf, 0.0], np.float32)
    b = O.to_bf16(x)
    # 1 + 2^-8 is a tie -> even (1.0); 1 + 3*2^-8 is a tie -> even (1.015625)
    assert O.from_bf16(b).tolist() == [1.0, 1.0, 1.015625, -2.5, np.inf, -np.inf, 0.0]
    import torch
    y = np.random.default_rng(3).standard_normal(4096).astype(np.float32)
    t = torch.from_numpy(y).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(O.to_bf16(y), t)


FWD_CASES = [(16, 32, 1, True), (32, 64, 2, True), (32, 32, 2, False), (16, 64, 1, False)]
BWD_CASES = [(64, 8, 1, True), (64, 32, 4, True), (64, 32, 1, False), (64, 8, 4, False)]


def _golden_mod():
    import importlib.util, os
    p = os.path.join(os.path.dirname(__file__), "golden", "make_golden.py")
    spec = importlib.util.spec_from_file_location("make_golden", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("seq,head,batch,causal", FWD_CASES)
def test_flash_fwd_restatement_meets_reference_test_formula(golden, seq, head, batch, causal):
    """Shapes, PRESET inputs and eps=1e-2 of tests/kernel/flash_sdpa_fwd_cudnn.cc."""
    mg = _golden_mod()
    g = golden("flash_preset.npz")
    Q, K, V, mask = mg.preset_fwd(seq, head, batch, causal)
    Qb, Kb, Vb = (O.to_bf16(mg._as5(x, head, seq, batch)) for x in (Q, K, V))
    mkq = O.to_bf16(F(mask.T))
    A, lse = O.flash_forward(Qb, Kb, Vb, mkq)
    tag = f"fwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
    assert O.rel_err(O.from_bf16(A), g[tag + "_A"]) <= 1e-2
    assert np.allclose(lse, g[tag + "_lse"], rtol=1e-2, atol=1e-6)


@pytest.mark.parametrize("seq,head,batch,causal", BWD_CASES)
def test_flash_bwd_restatement_meets_reference_test_formula(golden, seq, head, batch, causal):
    """Shapes, PRESET inputs (arbitrary A and lse) and eps=1e-2 of
    tests/kernel/flash_sdpa_bwd_cudnn.cc; gradients accumulate into non-zero
    buffers as tests/tile/flash_sdpa_bwd_cudnn.cc:298-325 requires."""
    mg = _golden_mod()
    g = golden("flash_preset.npz")
    Q, K, V, A, dA, lse, mask = mg.preset_bwd(seq, head, batch, causal)
    Qb, Kb, Vb, Ab, dAb = (O.to_bf16(mg._as5(x, head, seq, batch)) for x in (Q, K, V, A, dA))
    mkq = O.to_bf16(F(mask.T))
    l4 = F(lse.reshape(batch, seq).T.reshape(seq, batch, 1, 1))
    tag = f"bwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
    zero = O.zeros(Qb.shape, np.uint16)
    z = O.flash_backward(Qb, Kb, Vb, Ab, dAb, mkq, l4, zero.copy(order="F"), zero.copy(order="F"), zero)
    for got, key in zip(z, ("_dQ", "_dK", "_dV")):
        assert O.rel_err(O.from_bf16(got), g[tag + key]) <= 1e-2
    init = np.full(Qb.shape, 0.25, np.float32)
    dQ, dK, dV = (O.to_bf16(init) for _ in range(3))
    dQ, dK, dV = O.flash_backward(Qb, Kb, Vb, Ab, dAb, mkq, l4, dQ, dK, dV)
    for got, key in ((dQ, "_dQ"), (dK, "_dK"), (dV, "_dV")):
        assert O.rel_err(O.from_bf16(got), init + g[tag + key]) <= 1e-2


def test_flash_tiling_is_equivalent_to_one_tile():
    """tests/tensor/flash_sdpa_fwd_cudnn.cc:167-246: K/V tiles streamed through
    many tasks give the single-tile answer; banded mask |i-j|<=32 as in
    wrappers/python/tests/nntile_core/test_tensor_flash_sdpa_fwd_cudnn.py:96-104."""
    rng = np.random.default_rng(42)
    shape = (32, 128, 2, 1, 2)
    Q, K, V = (O.to_bf16(rng.standard_normal(shape).astype(np.float32) * 0.1) for _ in range(3))
    i = np.arange(128)
    band = np.where(np.abs(i[:, None] - i[None, :]) <= 32, 0.0, -np.inf).astype(np.float32)
    mk = O.to_bf16(F(band))
    A1, l1 = O.flash_forward(Q, K, V, mk)
    A2, l2 = O.flash_forward(Q, K, V, mk, seq_tile=32, batch_tile=(1, 1, 1))
    a64, l64 = O.sdpa_fp64(Q, K, V, mk)
    assert O.rel_err(O.from_bf16(A1), a64) <= 1e-2
    assert O.rel_err(O.from_bf16(A2), a64) <= 1e-2
    assert np.allclose(l1, l64, rtol=1e-4, atol=1e-5) and np.allclose(l2, l64, rtol=1e-4, atol=1e-5)


def test_decode_chain_against_fp64():
    rng = np.random.default_rng(4)
    D, L, B, G, H = 32, 200, 3, 4, 2
    q = O.to_bf16(rng.standard_normal((D, 1, B, G, H)).astype(np.float32))
    Kc, Vc = (O.to_bf16(rng.standard_normal((D, L, B, H)).astype(np.float32)) for _ in range(2))
    Y = O.decode_chain(q, Kc, Vc, length=150)
    Kr = np.repeat(O.from_bf16(Kc)[:, :150, :, None, :], G, axis=3)
    Vr = np.repeat(O.from_bf16(Vc)[:, :150, :, None, :], G, axis=3)
    a64, _ = O.sdpa_fp64(O.from_bf16(q), Kr, Vr, np.zeros((150, 1), np.float32))
    assert O.rel_err(O.from_bf16(Y), a64) <= 2e-2


def test_kv_cache_append_restatement():
    """KVCache.append semantics (cache_utils.py:146-176): copy at the current
    length, lengths add up, appending past max_cache_size is an error."""
    import oracle as O
    rng = np.random.default_rng(3)
    cache = np.zeros((8, 10, 2, 3), dtype=np.float32, order="F")
    n = 0
    parts = []
    for m in (4, 1, 5):
        p = np.asfortranarray(rng.standard_normal((8, m, 2, 3)).astype(np.float32))
        n = O.kv_cache_append(cache, n, p)
        parts.append(p)
    assert n == 10
    assert np.array_equal(cache, np.concatenate(parts, axis=1))
    with pytest.raises(ValueError):
        O.kv_cache_append(cache, n, parts[1])


@pytest.mark.parametrize("tag", ["llama_q", "llama_k", "gpt2"])
def test_prologue_restatement_matches_reference_kernels(golden, tag):
    """transpose + rope, transpose + bias and the transposition back, restated in C,
    against the outputs of the reference's own transpose / rope / add_fiber_inplace
    CPU kernels (tests/golden/ref_around.npz): bit for bit."""
    g = golden("ref_around.npz")
    proj, sin, cos, bias = (g[f"{tag}_{k}"] for k in ("proj", "sin", "cos", "bias"))
    assert np.array_equal(O.attention_prologue(proj, sin, cos), g[f"{tag}_rope"])
    assert np.array_equal(O.attention_prologue(proj), g[f"{tag}_plain"])
    assert np.array_equal(O.attention_prologue(proj, bias=bias), g[f"{tag}_biased"])
    assert np.array_equal(O.attention_epilogue(g[f"{tag}_rope"]), g[f"{tag}_back"])
    if O.have_ref():
        assert np.array_equal(O.attention_prologue(proj, sin, cos, backend="ref"),
                              g[f"{tag}_rope"])
