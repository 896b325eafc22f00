"""GPU parity of the fused flash-SDPA tile tasks, called through the C ABI.

Pins: (1) the reference kernel tests' own shapes, PRESET inputs, fp64 formulas
and eps 1e-2 (tests/golden/flash_preset.npz, from
tests/kernel/flash_sdpa_{fwd,bwd}_cudnn.cc); (2) the oracle's restatement of the
reference's tiled path on seeded inputs, <= 2e-2 relative (bf16 storage, fp32
accumulation - the path's stated bar); (3) the tensor-test property "K/V tiles
streamed through many tasks == one big tile"; (4) inputs bit-unchanged;
(5) accumulate-into-output contracts (lse merge, += of gradients)."""
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
BF16_TOL = 2e-2


def _mg():
    p = os.path.join(os.path.dirname(__file__), "golden", "make_golden.py")
    spec = importlib.util.spec_from_file_location("make_golden", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def dev(a):
    return from_fortran(a)


def bf(t):
    return O.from_bf16(to_fortran(t))


def causal_add(S, dtype=np.float32):
    """Fortran [k, q] additive causal mask: -inf where k > q."""
    k, q = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    return F(np.where(k > q, -np.inf, 0.0).astype(dtype))


def run_fwd(Q, K, V, mask, seq_tile=None, batch_tile=None):
    q, k, v, m = dev(Q), dev(K), dev(V), dev(mask)
    H, G, B, S, D = q.shape
    lse = torch.full((H, G, B, S), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    flash_sdpa_fwd_async(k, q, m, lse, v, A, seq_tile, batch_tile)
    torch.cuda.synchronize()
    return A, lse, (q, k, v, m)


FWD_CASES = [(16, 32, 1, True), (32, 64, 2, True), (32, 32, 2, False), (16, 64, 1, False)]
BWD_CASES = [(64, 8, 1, True), (64, 32, 4, True), (64, 32, 1, False), (64, 8, 4, False)]


@pytest.mark.parametrize("seq,head,batch,causal", FWD_CASES)
def test_fwd_reference_kernel_test_cases(golden, seq, head, batch, causal):
    mg, g = _mg(), golden("flash_preset.npz")
    Q, K, V, mask = mg.preset_fwd(seq, head, batch, causal)
    Qb, Kb, Vb = (O.to_bf16(mg._as5(x, head, seq, batch)) for x in (Q, K, V))
    mkq = O.to_bf16(F(mask.T))
    A, lse, ins = run_fwd(Qb, Kb, Vb, mkq)
    tag = f"fwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
    assert O.rel_err(bf(A), g[tag + "_A"]) <= 1e-2
    assert np.allclose(to_fortran(lse), g[tag + "_lse"], rtol=1e-2, atol=1e-6)
    # inputs must come back bit-identical (tests/kernel/flash_sdpa_fwd_cudnn.cc:345-362)
    for t, src in zip(ins, (Qb, Kb, Vb, mkq)):
        assert np.array_equal(to_fortran(t), src)


@pytest.mark.parametrize("seq,head,batch,causal", BWD_CASES)
def test_bwd_reference_kernel_test_cases(golden, seq, head, batch, causal):
    mg, g = _mg(), golden("flash_preset.npz")
    Q, K, V, A, dA, lse, mask = mg.preset_bwd(seq, head, batch, causal)
    Qb, Kb, Vb, Ab, dAb = (O.to_bf16(mg._as5(x, head, seq, batch)) for x in (Q, K, V, A, dA))
    mkq = O.to_bf16(F(mask.T))
    l4 = F(lse.reshape(batch, seq).T.reshape(seq, batch, 1, 1))
    tag = f"bwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
    args = [dev(x) for x in (Kb, Qb, Vb, Ab, dAb, mkq, l4)]
    for init in (0.0, 0.25):      # += contract, tests/tile/flash_sdpa_bwd_cudnn.cc:298-325
        dK, dQ, dV = (torch.full_like(args[0], init) for _ in range(3))
        flash_sdpa_bwd_async(*args, dK, dQ, dV)
        torch.cuda.synchronize()
        for got, key in ((dQ, "_dQ"), (dK, "_dK"), (dV, "_dV")):
            assert O.rel_err(bf(got), init + g[tag + key]) <= 1e-2


SEEDED = [
    # (head, seq, batch, group, kv_heads, mask kind)
    (64, 128, 2, 1, 2, "causal"),
    (128, 128, 1, 2, 1, "causal"),
    (64, 256, 1, 1, 3, "band"),
    (128, 384, 1, 1, 2, "causal"),
    (64, 128, 1, 1, 1, "none"),
    (32, 80, 2, 1, 1, "causal"),      # ragged for the fast path: generic kernels
    (128, 256, 2, 1, 1, "ragged"),    # finite biases and a fully masked query row
]


def make_mask(kind, S):
    if kind == "causal":
        return causal_add(S)
    if kind == "none":
        return F(np.zeros((S, S), np.float32))
    i = np.arange(S)
    if kind == "band":
        return F(np.where(np.abs(i[:, None] - i[None, :]) <= 32, 0.0, -np.inf).astype(np.float32))
    m = causal_add(S)
    rng = np.random.default_rng(5)
    m = np.where(np.isfinite(m), rng.standard_normal((S, S)).astype(np.float32)*0.5, m)
    m[:, 3] = -np.inf               # query 3 sees nothing at all
    return F(m.astype(np.float32))


@pytest.mark.parametrize("head,seq,batch,group,kvh,kind", SEEDED)
def test_fwd_bwd_against_oracle(head, seq, batch, group, kvh, kind):
    rng = np.random.default_rng(head + seq)
    shape = (head, seq, batch, group, kvh)
    Q, K, V, dA = (O.to_bf16(rng.standard_normal(shape).astype(np.float32)) for _ in range(4))
    mask = O.to_bf16(make_mask(kind, seq))
    wantA, wantL = O.flash_forward(Q, K, V, mask)
    A, lse, _ = run_fwd(Q, K, V, mask)
    assert O.rel_err(bf(A), O.from_bf16(wantA)) <= BF16_TOL
    gl = to_fortran(lse)
    fin = np.isfinite(wantL)
    assert np.array_equal(np.isfinite(gl), fin)
    assert np.allclose(gl[fin], wantL[fin], rtol=1e-3, atol=1e-3)
    if kind == "ragged":               # the fully masked row is left untouched
        assert np.all(bf(A)[:, 3] == 0.0) and np.all(np.isneginf(gl[3]))
    # backward from the oracle's A and lse
    z = lambda: O.zeros(shape, np.uint16)
    wq, wk, wv = O.flash_backward(Q, K, V, wantA, dA, mask, wantL, z(), z(), z())
    lse_in = np.where(fin, wantL, 0.0).astype(np.float32)
    dK, dQ, dV = (torch.zeros(tuple(reversed(shape)), dtype=torch.bfloat16, device="cuda")
                  for _ in range(3))
    flash_sdpa_bwd_async(dev(K), dev(Q), dev(V), dev(wantA), dev(dA), dev(mask),
                         dev(F(lse_in)), dK, dQ, dV)
    torch.cuda.synchronize()
    wq2, wk2, wv2 = O.flash_backward(Q, K, V, wantA, dA, mask, F(lse_in), z(), z(), z())
    for got, w in ((dQ, wq2), (dK, wk2), (dV, wv2)):
        assert O.rel_err(bf(got), O.from_bf16(w)) <= BF16_TOL


@pytest.mark.parametrize("shape,base", [
    # tilings of tests/tensor/flash_sdpa_fwd_cudnn.cc:244-246 (head, seq, batch, group, kv)
    ((32, 64, 1, 1, 1), (32, 64, 1, 1, 1)),
    ((128, 256, 2, 2, 2), (128, 128, 1, 1, 1)),
    ((32, 512, 4, 3, 4), (32, 64, 1, 1, 2)),
    ((64, 256, 3, 4, 2), (64, 64, 3, 2, 1)),   # wrappers/python/tests/layer/test_sdpa.py:86-109
])
def test_tiled_equals_single_tile(shape, base):
    rng = np.random.default_rng(42)
    Q, K, V, dA = (O.to_bf16(rng.standard_normal(shape).astype(np.float32)*0.1)
                   for _ in range(4))
    S = shape[1]
    i = np.arange(S)
    band = F(np.where(np.abs(i[:, None] - i[None, :]) <= 32, 0.0, -np.inf).astype(np.float32))
    mask = O.to_bf16(band)
    A1, l1, _ = run_fwd(Q, K, V, mask)
    A2, l2, _ = run_fwd(Q, K, V, mask, seq_tile=base[1], batch_tile=base[2:])
    a64, l64 = O.sdpa_fp64(Q, K, V, mask)
    assert O.rel_err(bf(A1), a64) <= 1e-2
    assert O.rel_err(bf(A2), a64) <= 1e-2
    assert np.allclose(to_fortran(l1), l64, rtol=1e-3, atol=1e-3)
    assert np.allclose(to_fortran(l2), l64, rtol=1e-3, atol=1e-3)
    q64, k64, v64 = O.sdpa_bwd_fp64(Q, K, V, to_fortran(A1), dA, mask, to_fortran(l1))
    for tiles in (None, base):
        dK, dQ, dV = (torch.zeros_like(A1) for _ in range(3))
        flash_sdpa_bwd_async(dev(K), dev(Q), dev(V), A1, dev(dA), dev(mask), l1, dK, dQ, dV,
                             None if tiles is None else base[1],
                             None if tiles is None else base[2:])
        torch.cuda.synchronize()
        # many bf16 `+=` steps when tiled: the reference's own tolerance is 1e-2 per step
        tol = 1e-2 if tiles is None else 3e-2
        for got, w in ((dQ, q64), (dK, k64), (dV, v64)):
            assert O.rel_err(bf(got), w) <= tol


def test_layer_flash_forward_backward_matches_vanilla_oracle():
    """nntile.layer.Sdpa with flash_attention=True against the unfused fp32 chain
    of the oracle (the reference's tiled path), bf16 bar 2e-2."""
    rng = np.random.default_rng(3)
    shape = (64, 256, 2, 2, 2)
    Qf, Kf, Vf, dYf = (F(rng.standard_normal(shape).astype(np.float32)) for _ in range(4))
    Q, K, V, dY = (O.to_bf16(x) for x in (Qf, Kf, Vf, dYf))
    maskb = F(np.triu(np.ones((256, 256), dtype=bool)))
    q32, k32, v32, dy32 = (O.from_bf16(x) for x in (Q, K, V, dY))
    want, attn, _ = O.vanilla_forward(q32, k32, v32, maskb)
    wq, wk, wv = (O.zeros(shape, np.float32) for _ in range(3))
    O.vanilla_backward(q32, k32, v32, want, dy32, attn, maskb, wq, wk, wv)
    layer = Sdpa(dev(Q), dev(K), dev(V), mask=dev(O.to_bf16(causal_add(256))),
                 flash_attention=True, seq_tile=128, batch_tile=(1, 2, 1))
    y = layer.forward_async()
    assert O.rel_err(bf(y), want) <= BF16_TOL
    dq, dk, dv = (torch.zeros_like(layer.q) for _ in range(3))
    layer.backward_async(dev(dY), dq, dk, dv)
    torch.cuda.synchronize()
    for got, w in ((dq, wq), (dk, wk), (dv, wv)):
        assert O.rel_err(bf(got), w) <= BF16_TOL


def test_forward_merges_into_existing_partial_result():
    """Two K/V tiles fed by hand through the tile-level entry point: the second
    call must merge with the (lse, A) the first one left (RW semantics)."""
    rng = np.random.default_rng(8)
    head, seq, batch = 64, 128, 2
    Q, K1, V1, K2, V2 = (O.to_bf16(rng.standard_normal((head, seq, batch, 1, 1))
                                   .astype(np.float32)) for _ in range(5))
    zero = O.to_bf16(np.zeros((seq, seq), np.float32))
    lse = torch.full((batch, seq), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros((batch, seq, head), dtype=torch.bfloat16, device="cuda")
    s_l = torch.empty_like(lse)
    s_A = torch.empty_like(A)
    for Kt, Vt in ((K1, V1), (K2, V2)):
        ops.flash_sdpa_fwd(seq, head, batch, dev(Kt), dev(Q), dev(zero), s_l, dev(Vt), s_A,
                           lse, A)
    torch.cuda.synchronize()
    if ops.flash_sdpa_path(seq, head, batch) == 2:
        # status word of the tcgen05 kernel at the start of the scratch buffer:
        # 0 = every bounded wait completed
        assert int(s_A.view(torch.int32).flatten()[0].item()) == 0
    Kc = np.concatenate([O.from_bf16(K1), O.from_bf16(K2)], axis=1)
    Vc = np.concatenate([O.from_bf16(V1), O.from_bf16(V2)], axis=1)
    a64, l64 = O.sdpa_fp64(O.from_bf16(Q), Kc, Vc, np.zeros((2*seq, seq), np.float32))
    got = O.from_bf16(to_fortran(A.view(1, 1, batch, seq, head)))
    assert O.rel_err(got, a64) <= 1e-2
    assert np.allclose(lse.cpu().numpy().T, l64[:, :, 0, 0], rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("head,seq,batch,group,kvh,kind", [
    (128, 256, 2, 4, 2, "causal"),
    (64, 384, 1, 3, 2, "ragged"),
    (128, 128, 3, 2, 1, "none"),
])
def test_grouped_query_entry_points(head, seq, batch, group, kvh, kind):
    """Native GQA: K, V un-replicated.  Oracle = the reference's way: replicate K/V
    over the group (llama_attention.py:605-616), run the tile tasks, sum dK/dV over
    the group (:786-793)."""
    rng = np.random.default_rng(head + seq + group)
    qshape, kshape = (head, seq, batch, group, kvh), (head, seq, batch, kvh)
    Q, dA = (O.to_bf16(rng.standard_normal(qshape).astype(np.float32)) for _ in range(2))
    Kkv, Vkv = (O.to_bf16(rng.standard_normal(kshape).astype(np.float32)) for _ in range(2))
    Krep = F(np.repeat(Kkv[:, :, :, None, :], group, axis=3))
    Vrep = F(np.repeat(Vkv[:, :, :, None, :], group, axis=3))
    mask = O.to_bf16(make_mask(kind, seq))
    wantA, wantL = O.flash_forward(Q, Krep, Vrep, mask)
    fin = np.isfinite(wantL)
    q, k, v, m = dev(Q), dev(Kkv), dev(Vkv), dev(mask)
    lse = torch.full((kvh, group, batch, seq), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    nbytes = ops.flash_sdpa_gqa_scratch_bytes(seq, head, batch, group, kvh)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ops.flash_sdpa_fwd_gqa(seq, head, batch, group, kvh, k, q, m, v, lse, A, scratch)
    torch.cuda.synchronize()
    assert O.rel_err(bf(A), O.from_bf16(wantA)) <= BF16_TOL
    gl = to_fortran(lse)
    assert np.array_equal(np.isfinite(gl), fin)
    assert np.allclose(gl[fin], wantL[fin], rtol=1e-3, atol=1e-3)
    # backward from the oracle's A and lse; dK, dV start from a non-zero value ("+=")
    z = lambda: O.zeros(qshape, np.uint16)
    lse_in = F(np.where(fin, wantL, 0.0).astype(np.float32))
    wq, wk, wv = O.flash_backward(Q, Krep, Vrep, wantA, dA, mask, lse_in, z(), z(), z())
    wk_kv = O.from_bf16(wk).sum(axis=3) + 0.5
    wv_kv = O.from_bf16(wv).sum(axis=3) + 0.5
    dQ = torch.zeros_like(q)
    dK = torch.full(tuple(reversed(kshape)), 0.5, dtype=torch.bfloat16, device="cuda")
    dV = torch.full_like(dK, 0.5)
    ops.flash_sdpa_bwd_gqa(seq, head, batch, group, kvh, k, q, v, dev(wantA), dev(dA), m,
                           dev(lse_in), dK, dQ, dV, scratch)
    torch.cuda.synchronize()
    assert O.rel_err(bf(dQ), O.from_bf16(wq)) <= BF16_TOL
    assert O.rel_err(bf(dK), wk_kv) <= BF16_TOL
    assert O.rel_err(bf(dV), wv_kv) <= BF16_TOL
    # inputs untouched
    assert np.array_equal(to_fortran(k), Kkv) and np.array_equal(to_fortran(v), Vkv)


def test_grouped_query_rejects_unsupported_shape_and_small_scratch():
    from nntile_b200 import _lib
    t = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device="cuda")
    q, k = t(1, 2, 1, 80, 32), t(1, 1, 80, 32)
    lse = torch.zeros((1, 2, 1, 80), dtype=torch.float32, device="cuda")
    sc = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.StatusError):      # seq 80, head 32: no tcgen05 kernel
        ops.flash_sdpa_fwd_gqa(80, 32, 1, 2, 1, k, q, t(80, 80), k, lse, q, sc)
    q, k = t(1, 2, 1, 128, 128), t(1, 1, 128, 128)
    lse = torch.zeros((1, 2, 1, 128), dtype=torch.float32, device="cuda")
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.StatusError):
        ops.flash_sdpa_bwd_gqa(128, 128, 1, 2, 1, k, q, k, q, q, t(128, 128), lse, k, q, k, small)


def test_null_mask_tile_skips_the_pair():
    """Tensor level: a NULL mask entry = fully masked pair, no task; the result is
    the one with every pair submitted and shared zero / diagonal / -inf tiles."""
    import ctypes
    from nntile_b200 import _lib
    lib = _lib.load()
    D, S, St, H = 64, 512, 128, 3
    nt = S//St
    g = torch.Generator(device="cuda").manual_seed(4)
    rnd = lambda: [torch.randn((H, 1, 1, St, D), generator=g, device="cuda").to(torch.bfloat16)
                   for _ in range(nt)]
    Q, K, V, dY = rnd(), rnd(), rnd(), rnd()
    mz = dev(O.to_bf16(F(np.zeros((St, St), np.float32))))
    md = dev(O.to_bf16(causal_add(St)))
    mi = dev(O.to_bf16(F(np.full((St, St), -np.inf, np.float32))))
    i64 = ctypes.c_int64
    shape, base = (i64*5)(D, S, 1, 1, H), (i64*5)(D, St, 1, 1, H)
    nbytes = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(shape, base)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    parr = lambda ps: ctypes.cast((ctypes.c_void_p*len(ps))(*ps), ctypes.POINTER(ctypes.c_void_p))
    ptrs = lambda ts: parr([t.data_ptr() for t in ts])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    results = []
    for skip in (False, True):
        mp = [(0 if skip else mi.data_ptr()) if ki > qi else (mz if ki < qi else md).data_ptr()
              for qi in range(nt) for ki in range(nt)]
        A = [torch.zeros_like(q) for q in Q]
        lse = [torch.full((H, 1, 1, St), -np.inf, dtype=torch.float32, device="cuda") for _ in Q]
        dQ, dK, dV = ([torch.zeros_like(q) for q in Q] for _ in range(3))
        st = lib.nntile_b200_tensor_flash_sdpa_fwd_bf16(stream, shape, base, ptrs(K), ptrs(Q),
                parr(mp), ptrs(lse), ptrs(V), ptrs(A), ctypes.c_void_p(scratch.data_ptr()), nbytes)
        assert st == 0
        st = lib.nntile_b200_tensor_flash_sdpa_bwd_bf16(stream, shape, base, ptrs(K), ptrs(Q),
                ptrs(V), ptrs(A), ptrs(dY), parr(mp), ptrs(lse), ptrs(dK), ptrs(dQ), ptrs(dV),
                ctypes.c_void_p(scratch.data_ptr()), nbytes)
        assert st == 0
        torch.cuda.synchronize()
        results.append([torch.stack(x) for x in (A, lse, dQ, dK, dV)])
    names = ("A", "lse", "dQ", "dK", "dV")
    for name, full, skipped in zip(names, *results):
        if name == "dQ":
            # dQ of a Q tile is summed in fp32 by red.add in whatever order the CTAs
            # finish; the sums agree to fp32 rounding, i.e. to one bf16 step at most
            d = (full.float() - skipped.float()).abs()
            assert float((d/(full.float().abs() + 1e-3)).max()) <= 2.0**-7
            assert float((d > 0).float().mean()) <= 1e-3
        else:
            assert torch.equal(full, skipped)   # a fully masked task changes nothing


def test_layer_forward_dynamic_prefill_then_decode():
    """Sdpa.forward_dynamic: fused path when the sequence lengths agree, the
    unfused chain against a longer key/value sequence, and the decode kernel on a
    KVCache - all against the oracle's unfused chain (sdpa.py:170-306)."""
    from nntile_b200.sdpa import KVCache
    rng = np.random.default_rng(8)
    D, S, B, G, H = 64, 128, 2, 2, 1
    shape = (D, S, B, G, H)
    Q, K, V = (O.to_bf16(F(rng.standard_normal(shape).astype(np.float32))) for _ in range(3))
    layer = Sdpa(dev(Q), dev(K), dev(V), mask=dev(O.to_bf16(causal_add(S))),
                 flash_attention=True)
    maskb = F(np.triu(np.ones((S, S), dtype=bool)))
    want, _, _ = O.vanilla_forward(O.from_bf16(Q), O.from_bf16(K), O.from_bf16(V), maskb)
    y = layer.forward_dynamic(dev(Q), dev(K), dev(V))
    torch.cuda.synchronize()
    assert O.rel_err(bf(y), want) <= BF16_TOL
    # one new query against S + 1 keys: unfused chain, no mask
    q1 = O.to_bf16(F(rng.standard_normal((D, 1, B, G, H)).astype(np.float32)))
    k1, v1 = (O.to_bf16(F(rng.standard_normal((D, 1, B, G, H)).astype(np.float32)))
              for _ in range(2))
    Kall, Vall = F(np.concatenate([K, k1], axis=1)), F(np.concatenate([V, v1], axis=1))
    want1, _, _ = O.vanilla_forward(O.from_bf16(q1), O.from_bf16(Kall), O.from_bf16(Vall), None)
    plain = Sdpa(dev(Q), dev(K), dev(V), flash_attention=False)
    y1 = plain.forward_dynamic(dev(q1), dev(Kall), dev(Vall))
    torch.cuda.synchronize()
    assert O.rel_err(bf(y1), want1) <= BF16_TOL
    # the same step on an un-replicated cache (group 2 shares one kv head here only if
    # the replicas are equal: build K/V with equal group entries)
    Kkv = F(Kall[:, :, :, 0, :])
    Vkv = F(Vall[:, :, :, 0, :])
    Krep = F(np.repeat(Kkv[:, :, :, None, :], G, axis=3))
    Vrep = F(np.repeat(Vkv[:, :, :, None, :], G, axis=3))
    want2, _, _ = O.vanilla_forward(O.from_bf16(q1), O.from_bf16(Krep), O.from_bf16(Vrep), None)
    cache = KVCache(256, H, B, D)
    cache.append(dev(Kkv), dev(Vkv))
    y2 = layer.forward_dynamic(dev(q1), None, None, kv_cache=cache)
    torch.cuda.synchronize()
    assert O.rel_err(bf(y2), want2) <= BF16_TOL
