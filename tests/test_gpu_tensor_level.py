"""GPU tests of the tensor-level entry points and of the layer above them at the
sizes the tile loops exist for:

* config 4's real shape (seq 16384, seq-tile 2048: 8 x 8 (Q tile, K/V tile) tasks)
  against the single-tile call on the same data and against fp32 torch;
* config 3's full shape through the grouped-query entry points against the
  replicated-K/V entry points, and run to run;
* the grouped-query form of the tile loops;
* the tile loops of the unfused chain (K tiles accumulate into one (max, sum) pair);
* the failure report: a wait that runs out sets the status word, the kernel returns
  normally, every later task of the call is skipped, the next call is clean.

Tolerances (bf16 storage, fp32 accumulation): forward 2e-2, backward 2e-2 relative
(3e-2 where one side rounds per tile task and the other once), Frobenius over the
tensor AND as a maximum over (batch, head) slices."""
import ctypes
import math

import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import _lib, ops
from nntile_b200.sdpa import (Sdpa, flash_sdpa_bwd_async, flash_sdpa_fwd_async, from_fortran,
                              to_fortran)

pytestmark = pytest.mark.gpu
F = np.asfortranarray


def causal(S, dtype=torch.bfloat16):
    q = torch.arange(S, device="cuda")[:, None]
    k = torch.arange(S, device="cuda")[None, :]
    return torch.where(k > q, -math.inf, 0.0).to(dtype)


def slice_errs(got, want, slice_dims):
    """Frobenius relative error over the whole tensor and its maximum over slices
    (`slice_dims` = leading axes that index the slices)."""
    g, w = got.float(), want.float()
    whole = float((g - w).norm()/w.norm())
    g2, w2 = g.flatten(0, slice_dims - 1).flatten(1), w.flatten(0, slice_dims - 1).flatten(1)
    per = (g2 - w2).norm(dim=1)/w2.norm(dim=1).clamp_min(1e-30)
    return whole, float(per.max())


def parr(ptrs):
    return ctypes.cast((ctypes.c_void_p*len(ptrs))(*ptrs), ctypes.POINTER(ctypes.c_void_p))


def test_config4_tile_tasks_equal_one_tile_and_fp32():
    """BASELINE config 4 on 2 of its 16 heads: seq 16384 as 8 x 8 tile tasks of 2048,
    once with every pair submitted and once with NULL mask tiles for the 28 fully
    masked pairs, against ONE tile task of seq 16384 (128 blocks) on the same data."""
    lib = _lib.load()
    D, S, St, H = 128, 16384, 2048, 2
    nt = S//St
    g = torch.Generator(device="cuda").manual_seed(3)
    rnd = lambda: torch.randn((H, S, D), generator=g, device="cuda").to(torch.bfloat16)
    q, k, v, dy = rnd(), rnd(), rnd(), rnd()
    # ---- single tile: one task over the whole sequence
    big_mask = causal(S)
    lse1 = torch.full((H, S), -math.inf, dtype=torch.float32, device="cuda")
    A1 = torch.zeros_like(q)
    s_l, s1, s2, s3 = torch.empty_like(lse1), torch.empty_like(q), torch.empty_like(q), \
        torch.empty_like(q)
    ops.flash_sdpa_fwd(S, D, H, k, q, big_mask, s_l, v, s1, lse1, A1)
    dK1, dQ1, dV1 = (torch.zeros_like(q) for _ in range(3))
    ops.flash_sdpa_bwd(S, D, H, k, q, v, A1, dy, big_mask, lse1, s1, s2, s3, dK1, dQ1, dV1)
    torch.cuda.synchronize()
    assert ops.flash_sdpa_read_status(s3) == 0
    del big_mask
    # ---- tiled: every tile its own buffer, three mask buffers shared by the 64 pairs
    cut = lambda x: [x[:, i*St:(i + 1)*St].contiguous() for i in range(nt)]
    Q, K, V, dY = cut(q), cut(k), cut(v), cut(dy)
    mz = torch.zeros((St, St), dtype=torch.bfloat16, device="cuda")
    mi = torch.full((St, St), -math.inf, dtype=torch.bfloat16, device="cuda")
    md = causal(St)
    i64 = ctypes.c_int64
    shape, base = (i64*5)(D, S, 1, 1, H), (i64*5)(D, St, 1, 1, H)
    nbytes = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(shape, base)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptrs = lambda ts: parr([t.data_ptr() for t in ts])
    outs = []
    for skip in (False, True):
        mp = [(0 if skip else mi.data_ptr()) if ki > qi else (mz if ki < qi else md).data_ptr()
              for qi in range(nt) for ki in range(nt)]
        A = [torch.zeros_like(t) for t in Q]
        lse = [torch.full((H, St), -math.inf, dtype=torch.float32, device="cuda") for _ in Q]
        dQ, dK, dV = ([torch.zeros_like(t) for t in Q] for _ in range(3))
        st = lib.nntile_b200_tensor_flash_sdpa_fwd_bf16(
            stream, shape, base, ptrs(K), ptrs(Q), parr(mp), ptrs(lse), ptrs(V), ptrs(A),
            ctypes.c_void_p(scratch.data_ptr()), nbytes)
        assert st == 0
        st = lib.nntile_b200_tensor_flash_sdpa_bwd_bf16(
            stream, shape, base, ptrs(K), ptrs(Q), ptrs(V), ptrs(A), ptrs(dY), parr(mp),
            ptrs(lse), ptrs(dK), ptrs(dQ), ptrs(dV), ctypes.c_void_p(scratch.data_ptr()), nbytes)
        assert st == 0
        torch.cuda.synchronize()
        assert ops.flash_sdpa_read_status(scratch) == 0
        outs.append([torch.cat(x, dim=1) for x in (A, lse, dQ, dK, dV)])
    for name, full, skipped in zip(("A", "lse", "dQ", "dK", "dV"), *outs):
        if name == "dQ":       # fp32 red.add order: equal to fp32 rounding
            assert slice_errs(full, skipped, 1)[1] <= 1e-3
        else:
            assert torch.equal(full, skipped)
    A, lse, dQ, dK, dV = outs[1]
    # tiled (one bf16 rounding of A per K/V tile) against the single tile
    for name, got, want, tol in (("A", A, A1, 2e-2), ("dQ", dQ, dQ1, 3e-2), ("dK", dK, dK1, 3e-2),
                                 ("dV", dV, dV1, 3e-2)):
        whole, worst = slice_errs(got, want, 1)
        assert whole <= tol and worst <= tol, (name, whole, worst)
    assert torch.allclose(lse, lse1, rtol=1e-3, atol=1e-3)
    # fp32 torch on both heads, the last 2048 queries (they see all 16384 keys)
    for h in range(H):
        qs = q[h, -St:].float()
        sc = (qs @ k[h].float().T)/math.sqrt(D)
        sc = sc + torch.where(torch.arange(S, device="cuda")[None, :]
                              > (S - St + torch.arange(St, device="cuda"))[:, None],
                              -math.inf, 0.0)
        ref = torch.softmax(sc, dim=1) @ v[h].float()
        assert float((A[h, -St:].float() - ref).norm()/ref.norm()) <= 2e-2
        assert torch.allclose(lse[h, -St:], torch.logsumexp(sc, dim=1), rtol=1e-3, atol=1e-3)


def test_config3_grouped_query_equals_replicated_at_full_size():
    """BASELINE config 3 (seq 4096, head 128, batch 4, group 4, 8 kv heads) through
    the grouped-query entry points against the replicated-K/V entry points: A, lse and
    dQ agree, dK/dV equal the sum over the group; two runs in a row differ by no more
    than the order of the bf16 additions of the `group` CTAs that share a tile."""
    S, D, B, G, H = 4096, 128, 4, 4, 8
    g = torch.Generator(device="cuda").manual_seed(2)
    q, dy = (torch.randn((H, G, B, S, D), generator=g, device="cuda").to(torch.bfloat16)
             for _ in range(2))
    k, v = (torch.randn((H, B, S, D), generator=g, device="cuda").to(torch.bfloat16)
            for _ in range(2))
    mask = causal(S)
    nb = H*G*B
    # replicated reference run
    krep = k[:, None].expand(H, G, B, S, D).contiguous()
    vrep = v[:, None].expand(H, G, B, S, D).contiguous()
    lse_r = torch.full((H, G, B, S), -math.inf, dtype=torch.float32, device="cuda")
    A_r = torch.zeros_like(q)
    s_l, s1, s2, s3 = torch.empty_like(lse_r), torch.empty_like(q), torch.empty_like(q), \
        torch.empty_like(q)
    ops.flash_sdpa_fwd(S, D, nb, krep, q, mask, s_l, vrep, s1, lse_r, A_r)
    dK_r, dQ_r, dV_r = (torch.zeros_like(q) for _ in range(3))
    ops.flash_sdpa_bwd(S, D, nb, krep, q, vrep, A_r, dy, mask, lse_r, s1, s2, s3, dK_r, dQ_r,
                       dV_r)
    torch.cuda.synchronize()
    assert ops.flash_sdpa_read_status(s3) == 0
    dK_sum, dV_sum = dK_r.float().sum(dim=1), dV_r.float().sum(dim=1)
    del krep, vrep, s1, s2, s3, dK_r, dV_r
    scratch = torch.empty(ops.flash_sdpa_gqa_scratch_bytes(S, D, B, G, H), dtype=torch.uint8,
                          device="cuda")
    runs = []
    for _ in range(2):
        lse = torch.full((H, G, B, S), -math.inf, dtype=torch.float32, device="cuda")
        A = torch.zeros_like(q)
        ops.flash_sdpa_fwd_gqa(S, D, B, G, H, k, q, mask, v, lse, A, scratch)
        dQ = torch.zeros_like(q)
        dK, dV = torch.zeros_like(k), torch.zeros_like(k)
        ops.flash_sdpa_bwd_gqa(S, D, B, G, H, k, q, v, A, dy, mask, lse, dK, dQ, dV, scratch)
        torch.cuda.synchronize()
        assert ops.flash_sdpa_read_status(scratch) == 0
        runs.append((A, lse, dQ, dK, dV))
    A, lse, dQ, dK, dV = runs[0]
    assert torch.equal(A, A_r) and torch.equal(lse, lse_r)      # same kernel, same data
    assert slice_errs(dQ, dQ_r, 3)[1] <= 1e-3
    for name, got, want in (("dK", dK, dK_sum), ("dV", dV, dV_sum)):
        whole, worst = slice_errs(got, want, 2)
        assert whole <= 2e-2 and worst <= 2e-2, (name, whole, worst)
    # run to run: `group` = 4 bf16 additions per element in any order; each addition
    # rounds to 2^-9 relative of the running value, so two orders differ by a few
    # bf16 steps of the largest partial sum at most
    for got, again in ((dK, runs[1][3]), (dV, runs[1][4])):
        d = (got.float() - again.float()).abs()
        bound = 4*2.0**-8*got.float().abs().amax()
        assert float(d.max()) <= float(bound)
        assert slice_errs(got, again, 2)[1] <= 5e-3
    assert torch.equal(runs[0][0], runs[1][0])


@pytest.mark.parametrize("seq_tile,batch_tile", [(128, (1, 2, 1)), (256, (2, 1, 2))])
def test_grouped_query_tile_loops(seq_tile, batch_tile):
    """K, V un-replicated at the tensor level: the oracle runs the reference's way
    (replicate, tile tasks, sum dK/dV over the group)."""
    rng = np.random.default_rng(seq_tile)
    D, S, B, G, H = 64, 512, 2, 2, 2
    qshape, kshape = (D, S, B, G, H), (D, S, B, H)
    Q, dA = (O.to_bf16(rng.standard_normal(qshape).astype(np.float32)) for _ in range(2))
    Kkv, Vkv = (O.to_bf16(rng.standard_normal(kshape).astype(np.float32)) for _ in range(2))
    Krep = F(np.repeat(Kkv[:, :, :, None, :], G, axis=3))
    Vrep = F(np.repeat(Vkv[:, :, :, None, :], G, axis=3))
    kk, qq = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
    mask = O.to_bf16(F(np.where(kk > qq, -np.inf, 0.0).astype(np.float32)))
    wantA, wantL = O.flash_forward(Q, Krep, Vrep, mask, seq_tile=seq_tile)
    q, k, v, m = (from_fortran(x) for x in (Q, Kkv, Vkv, mask))
    lse = torch.full((H, G, B, S), -np.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(q)
    flash_sdpa_fwd_async(k, q, m, lse, v, A, seq_tile, batch_tile)
    torch.cuda.synchronize()
    assert O.rel_err(O.from_bf16(to_fortran(A)), O.from_bf16(wantA)) <= 2e-2
    assert np.allclose(to_fortran(lse), wantL, rtol=1e-3, atol=1e-3)
    z = lambda: O.zeros(qshape, np.uint16)
    wq, wk, wv = O.flash_backward(Q, Krep, Vrep, wantA, dA, mask, wantL, z(), z(), z(),
                                  seq_tile=seq_tile)
    dQ = torch.zeros_like(q)
    dK, dV = torch.zeros_like(k), torch.zeros_like(k)
    flash_sdpa_bwd_async(k, q, v, from_fortran(wantA), from_fortran(dA), m, from_fortran(wantL),
                         dK, dQ, dV, seq_tile, batch_tile)
    torch.cuda.synchronize()
    assert O.rel_err(O.from_bf16(to_fortran(dQ)), O.from_bf16(wq)) <= 3e-2
    assert O.rel_err(O.from_bf16(to_fortran(dK)), O.from_bf16(wk).sum(axis=3)) <= 3e-2
    assert O.rel_err(O.from_bf16(to_fortran(dV)), O.from_bf16(wv).sum(axis=3)) <= 3e-2


@pytest.mark.parametrize("dtype,tol", [(np.float32, 1e-5), (np.uint16, 2e-2)])
def test_unfused_chain_tile_loops(dtype, tol):
    """Sdpa(flash_attention=False) on tensors cut along queries, keys and batch: the
    K tiles of a query tile accumulate into one (max, sum) pair and into one output
    tile, as src/tensor/{gemm,maxsumexp,softmax_inplace}.cc loop.  Forward against the
    oracle's tile loops, backward against the single-tile chain."""
    rng = np.random.default_rng(9)
    D, S, B, G, H = 32, 96, 2, 1, 2
    shape = (D, S, B, G, H)
    mk = lambda: O.cast(F(rng.standard_normal(shape).astype(np.float32)), dtype)
    Q, K, V, dY = mk(), mk(), mk(), mk()
    mask = F(np.triu(np.ones((S, S), dtype=bool)))           # [k, q]: keep k <= q
    wantY, want_attn, want_mse = O.vanilla_forward(Q, K, V, mask, q_tile=32, k_tile=48,
                                                   batch_tile=(1, 1, 2))
    q, k, v, dy, m = (from_fortran(x) for x in (Q, K, V, dY, mask))
    layer = Sdpa(q, k, v, mask=m, q_tile=32, k_tile=48, batch_tile=(1, 1, 2))
    y = layer.forward_async()
    torch.cuda.synchronize()
    got = O.as_f32(to_fortran(y))
    assert O.rel_err(got, O.as_f32(wantY)) <= tol
    assert O.rel_err(O.as_f32(to_fortran(layer.attn)), O.as_f32(want_attn)) <= tol
    # backward: tiled against the one-tile chain of the oracle
    z = lambda: O.zeros(shape, dtype)
    wq, wk, wv = z(), z(), z()
    Y1, attn1, _ = O.vanilla_forward(Q, K, V, mask)
    O.vanilla_backward(Q, K, V, Y1, dY, attn1, mask, wq, wk, wv)
    dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
    layer.backward_async(dy, dq, dk, dv)
    torch.cuda.synchronize()
    btol = tol if dtype == np.float32 else 3e-2
    for got_t, want in ((dq, wq), (dk, wk), (dv, wv)):
        assert O.rel_err(O.as_f32(to_fortran(got_t)), O.as_f32(want)) <= btol


def test_a_wait_that_runs_out_is_reported_and_contained():
    """Failure detection without a fault: the armed test instantiation of the forward
    kernel gives up a wait after 1 ms (its producer withholds one K copy), records a
    status code and returns; the C call had returned 0 long before.  In a tensor-level
    call the word is shared by all tasks and never cleared, so the tasks behind the
    failing one are skipped and the code survives; the next call is clean."""
    lib = _lib.load()
    D, S, St, H = 128, 512, 128, 1
    nt = S//St
    g = torch.Generator(device="cuda").manual_seed(8)
    rnd = lambda: [torch.randn((H, St, D), generator=g, device="cuda").to(torch.bfloat16)
                   for _ in range(nt)]
    Q, K, V = rnd(), rnd(), rnd()
    mz = torch.zeros((St, St), dtype=torch.bfloat16, device="cuda")
    md = causal(St)
    i64 = ctypes.c_int64
    shape, base = (i64*5)(D, S, 1, 1, H), (i64*5)(D, St, 1, 1, H)
    nbytes = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(shape, base)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptrs = lambda ts: parr([t.data_ptr() for t in ts])
    mp = [0 if ki > qi else (mz if ki < qi else md).data_ptr()
          for qi in range(nt) for ki in range(nt)]

    def run():
        A = [torch.zeros_like(t) for t in Q]
        lse = [torch.full((H, St), -math.inf, dtype=torch.float32, device="cuda") for _ in Q]
        st = lib.nntile_b200_tensor_flash_sdpa_fwd_bf16(
            stream, shape, base, ptrs(K), ptrs(Q), parr(mp), ptrs(lse), ptrs(V), ptrs(A),
            ctypes.c_void_p(scratch.data_ptr()), nbytes)
        assert st == 0                          # enqueue-only: nothing has failed yet
        torch.cuda.synchronize()                # the kernels return by themselves
        return torch.cat(A, dim=1), torch.cat(lse, dim=1)

    good_A, good_lse = run()
    assert ops.flash_sdpa_read_status(scratch) == 0
    lib.nntile_b200_test_arm_wait_timeout()     # the next forward launch only
    bad_A, bad_lse = run()
    code = ops.flash_sdpa_read_status(scratch)
    assert code in (1, 2, 3), code              # a forward role gave up
    # the failing task (Q tile 0) and everything enqueued behind it did no work
    assert not torch.equal(bad_lse, good_lse)
    again_A, again_lse = run()                  # hook disarmed, status cleared by the call
    assert ops.flash_sdpa_read_status(scratch) == 0
    assert torch.equal(again_A, good_A) and torch.equal(again_lse, good_lse)
    # tile level: the word sits at the start of scratch_A and is cleared per task
    s_l = torch.empty((H, St), dtype=torch.float32, device="cuda")
    s_A = torch.empty_like(Q[0])
    lse = torch.full((H, St), -math.inf, dtype=torch.float32, device="cuda")
    A = torch.zeros_like(Q[0])
    lib.nntile_b200_test_arm_wait_timeout()
    ops.flash_sdpa_fwd(St, D, H, K[0], Q[0], md, s_l, V[0], s_A, lse, A)
    assert ops.flash_sdpa_read_status(s_A) in (1, 2, 3)
    ops.flash_sdpa_fwd(St, D, H, K[0], Q[0], md, s_l, V[0], s_A, lse, A)
    assert ops.flash_sdpa_read_status(s_A) == 0
    assert torch.equal(A, good_A[:, :St])
