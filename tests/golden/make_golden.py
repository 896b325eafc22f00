"""Regenerate the golden vectors under tests/golden/.

Needs the reference checkout: the expected outputs of the unfused kernels come
from the reference's own CPU kernels (oracle/_ref, built in place from the
reference sources by oracle/build.py).  The fused-path vectors use the fp64
formulas and the PRESET / banded-mask input generators of the reference's own
tests (tests/kernel/flash_sdpa_{fwd,bwd}_cudnn.cc,
wrappers/python/tests/nntile_core/test_tensor_flash_sdpa_fwd_cudnn.py).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def ref_kernel_vectors():
    """Each unfused kernel on seeded inputs, outputs from the reference build."""
    assert O.have_ref(), "build oracle/_ref first (needs the reference checkout)"
    rng = np.random.default_rng(1234)
    out = {}
    F = np.asfortranarray

    def rnd(*shape):
        return F(rng.standard_normal(shape).astype(np.float32))

    for tag, (m, n, k) in {"m1": (1, 24, 37), "m3": (3, 5, 11)}.items():
        src = rnd(m, k, n)
        src[:, 1::5, :] = -np.inf                     # masked entries
        src[:, :, 2] = -np.inf                        # one fully masked fibre
        dst = O.zeros((2, m, n), np.float32)
        O.maxsumexp(m, n, k, src, dst, backend="ref")
        first = dst.copy(order="F")
        src2 = rnd(m, k, n) * 2
        O.maxsumexp(m, n, k, src2, dst, backend="ref")  # accumulate a second tile
        out[f"maxsumexp_{tag}_src"] = src
        out[f"maxsumexp_{tag}_src2"] = src2
        out[f"maxsumexp_{tag}_first"] = first
        out[f"maxsumexp_{tag}_second"] = dst
        sm = src.copy(order="F")
        O.softmax_inplace(m, n, k, first, 0.75, sm, backend="ref")
        out[f"softmax_{tag}_out"] = sm
        a, b = rnd(m, k, n), rnd(m, k, n)
        d0 = rnd(m, n)
        d = d0.copy(order="F")
        O.sumprod_slice(m, n, k, 1.5, a, b, -0.5, d, backend="ref")
        dz = d0.copy(order="F")
        O.sumprod_slice(m, n, k, 1.0, a, b, 0.0, dz, backend="ref")
        out[f"sumprod_{tag}_a"], out[f"sumprod_{tag}_b"] = a, b
        out[f"sumprod_{tag}_dst0"] = d0
        out[f"sumprod_{tag}_out"], out[f"sumprod_{tag}_out_beta0"] = d, dz
        s = rnd(m, n)
        t0 = rnd(m, k, n)
        t = t0.copy(order="F")
        O.add_slice_inplace(m, n, k, -1.0, s, 1.0, t, backend="ref")
        out[f"addslice_{tag}_src"], out[f"addslice_{tag}_dst0"] = s, t0
        out[f"addslice_{tag}_out"] = t
    nrows, ncols = 35, 6
    mask = F((rng.random(nrows) > 0.4).astype(np.uint8))
    d0 = rnd(nrows, ncols)
    d = d0.copy(order="F")
    O.mask_scalar(nrows, ncols, mask, -np.inf, d, backend="ref")
    out["mask_mask"], out["mask_dst0"], out["mask_out"] = mask, d0, d
    x, y0 = rnd(301), rnd(301)
    y = y0.copy()
    O.multiply_inplace(301, 0.5, x, y, backend="ref")
    out["mul_src"], out["mul_dst0"], out["mul_out"] = x, y0, y
    y = y0.copy()
    O.add_inplace(301, 2.0, x, -1.0, y, backend="ref")
    out["add_out"] = y
    # accumulate_attn_output, CPU-build rules (the only ones the reference
    # compiles on a CPU): head 15 exercises the non-vector path
    head, seq, batch = 15, 9, 2
    sl, dl = rnd(seq * batch), rnd(seq * batch)
    sl[3], dl[5], sl[7], dl[7] = -np.inf, -np.inf, -np.inf, -np.inf
    sa, da0 = rnd(head, seq * batch), rnd(head, seq * batch)
    da, dl2 = da0.copy(order="F"), dl.copy()
    O.accumulate_attn_output(head, seq, batch, sl, sa, dl2, da, backend="ref")
    out["acc_src_lse"], out["acc_dst_lse0"] = sl, dl
    out["acc_src_attn"], out["acc_dst_attn0"] = sa, da0
    out["acc_dst_lse"], out["acc_dst_attn"] = dl2, da
    # batched gemm as the chain uses it
    m, n, k, batch = 7, 5, 16, 3
    A, B = rnd(k, m, batch), rnd(k, n, batch)
    C0 = rnd(m, n, batch)
    C = C0.copy(order="F")
    O.gemm(1, 0, m, n, k, batch, 0.125, A, B, 1.0, C, backend="ref")
    out["gemm_A"], out["gemm_B"], out["gemm_C0"], out["gemm_out"] = A, B, C0, C
    return out


def chain_vectors():
    """The unfused forward+backward chain of BASELINE config 1 at reduced size
    (head 16, seq 48, batch 2, one kv head), run by the reference's kernels."""
    rng = np.random.default_rng(0)
    D, S, B, G, H = 16, 48, 2, 1, 1
    F = np.asfortranarray
    Q, K, V, dY = (F(rng.standard_normal((D, S, B, G, H)).astype(np.float32))
                   for _ in range(4))
    mask = F(np.triu(np.ones((S, S), dtype=bool)))      # [k, q]: keep k <= q
    Y, attn, mse = O.vanilla_forward(Q, K, V, mask, backend="ref")
    dQ, dK, dV = (O.zeros(Q.shape, np.float32) for _ in range(3))
    O.vanilla_backward(Q, K, V, Y, dY, attn, mask, dQ, dK, dV, backend="ref")
    return dict(chain_Q=Q, chain_K=K, chain_V=V, chain_dY=dY, chain_Y=Y,
                chain_mse=mse, chain_dQ=dQ, chain_dK=dK, chain_dV=dV)


def preset_fwd(seq, head, batch, causal):
    """tests/kernel/flash_sdpa_fwd_cudnn.cc:211-263 PRESET generator."""
    i = np.arange(batch * seq * head)
    val = ((i % 20 - 10) * 0.1).astype(np.float32)
    K = val
    Q = (val * np.float32(0.8)).astype(np.float32)
    V = (val * np.float32(1.2)).astype(np.float32)
    mask = np.zeros((seq, seq), dtype=np.float32)          # [q][k] row major
    if causal:
        mask[np.triu_indices(seq, 1)] = -np.inf
    return Q, K, V, mask


def preset_bwd(seq, head, batch, causal):
    """tests/kernel/flash_sdpa_bwd_cudnn.cc:114-129 PRESET generator."""
    total = batch * seq * head
    i = np.arange(total)
    base = ((i % 23 - 11) * 0.04).astype(np.float32)
    K = base
    Q = (base * np.float32(0.7)).astype(np.float32)
    V = (base * np.float32(1.1)).astype(np.float32)
    A = (base * np.float32(-0.3)).astype(np.float32)
    dA = (0.02 * ((i % 17) - 8)).astype(np.float32)
    j = np.arange(batch * seq)
    lse = ((j % 13 - 6) * 0.01).astype(np.float32)
    mask = np.zeros((seq, seq), dtype=np.float32)
    if causal:
        mask[np.triu_indices(seq, 1)] = -np.inf
    return Q, K, V, A, dA, lse, mask


def _as5(flat, head, seq, batch):
    """[batch][seq][head] row major == Fortran [head, seq, batch, 1, 1]."""
    return np.asfortranarray(flat.reshape(batch, seq, head).transpose(2, 1, 0)
                             .reshape(head, seq, batch, 1, 1))


def flash_vectors():
    out = {}
    for seq, head, batch, causal in [(16, 32, 1, True), (32, 64, 2, True),
                                     (32, 32, 2, False), (16, 64, 1, False)]:
        Q, K, V, mask = preset_fwd(seq, head, batch, causal)
        Qb, Kb, Vb = (O.to_bf16(_as5(x, head, seq, batch)) for x in (Q, K, V))
        mkq = O.to_bf16(np.asfortranarray(mask.T))          # Fortran [k, q]
        a, lse = O.sdpa_fp64(Qb, Kb, Vb, mkq)
        tag = f"fwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
        out[tag + "_A"] = a.astype(np.float32)
        out[tag + "_lse"] = lse.astype(np.float32)
    for seq, head, batch, causal in [(64, 8, 1, True), (64, 32, 4, True),
                                     (64, 32, 1, False), (64, 8, 4, False)]:
        Q, K, V, A, dA, lse, mask = preset_bwd(seq, head, batch, causal)
        Qb, Kb, Vb, Ab, dAb = (O.to_bf16(_as5(x, head, seq, batch))
                               for x in (Q, K, V, A, dA))
        mkq = O.to_bf16(np.asfortranarray(mask.T))
        l4 = np.asfortranarray(lse.reshape(batch, seq).T.reshape(seq, batch, 1, 1))
        dq, dk, dv = O.sdpa_bwd_fp64(Qb, Kb, Vb, Ab, dAb, mkq, l4)
        tag = f"bwd_s{seq}_h{head}_b{batch}_{'causal' if causal else 'full'}"
        out[tag + "_dQ"] = dq.astype(np.float32)
        out[tag + "_dK"] = dk.astype(np.float32)
        out[tag + "_dV"] = dv.astype(np.float32)
    return out


def around_vectors():
    """The passes the reference's attention layers run around the SDPA layer
    (transpose + rope, transpose + bias, transpose back), by its own CPU kernels."""
    assert O.have_ref(), "build oracle/_ref first (needs the reference checkout)"
    rng = np.random.default_rng(77)
    out = {}
    for tag, (lead, head, seq, batch) in {"llama_q": (8, 64, 7, 3), "llama_k": (2, 128, 5, 2),
                                           "gpt2": (12, 64, 6, 2)}.items():
        proj = O.to_bf16(np.asfortranarray(
            rng.standard_normal((lead, head, seq, batch)).astype(np.float32)))
        pos = np.tile(np.arange(seq) + 3, (batch, 1))
        sin, cos = (O.to_bf16(x) for x in O.rope_sin_cos(head, pos))
        bias = O.to_bf16(np.asfortranarray(rng.standard_normal((head, lead)).astype(np.float32)))
        out[f"{tag}_proj"], out[f"{tag}_sin"], out[f"{tag}_cos"] = proj, sin, cos
        out[f"{tag}_bias"] = bias
        out[f"{tag}_rope"] = O.attention_prologue(proj, sin, cos, backend="ref")
        out[f"{tag}_plain"] = O.attention_prologue(proj, backend="ref")
        out[f"{tag}_biased"] = O.attention_prologue(proj, bias=bias, backend="ref")
        out[f"{tag}_back"] = O.attention_epilogue(out[f"{tag}_rope"], backend="ref")
    return out


def main():
    np.savez_compressed(os.path.join(HERE, "ref_around.npz"), **around_vectors())
    np.savez_compressed(os.path.join(HERE, "ref_kernels.npz"), **ref_kernel_vectors())
    np.savez_compressed(os.path.join(HERE, "ref_chain.npz"), **chain_vectors())
    np.savez_compressed(os.path.join(HERE, "flash_preset.npz"), **flash_vectors())
    for f in ("ref_kernels.npz", "ref_chain.npz", "flash_preset.npz", "ref_around.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
