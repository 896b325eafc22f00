"""Second parity witness of the fused pair: the reference's OWN GPU code path -
its cuDNN graph wrappers src/kernel/flash_sdpa_{fwd,bwd}_cudnn/cuda.cc with the merge
kernel (accumulate_attn_output/cuda.cu) and the three add_inplace passes, compiled in
place into oracle/_ref_gpu - fed the same seeded tiles as the C ABI of this library.

Tolerance: 2e-2 relative (bf16 storage, fp32 accumulation on both sides; cuDNN's
kernels and ours round P, dS and the outputs at the same points but sum in different
orders).  Skipped with the reason when the library is absent or cuDNN declines to
build a graph on the box."""
import ctypes
import math

import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops

pytestmark = pytest.mark.gpu


def rel(a, b):
    return float((a.float() - b.float()).norm()/b.float().norm())


@pytest.mark.parametrize("seq,head,batch,kind,dtype", [
    (256, 64, 6, "causal", torch.bfloat16),   # the reference's Python flash case (head 64, seq 256)
    (512, 128, 4, "causal", torch.bfloat16),
    (256, 128, 3, "band", torch.bfloat16),    # |q - k| <= 32, the reference tests' banded mask
    (128, 64, 2, "none", torch.bfloat16),
    (256, 128, 2, "causal", torch.float16),   # the fp16 instantiation of both sides
    (256, 64, 3, "band", torch.float16),
])
def test_reference_gpu_wrappers_agree_with_the_c_abi(seq, head, batch, kind, dtype):
    ref = O.ref_gpu()
    if ref is None:
        pytest.skip("oracle/_ref_gpu not built (needs the reference checkout at build time)")
    g = torch.Generator(device="cuda").manual_seed(seq + head)
    mk = lambda: torch.randn((batch, seq, head), generator=g, device="cuda").to(dtype)
    sfx = "fp16" if dtype == torch.float16 else "bf16"
    ref_fwd = getattr(ref, f"refgpu_flash_sdpa_fwd_{sfx}")
    ref_bwd = getattr(ref, f"refgpu_flash_sdpa_bwd_{sfx}")
    Q, K, V, dA = mk(), mk(), mk(), mk()
    qi = torch.arange(seq, device="cuda")[:, None]
    ki = torch.arange(seq, device="cuda")[None, :]
    keep = {"causal": ki <= qi, "band": (qi - ki).abs() <= 32,
            "none": torch.ones((seq, seq), dtype=torch.bool, device="cuda")}[kind]
    mask = torch.where(keep, 0.0, -math.inf).to(dtype)                # [q][k] row major
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    # the reference's execute_graph refuses the null stream for its add passes
    side = torch.cuda.Stream()
    out = {}
    for who in ("ref", "ours"):
        # two K/V "tiles" in a row: the second call merges into (lse, A) and adds into
        # the gradients, so the merge kernel and the += passes are exercised too
        lse = torch.full((batch, seq), -math.inf, dtype=torch.float32, device="cuda")
        A = torch.zeros_like(Q)
        s_l, s1, s2, s3 = torch.empty_like(lse), torch.empty_like(Q), torch.empty_like(Q), \
            torch.empty_like(Q)
        dK, dQ, dV = (torch.full_like(Q, 0.25) for _ in range(3))
        K2 = (K.float()*0.5).to(dtype)
        with torch.cuda.stream(side):
            side.wait_stream(torch.cuda.default_stream())
            sp = ctypes.c_void_p(side.cuda_stream)
            for kk in (K, K2):
                if who == "ref":
                    st = ref_fwd(sp, seq, head, batch, p(kk), p(Q), p(mask),
                                                        p(s_l), p(V), p(s1), p(lse), p(A))
                    if st == 2:
                        pytest.skip("cuDNN did not build the reference's forward graph here")
                    assert st == 0
                else:
                    ops.flash_sdpa_fwd(seq, head, batch, kk, Q, mask, s_l, V, s1, lse, A)
            side.synchronize()
            Afin, lfin = A.clone(), lse.clone()
            # backward of the FIRST tile against the merged A and lse, as the
            # reference's tensor loop calls it
            if who == "ref":
                st = ref_bwd(sp, seq, head, batch, p(K), p(Q), p(V), p(Afin),
                                                    p(dA), p(mask), p(lfin), p(s1), p(s2), p(s3),
                                                    p(dK), p(dQ), p(dV))
                if st == 2:
                    pytest.skip("cuDNN did not build the reference's backward graph here")
                assert st == 0
            else:
                ops.flash_sdpa_bwd(seq, head, batch, K, Q, V, Afin, dA, mask, lfin, s1, s2, s3,
                                   dK, dQ, dV)
            side.synchronize()
        out[who] = (Afin, lfin, dK, dQ, dV)
    rA, rl, rdK, rdQ, rdV = out["ref"]
    oA, ol, odK, odQ, odV = out["ours"]
    assert rel(oA, rA) <= 2e-2
    assert torch.allclose(ol, rl, rtol=1e-3, atol=1e-3)
    # the backward ran on each side's own (A, lse), which agree to 2e-2
    for name, a, b in (("dK", odK, rdK), ("dQ", odQ, rdQ), ("dV", odV, rdV)):
        assert rel(a - 0.25, b - 0.25) <= 3e-2, name
