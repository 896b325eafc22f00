"""GPU parity of the fused layout-change kernels around the SDPA layer
(nntile_b200_transpose_rope_bf16, _transpose_bias_bf16, _transpose_heads_back_bf16)
through the C ABI: bit for bit against the outputs of the reference's own
transpose / rope / add_fiber_inplace CPU kernels (tests/golden/ref_around.npz) and
against the oracle on fresh, larger inputs."""
import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import from_fortran, to_fortran

pytestmark = pytest.mark.gpu


def run_in(proj, sin=None, cos=None, bias=None):
    lead, head, seq, batch = proj.shape
    src = from_fortran(proj)
    dst = torch.full((lead, batch, seq, head), float("nan"), dtype=torch.bfloat16, device="cuda")
    if bias is not None:
        ops.transpose_bias(lead, head, seq, batch, from_fortran(bias), src, dst)
    else:
        ops.transpose_rope(lead, head, seq, batch,
                           None if sin is None else from_fortran(sin),
                           None if cos is None else from_fortran(cos), src, dst)
    torch.cuda.synchronize()
    assert np.array_equal(to_fortran(src), proj)            # input untouched
    return to_fortran(dst)


def run_back(attn):
    head, seq, batch, lead = attn.shape
    dst = torch.full((batch, seq, head, lead), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.transpose_heads_back(lead, head, seq, batch, from_fortran(attn), dst)
    torch.cuda.synchronize()
    return to_fortran(dst)


@pytest.mark.parametrize("tag", ["llama_q", "llama_k", "gpt2"])
def test_against_reference_kernel_outputs(golden, tag):
    g = golden("ref_around.npz")
    proj, sin, cos, bias = (g[f"{tag}_{k}"] for k in ("proj", "sin", "cos", "bias"))
    assert np.array_equal(run_in(proj, sin, cos), g[f"{tag}_rope"])
    assert np.array_equal(run_in(proj), g[f"{tag}_plain"])
    assert np.array_equal(run_in(proj, bias=bias), g[f"{tag}_biased"])
    assert np.array_equal(run_back(g[f"{tag}_rope"]), g[f"{tag}_back"])


@pytest.mark.parametrize("lead,head,seq,batch", [
    (32, 128, 257, 2),       # config 3's Q layout: 32 query heads, ragged position count
    (8, 128, 512, 3),        # its K layout
    (12, 64, 1024, 1),       # config 2: 12 heads (rows are not whole 16-byte pieces)
    (2, 96, 33, 5),          # odd sizes: head/2 not a power of two
    (64, 256, 9, 1),         # one position needs more than the default chunk
    (24, 64, 130, 2),        # a multiple of 8 that is not a power of two (three column blocks)
])
def test_against_oracle_on_fresh_inputs(lead, head, seq, batch):
    rng = np.random.default_rng(lead*1000 + head + seq)
    proj = O.to_bf16(np.asfortranarray(
        rng.standard_normal((lead, head, seq, batch)).astype(np.float32)))
    pos = rng.integers(0, 4096, size=(batch, seq))
    sin, cos = (O.to_bf16(x) for x in O.rope_sin_cos(head, pos))
    bias = O.to_bf16(np.asfortranarray(rng.standard_normal((head, lead)).astype(np.float32)))
    be = "ref" if O.have_ref() else "port"
    want = O.attention_prologue(proj, sin, cos, backend=be)
    assert np.array_equal(run_in(proj, sin, cos), want)
    assert np.array_equal(run_in(proj, bias=bias), O.attention_prologue(proj, bias=bias, backend=be))
    plain = run_in(proj)
    assert np.array_equal(plain, O.attention_prologue(proj, backend=be))
    # round trip: back(in(x)) == x
    assert np.array_equal(run_back(plain), proj)


def test_rejects_what_it_cannot_take():
    from nntile_b200 import _lib
    t = torch.zeros(7*64*4, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.StatusError):
        ops.transpose_rope(7, 64, 4, 1, None, None, t, t.clone())       # odd lead
    with pytest.raises(_lib.StatusError):
        ops.transpose_rope(8, 64, 4, 1, t, None, t, t.clone())          # sin without cos
