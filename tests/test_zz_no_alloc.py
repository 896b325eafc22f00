"""The decode entry point that brings its own workspace.

Some hosts of the library cannot allocate device memory where they call it (a
task-runtime worker callback such as a StarPU codelet body, or a C host that was
only ever given device pointers), so `nntile_b200_decode_sdpa_noalloc_bf16` uses a
fixed array inside the library instead of a caller-provided workspace.  This test
drives it through the C ABI exactly as such a host would - raw pointers, no
workspace argument - and requires the same output as the ordinary entry point,
on two calls in a row (the array is shared and keeps the previous call's
contents, which must not leak into the next result).

The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from nntile_b200 import _lib

pytestmark = pytest.mark.gpu


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _run_both(lib, D, L, length, B, G, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((H, G, B, 1, D), generator=g, device="cuda").to(torch.bfloat16)
    Kc = torch.randn((H, B, L, D), generator=g, device="cuda").to(torch.bfloat16)
    Vc = torch.randn((H, B, L, D), generator=g, device="cuda").to(torch.bfloat16)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # ordinary entry point, caller-provided workspace
    nbytes = lib.nntile_b200_decode_sdpa_workspace_bytes(D, length, B, G, H)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ref_out = torch.empty_like(q)
    ref_lse = torch.empty((H, G, B), dtype=torch.float32, device="cuda")
    st = lib.nntile_b200_decode_sdpa_bf16(stream, D, L, length, B, G, H, _vp(q), _vp(Kc),
                                          _vp(Vc), _vp(ref_out), _vp(ref_lse), _vp(ws), nbytes)
    assert st == 0
    # the entry point under test: no workspace, nothing allocated by the call
    out = torch.full_like(q, float("nan"))
    lse = torch.full_like(ref_lse, float("nan"))
    st = lib.nntile_b200_decode_sdpa_noalloc_bf16(stream, D, L, length, B, G, H, _vp(q),
                                                  _vp(Kc), _vp(Vc), _vp(out), _vp(lse))
    assert st == 0
    torch.cuda.synchronize()
    return out, lse, ref_out, ref_lse


def test_noalloc_decode_matches_the_workspace_entry_point_twice_in_a_row():
    lib = _lib.load()
    assert lib.nntile_b200_decode_sdpa_noalloc_max_bytes() == 32 << 20
    # first call: several chunks, GQA group 4; second call: a different, smaller
    # problem that reuses the front of the array the first call filled
    for D, L, length, B, G, H, seed in ((128, 2048, 2048, 3, 4, 2, 11),
                                        (64, 1024, 700, 2, 8, 1, 12)):
        out, lse, ref_out, ref_lse = _run_both(lib, D, L, length, B, G, H, seed)
        # the tolerance of the decode tests (2e-2 relative, bf16 storage) ...
        a, b = out.float().cpu().numpy(), ref_out.float().cpu().numpy()
        assert np.isfinite(a).all()
        assert np.linalg.norm(a - b) <= 2e-2*np.linalg.norm(b)
        assert np.allclose(lse.cpu().numpy(), ref_lse.cpu().numpy(), rtol=1e-3, atol=1e-3)
        # ... and, tighter: same kernels, same chunking, same arithmetic, so the two
        # entry points agree bit for bit - one stale slot of the shared array would show
        assert torch.equal(out, ref_out)
        assert torch.equal(lse, ref_lse)


def test_noalloc_decode_rejects_what_does_not_fit():
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    # 4096 x 64 query heads need 135 MB of chunk results, more than the 32 MiB array
    D, L, B, G, H = 128, 1024, 4096, 8, 8
    assert lib.nntile_b200_decode_sdpa_workspace_bytes(D, L, B, G, H) > (32 << 20)
    st = lib.nntile_b200_decode_sdpa_noalloc_bf16(null, D, L, L, B, G, H, null, null, null,
                                                  null, null)
    assert st == -4
