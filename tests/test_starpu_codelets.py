"""The replacement StarPU codelets of nntile_b200/starpu/ (the reference's
src/starpu/flash_sdpa_{fwd,bwd}_cudnn.cc without cuDNN), compiled against the
reference's own Codelet / Handle classes and a one-worker stand-in for StarPU
(tests/starpu_fake/), and driven the way the reference's tile layer drives them.

CPU: the sources compile and link, the codelets carry the reference's names and
buffer counts, and a task reaches libnntile_b200.so (which rejects null buffers
before any launch).  GPU: a task submitted through the codelet gives bit-identical
results to the direct C-ABI call."""
import ctypes
import importlib.util
import os

import numpy as np
import pytest

from conftest import reference_root

HERE = os.path.dirname(os.path.abspath(__file__))


def _builder():
    spec = importlib.util.spec_from_file_location(
        "starpu_fake_build", os.path.join(HERE, "starpu_fake", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def chk():
    from nntile_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    path = _builder().build(reference_root())
    if path is None:
        pytest.skip("no reference checkout here and no prebuilt codelet check library")
    lib = ctypes.CDLL(path)
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    lib.codelet_check_fwd.argtypes = [vp, ctypes.c_int, i64, i64, i64] + [vp]*8
    lib.codelet_check_bwd.argtypes = [vp, ctypes.c_int, i64, i64, i64] + [vp]*13
    lib.codelet_check_footprint.argtypes = [ctypes.c_int, i64, i64, i64]
    lib.codelet_check_footprint.restype = ctypes.c_uint32
    lib.codelet_check_name.argtypes = [ctypes.c_int, ctypes.c_int]
    lib.codelet_check_name.restype = ctypes.c_char_p
    lib.starpu_fake_tasks_run.restype = ctypes.c_int
    return lib


def test_codelets_keep_the_reference_names_and_footprints(chk):
    # src/starpu/flash_sdpa_fwd_cudnn.cc:42 / flash_sdpa_bwd_cudnn.cc:37 + type postfix
    assert chk.codelet_check_name(1, 0) == b"nntile_flash_sdpa_fwd_cudnn_bf16"
    assert chk.codelet_check_name(0, 0) == b"nntile_flash_sdpa_bwd_cudnn_bf16"
    assert chk.codelet_check_name(1, 1) == b"nntile_flash_sdpa_fwd_cudnn_fp16"
    assert chk.codelet_check_name(0, 1) == b"nntile_flash_sdpa_bwd_cudnn_fp16"
    a = chk.codelet_check_footprint(1, 1024, 64, 96)
    assert a == chk.codelet_check_footprint(1, 1024, 64, 96)
    assert a != chk.codelet_check_footprint(1, 2048, 64, 96)
    assert a == chk.codelet_check_footprint(0, 1024, 64, 96)


def test_a_submitted_task_reaches_the_library(chk, capfd):
    """8 and 13 buffers as in the reference; with null device pointers the library
    refuses before any launch and the worker body reports it on stderr."""
    null = ctypes.c_void_p(0)
    before = chk.starpu_fake_tasks_run()
    for fp16 in (0, 1):
        assert chk.codelet_check_fwd(null, fp16, 128, 64, 1, *([null]*8)) == 8
        assert chk.codelet_check_bwd(null, fp16, 128, 64, 1, *([null]*13)) == 13
    assert chk.starpu_fake_tasks_run() == before + 4
    err = capfd.readouterr().err
    assert err.count("nntile_b200_flash_sdpa_fwd: bad argument") == 2
    assert err.count("nntile_b200_flash_sdpa_bwd: bad argument") == 2


@pytest.mark.gpu
@pytest.mark.parametrize("fp16", [0, 1])
def test_codelet_task_equals_direct_call(chk, fp16):
    import torch

    from nntile_b200 import ops
    torch.manual_seed(5)
    seq, head, batch = 256, 128, 3
    dt = torch.float16 if fp16 else torch.bfloat16
    mk = lambda: torch.randn((batch, seq, head), device="cuda").to(dt)
    Q, K, V, dA = mk(), mk(), mk(), mk()
    qi = torch.arange(seq, device="cuda")
    mask = torch.where(qi[None, :] > qi[:, None], float("-inf"), 0.0).to(dt)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    res = []
    for via_codelet in (False, True):
        lse = torch.full((batch, seq), -np.inf, dtype=torch.float32, device="cuda")
        A = torch.zeros_like(Q)
        s_lse, s1, s2, s3 = torch.empty_like(lse), torch.empty_like(Q), torch.empty_like(Q), \
            torch.empty_like(Q)
        dK, dQ, dV = (torch.zeros_like(Q) for _ in range(3))
        if via_codelet:
            assert chk.codelet_check_fwd(stream, fp16, seq, head, batch, p(K), p(Q), p(mask), p(lse),
                                         p(V), p(A), p(s_lse), p(s1)) == 8
            assert chk.codelet_check_bwd(stream, fp16, seq, head, batch, p(K), p(Q), p(V), p(A), p(dA),
                                         p(mask), p(lse), p(dK), p(dQ), p(dV), p(s1), p(s2),
                                         p(s3)) == 13
        else:
            ops.flash_sdpa_fwd(seq, head, batch, K, Q, mask, s_lse, V, s1, lse, A)
            ops.flash_sdpa_bwd(seq, head, batch, K, Q, V, A, dA, mask, lse, s1, s2, s3, dK, dQ,
                               dV)
        torch.cuda.synchronize()
        res.append((A, lse, dK, dQ, dV))
    assert float(res[0][0].float().abs().sum()) > 0
    for a, b in zip(*res):
        assert torch.equal(a, b)
