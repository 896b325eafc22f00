"""CPU checks of the boundary: the library builds for sm_100a, loads, and exports
every symbol include/nntile_b200.h declares (no compute call needs a GPU here)."""
import ctypes
import os
import re

import pytest

from nntile_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        build.build()
    return _lib.load()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nntile_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nntile_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    # and the Python binding knows the signature of each of them
    assert set(names) == set(_lib.SIGNATURES)


def test_version_and_status_strings(lib):
    assert lib.nntile_b200_version() >= 100
    assert lib.nntile_b200_status_string(0) == b"ok"
    assert b"scratch" in lib.nntile_b200_status_string(-4)


def test_argument_errors_are_reported_before_any_launch(lib):
    """Failure detection on the host: bad shapes / null pointers come back as
    negative statuses without touching a device (none exists here)."""
    null = ctypes.c_void_p(0)
    st = lib.nntile_b200_flash_sdpa_fwd_bf16(null, 128, 64, 1, null, null, null, null, null,
                                             null, null, null)
    assert st == -1
    st = lib.nntile_b200_flash_sdpa_fwd_bf16(null, 128, 512, 1, null, null, null, null, null,
                                             null, null, null)
    assert st == -2
    assert lib.nntile_b200_flash_sdpa_fwd_bf16(null, 0, 64, 1, *([null]*8)) == 0
    assert lib.nntile_b200_maxsumexp_fp32(null, -1, 1, 1, null, null) == -1
    assert lib.nntile_b200_decode_sdpa_bf16(null, 128, 16, 32, 1, 1, 1, *([null]*6), 0) == -1
    assert lib.nntile_b200_decode_sdpa_bf16(null, 128, 16, 0, 1, 1, 1, *([null]*6), 0) == -2
    assert lib.nntile_b200_decode_sdpa_workspace_bytes(128, 8192, 64, 4, 8) > 0


def test_path_selection(lib):
    # the reference's own kernel-test shapes go to the generic kernels
    assert lib.nntile_b200_flash_sdpa_fwd_path(16, 32, 1) == 1
    assert lib.nntile_b200_flash_sdpa_bwd_path(64, 8, 4) == 1
    assert lib.nntile_b200_flash_sdpa_fwd_path(64, 512, 1) == 0
    assert lib.nntile_b200_flash_sdpa_bwd_path(64, 1, 1) == 0


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libnntile_b200.so")
    with pytest.raises(_lib.LibraryMissing):
        _lib.load()


def test_cpp_shims_compile_and_reach_the_library(lib, tmp_path):
    """include/nntile_b200/kernel_shims.hh re-creates nntile::kernel::<op>::cuda<T>;
    tests/shim_check.cc instantiates every shim and calls it with null pointers,
    which the library rejects before any launch (no GPU needed)."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "shim_check")
    libdir = os.path.dirname(_lib.LIB_PATH)
    subprocess.run(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-o", exe,
                    os.path.join(ROOT, "tests", "shim_check.cc"), _lib.LIB_PATH,
                    "-Wl,-rpath," + libdir], check=True)
    assert subprocess.run([exe]).returncode == 0


def test_per_device_bookkeeping(tmp_path):
    """The shared-memory opt-in of the fused kernels, the helper streams and the
    no-allocation scratch address are set up once PER DEVICE (one process may drive
    several GPUs); the bookkeeping class is plain C++ and is checked here."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "per_device_check")
    subprocess.run(["g++", "-std=c++17", "-o", exe,
                    os.path.join(ROOT, "tests", "per_device_check.cc")], check=True)
    assert subprocess.run([exe]).returncode == 0


def test_new_entry_points_check_their_arguments(lib):
    null = ctypes.c_void_p(0)
    # GEMM: null handle / buffers, negative size
    assert lib.nntile_b200_gemm_fp32(null, 1, 0, 4, 4, 4, 1, 1.0, null, null, 0.0, null) == -1
    assert lib.nntile_b200_gemm_bf16(null, 0, 0, -1, 4, 4, 1, 1.0, null, null, 0.0, null) == -1
    assert lib.nntile_b200_gemm_bf16(null, 0, 0, 0, 4, 4, 1, 1.0, null, null, 0.0, null) == 0
    # layout changes: odd lead / head are rejected, empty problems are fine
    assert lib.nntile_b200_transpose_rope_bf16(null, 7, 64, 4, 1, null, null, null, null) == -2
    assert lib.nntile_b200_transpose_rope_bf16(null, 8, 64, 0, 1, null, null, null, null) == 0
    assert lib.nntile_b200_transpose_rope_bf16(null, 8, 64, 4, 1, null, null, null, null) == -1
    assert lib.nntile_b200_transpose_bias_bf16(null, 12, 64, 4, 1, null, null, null) == -1
    assert lib.nntile_b200_transpose_heads_back_bf16(null, 12, 63, 4, 1, null, null) == -2
    # status reader
    assert lib.nntile_b200_flash_sdpa_read_status(null, null, None) == -1
    # tensor level: scratch size grows with the tensor, not only with the tile
    i64 = ctypes.c_int64
    base = (i64*5)(128, 2048, 1, 1, 16)
    small = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes((i64*5)(128, 2048, 1, 1, 16), base)
    big = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes((i64*5)(128, 16384, 1, 1, 16), base)
    assert 0 < small < big
    assert lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(None, base) == 0
