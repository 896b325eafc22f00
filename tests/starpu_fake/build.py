"""Build tests/starpu_fake/_build/libcodelet_check.so.  TEST INFRASTRUCTURE ONLY.

Compiles, with plain g++: the two replacement codelet sources of
nntile_b200/starpu/, the reference's own src/starpu/{codelet,handle}.cc where
they lie in the reference checkout (nothing is copied), the fake runtime and
the C doors of this folder - against the reference's own headers plus ./starpu.h
- and links libnntile_b200.so.  Needs the reference checkout; the built file
travels with the repository.

    python tests/starpu_fake/build.py --ref-root DIR
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libcodelet_check.so")


def build(ref_root: str | None, force: bool = False) -> str | None:
    """Returns the library path, or None when it cannot be (re)built and no
    earlier build exists."""
    lib = os.path.join(ROOT, "nntile_b200", "csrc", "libnntile_b200.so")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "src", "starpu")) \
            or not os.path.exists(lib):
        return OUT if os.path.exists(OUT) else None
    mine = os.path.join(ROOT, "nntile_b200", "starpu")
    srcs = [os.path.join(mine, "flash_sdpa_fwd_cudnn.cc"),
            os.path.join(mine, "flash_sdpa_bwd_cudnn.cc"),
            os.path.join(ref_root, "src", "starpu", "codelet.cc"),
            os.path.join(ref_root, "src", "starpu", "handle.cc"),
            os.path.join(HERE, "starpu_fake.cc"), os.path.join(HERE, "codelet_check.cc")]
    deps = srcs + [os.path.join(HERE, "starpu.h"), lib,
                   os.path.join(mine, "flash_sdpa_fwd_cudnn.hh"),
                   os.path.join(mine, "flash_sdpa_bwd_cudnn.hh")]
    if not force and os.path.exists(OUT) and all(
            os.path.getmtime(d) <= os.path.getmtime(OUT) for d in deps):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    with tempfile.TemporaryDirectory() as tmp:
        # the replacement headers take the place of the reference's two: give them
        # the path the sources include them by, ahead of the reference's include/
        over = os.path.join(tmp, "nntile", "starpu")
        os.makedirs(over)
        for h in ("flash_sdpa_fwd_cudnn.hh", "flash_sdpa_bwd_cudnn.hh"):
            shutil.copy(os.path.join(mine, h), os.path.join(over, h))
        cmd = ["g++", "-O1", "-fPIC", "-shared", "-std=c++17", "-DNNTILE_USE_CUDA",
               "-I", tmp, "-I", HERE, "-I", os.path.join(ROOT, "include"),
               "-I", os.path.join(ROOT, "oracle", "shim"),      # nntile/defs.h
               "-I", os.path.join(ref_root, "include"), "-I", cuda_inc,
               "-o", OUT] + srcs + [lib, "-Wl,-rpath," + os.path.dirname(lib)]
        subprocess.run(cmd, check=True)
    return OUT


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ref-root", default=os.environ.get("NNTILE_REFERENCE_ROOT"))
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print(build(a.ref_root, a.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
