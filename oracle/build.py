"""Build recipe for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two targets, both plain compiler invocations (the reference's own build system
is never run):

``port``  oracle/sdpa_oracle.c -> oracle/libsdpa_oracle.so
          The C restatement of the path's arithmetic.  Always buildable.

``_ref``  the reference's own CPU kernels, compiled from the files where they
          lie in the reference checkout (nothing is copied into this repo), plus
          oracle/ref_shim.cc -> oracle/_ref/libnntile_ref_cpu.so.  Only when the
          reference checkout is present; the built file travels with the repo.

Run ``python oracle/build.py [--ref-root DIR]``.
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "libsdpa_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libnntile_ref_cpu.so")
DEFAULT_REF_ROOT = os.environ.get("NNTILE_REFERENCE_ROOT", "/root/reference")

# Reference kernels on the path (relative to the reference root).
REF_OPS = [
    "maxsumexp", "softmax_inplace", "sumprod_slice", "mask_scalar",
    "add_slice_inplace", "multiply_inplace", "add_inplace",
    "accumulate_attn_output",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def find_openblas() -> str | None:
    """SciPy's bundled OpenBLAS (exports scipy_cblas_sgemm)."""
    try:
        import scipy
    except ImportError:
        return None
    root = os.path.join(os.path.dirname(os.path.dirname(scipy.__file__)),
                        "scipy.libs")
    hits = sorted(glob.glob(os.path.join(root, "libscipy_openblas*.so")))
    return hits[0] if hits else None


def build_port(force: bool = False) -> str:
    srcs = [os.path.join(HERE, "sdpa_oracle.c"),
            os.path.join(HERE, "ops_impl.inc")]
    if not force and _newer(PORT_SO, srcs):
        return PORT_SO
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-o", PORT_SO,
           srcs[0], "-lm"]
    subprocess.run(cmd, check=True)
    return PORT_SO


def build_ref(ref_root: str = DEFAULT_REF_ROOT, force: bool = False) -> str | None:
    """Compile the reference's CPU kernels in place; None if not possible."""
    if not os.path.isdir(os.path.join(ref_root, "src", "kernel")):
        return REF_SO if os.path.exists(REF_SO) else None
    blas = find_openblas()
    if blas is None:
        return REF_SO if os.path.exists(REF_SO) else None
    srcs = [os.path.join(ref_root, "src", "kernel", op, "cpu.cc")
            for op in REF_OPS]
    srcs.append(os.path.join(ref_root, "src", "kernel", "cblas.cc"))
    srcs.append(os.path.join(HERE, "ref_shim.cc"))
    if not force and _newer(REF_SO, srcs):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"),
                            "include")
    cmd = ["g++", "-O2", "-fPIC", "-shared", "-std=c++17",
           # bf16 stores round to nearest even, as in the reference's CUDA build
           "-DNNTILE_USE_CUDA", "-I", cuda_inc,
           "-I", os.path.join(HERE, "shim"),
           "-I", os.path.join(ref_root, "include"),
           "-o", REF_SO] + srcs + [
           blas, "-Wl,-rpath," + os.path.dirname(blas)]
    subprocess.run(cmd, check=True)
    return REF_SO


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ref-root", default=DEFAULT_REF_ROOT)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    print("port:", build_port(args.force))
    print("_ref:", build_ref(args.ref_root, args.force))
    return 0


if __name__ == "__main__":
    sys.exit(main())
