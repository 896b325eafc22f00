"""Build recipe for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Two targets, both plain compiler invocations (the reference's own build system
is never run):

``port``  oracle/sdpa_oracle.c -> oracle/libsdpa_oracle.so
          The C restatement of the path's arithmetic.  Always buildable.

``_ref``  the reference's own CPU kernels, compiled from the files where they
          lie in the reference checkout (nothing is copied into this repo), plus
          oracle/ref_shim.cc -> oracle/_ref/libnntile_ref_cpu.so.  Only when the
          reference checkout is present; the built file travels with the repo.

``_ref_gpu``  the reference's own GPU wrappers of the fused pair (cuDNN graphs +
          merge / add_inplace kernels), compiled in place the same way, plus
          oracle/ref_gpu_shim.cc -> oracle/_ref_gpu/libnntile_ref_gpu.so: the
          second parity witness and the timing comparator on a GPU box.

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
REF_GPU_DIR = os.path.join(HERE, "_ref_gpu")
REF_GPU_SO = os.path.join(REF_GPU_DIR, "libnntile_ref_gpu.so")


def default_ref_root() -> str | None:
    """Where the reference checkout is: the NNTILE_REFERENCE_ROOT variable, else a
    directory named ``reference`` beside this repository, else nowhere."""
    env = os.environ.get("NNTILE_REFERENCE_ROOT")
    if env:
        return env
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return beside if os.path.isdir(os.path.join(beside, "src", "kernel")) else None


# Reference kernels on the path (relative to the reference root).
REF_OPS = [
    "maxsumexp", "softmax_inplace", "sumprod_slice", "mask_scalar",
    "add_slice_inplace", "multiply_inplace", "add_inplace",
    "accumulate_attn_output", "rope", "transpose", "add_fiber_inplace",
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


def build_ref(ref_root: str | None = None, force: bool = False) -> str | None:
    """Compile the reference's CPU kernels in place; None if not possible."""
    ref_root = ref_root or default_ref_root()
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "src", "kernel")):
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


def _site_packages() -> str | None:
    try:
        import nvidia.cudnn as cudnn_pkg
    except ImportError:
        return None
    paths = list(getattr(cudnn_pkg, "__path__", []))      # a namespace package has no __file__
    return os.path.dirname(os.path.dirname(paths[0])) if paths else None


def build_ref_gpu(ref_root: str | None = None, force: bool = False) -> str | None:
    """Compile the reference's GPU wrappers of the fused pair in place
    (src/kernel/flash_sdpa_{fwd,bwd}_cudnn/cuda.cc, accumulate_attn_output/cuda.cu,
    add_inplace/cuda.cu) against the cuDNN and cudnn_frontend that ship with the
    Python environment; None if that is not possible here.  The reference pins
    cudnn_frontend v1.11.0 (external/cudnn_frontend/CMakeLists.txt:2-9); whatever
    version the environment holds is used."""
    ref_root = ref_root or default_ref_root()
    site = _site_packages()
    if not ref_root or not site or not os.path.isdir(os.path.join(ref_root, "src", "kernel")):
        return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
    fe_inc = os.path.join(site, "include")
    cudnn_inc = os.path.join(site, "nvidia", "cudnn", "include")
    cudnn_lib = os.path.join(site, "nvidia", "cudnn", "lib")
    if not os.path.exists(os.path.join(fe_inc, "cudnn_frontend.h")) \
            or not os.path.exists(os.path.join(cudnn_lib, "libcudnn.so.9")):
        return REF_GPU_SO if os.path.exists(REF_GPU_SO) else None
    k = os.path.join(ref_root, "src", "kernel")
    srcs = [os.path.join(k, "flash_sdpa_fwd_cudnn", "cuda.cc"),
            os.path.join(k, "flash_sdpa_bwd_cudnn", "cuda.cc"),
            os.path.join(k, "accumulate_attn_output", "cuda.cu"),
            os.path.join(k, "add_inplace", "cuda.cu"),
            os.path.join(HERE, "ref_gpu_shim.cc")]
    if not force and _newer(REF_GPU_SO, srcs):
        return REF_GPU_SO
    os.makedirs(REF_GPU_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-shared", "-O2", "-std=c++17", "-x", "cu",
           "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
           "-DNNTILE_USE_CUDA", "-I", os.path.join(HERE, "shim"),
           "-I", os.path.join(ref_root, "include"), "-I", fe_inc, "-I", cudnn_inc,
           "-o", REF_GPU_SO] + srcs + [
           "-L", cudnn_lib, "-l:libcudnn.so.9", "-Xlinker", "-rpath=" + cudnn_lib]
    subprocess.run(cmd, check=True)
    return REF_GPU_SO


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--ref-root", default=None,
                    help="reference checkout (default: $NNTILE_REFERENCE_ROOT, else a "
                         "directory named 'reference' beside this repository)")
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args(argv)
    print("port:", build_port(args.force))
    print("_ref:", build_ref(args.ref_root, args.force))
    try:
        print("_ref_gpu:", build_ref_gpu(args.ref_root, args.force))
    except subprocess.CalledProcessError as exc:
        print("_ref_gpu: not built:", exc)
    return 0


if __name__ == "__main__":
    sys.exit(main())
