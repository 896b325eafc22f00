"""Compile the CUDA library in-tree for sm_100a.

    python -m nntile_b200.build [--force]

One nvcc invocation per source (object files are cached under csrc/build/), then
one link step into ``csrc/libnntile_b200.so``.  nvcc cross-compiles without a
GPU.  The library has no link-time dependency beyond the CUDA runtime (linked
statically): the driver entry point needed for TMA descriptors and the cuBLAS
routine behind the GEMM entry points are looked up at run time.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(CSRC, "build")
LIB = os.path.join(CSRC, "libnntile_b200.so")
SOURCES = [
    "vanilla_ops.cu", "flash_generic.cu", "flash_api.cu", "decode.cu",
    "flash_fwd_sm100.cu", "flash_bwd_sm100.cu", "host_tensor.cu", "gemm_cublas.cu",
    "sdpa_prologue.cu",
]
# the fused-attention sources are compiled a second time for IEEE half (elem.cuh)
FP16_SOURCES = [
    "flash_generic.cu", "flash_api.cu", "flash_fwd_sm100.cu", "flash_bwd_sm100.cu",
    "host_tensor.cu",
]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _deps(src: str) -> list[str]:
    deps = [os.path.join(CSRC, src)]
    deps += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".hh"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "nntile_b200.h"))
    return deps


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(job, force: bool) -> str:
    src, fp16 = job
    obj = os.path.join(OBJ_DIR, src.replace(".cu", "_fp16.o" if fp16 else ".o"))
    if force or _stale(obj, _deps(src)):
        log = obj + ".log"
        cmd = [_nvcc()] + NVCC_FLAGS + (["-DNB200_FP16"] if fp16 else []) \
            + ["-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}{res.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs = [(s, False) for s in SOURCES] + [(s, True) for s in FP16_SOURCES]
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
        objs = list(ex.map(lambda j: _compile(j, force), jobs))
    if force or _stale(LIB, objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode",
               "arch=compute_100a,code=sm_100a", "-ldl"]
        subprocess.run(cmd, check=True)
    if verbose:
        for o in objs:
            with open(o + ".log") as f:
                for line in f:
                    if "registers" in line or "spill" in line or "Compiling entry" in line:
                        print(line.rstrip())
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args(argv)
    print(build(a.force, a.verbose))
    return 0


if __name__ == "__main__":
    sys.exit(main())
