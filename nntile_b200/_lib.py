"""ctypes binding of libnntile_b200.so (the C ABI of include/nntile_b200.h)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libnntile_b200.so")

i64, f32, vp, sz = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
_pp = ctypes.POINTER(ctypes.c_void_p)
_pi = ctypes.POINTER(ctypes.c_int64)

_TYPED = {
    "mask_scalar": [vp, i64, i64, vp, f32, vp],
    "maxsumexp": [vp, i64, i64, i64, vp, vp],
    "softmax_inplace": [vp, i64, i64, i64, vp, f32, vp],
    "sumprod_slice": [vp, i64, i64, i64, f32, vp, vp, f32, vp],
    "add_slice_inplace": [vp, i64, i64, i64, f32, vp, f32, vp],
    "multiply_inplace": [vp, i64, f32, vp, vp],
    "add_inplace": [vp, i64, f32, vp, f32, vp],
    "accumulate_attn_output": [vp, i64, i64, i64, vp, vp, vp, vp],
}

# every symbol include/nntile_b200.h declares -> (argtypes, restype)
SIGNATURES = {
    "nntile_b200_version": ([], ctypes.c_int),
    "nntile_b200_status_string": ([ctypes.c_int], ctypes.c_char_p),
    "nntile_b200_launch_count": ([], ctypes.c_ulonglong),
    "nntile_b200_fill_fp32": ([vp, i64, f32, vp], ctypes.c_int),
    "nntile_b200_clear": ([vp, i64, vp], ctypes.c_int),
    "nntile_b200_flash_sdpa_fwd_bf16": ([vp, i64, i64, i64] + [vp]*8, ctypes.c_int),
    "nntile_b200_flash_sdpa_bwd_bf16": ([vp, i64, i64, i64] + [vp]*13, ctypes.c_int),
    "nntile_b200_flash_sdpa_fwd_path": ([i64, i64, i64], ctypes.c_int),
    "nntile_b200_flash_sdpa_bwd_path": ([i64, i64, i64], ctypes.c_int),
    "nntile_b200_flash_sdpa_fwd_gqa_bf16": ([vp] + [i64]*5 + [vp]*7 + [sz], ctypes.c_int),
    "nntile_b200_flash_sdpa_bwd_gqa_bf16": ([vp] + [i64]*5 + [vp]*11 + [sz], ctypes.c_int),
    "nntile_b200_flash_sdpa_gqa_scratch_bytes": ([i64]*5, sz),
    "nntile_b200_decode_sdpa_bf16": ([vp] + [i64]*6 + [vp]*6 + [sz], ctypes.c_int),
    "nntile_b200_decode_sdpa_workspace_bytes": ([i64]*5, sz),
    "nntile_b200_kv_cache_append_bf16": ([vp] + [i64]*6 + [vp]*2, ctypes.c_int),
    "nntile_b200_decode_sdpa_noalloc_bf16": ([vp] + [i64]*6 + [vp]*5, ctypes.c_int),
    "nntile_b200_decode_sdpa_noalloc_max_bytes": ([], sz),
    "nntile_b200_tensor_flash_sdpa_fwd_bf16": ([vp, _pi, _pi] + [_pp]*6 + [vp, sz], ctypes.c_int),
    "nntile_b200_tensor_flash_sdpa_bwd_bf16": ([vp, _pi, _pi] + [_pp]*10 + [vp, sz], ctypes.c_int),
    "nntile_b200_tensor_flash_sdpa_scratch_bytes": ([_pi, _pi], sz),
    "nntile_b200_tensor_flash_sdpa_fwd_gqa_bf16": ([vp, _pi, _pi] + [_pp]*6 + [vp, sz], ctypes.c_int),
    "nntile_b200_tensor_flash_sdpa_bwd_gqa_bf16": ([vp, _pi, _pi] + [_pp]*10 + [vp, sz], ctypes.c_int),
    "nntile_b200_gemm_fp32": ([vp, ctypes.c_int, ctypes.c_int] + [i64]*4 + [f32, vp, vp, f32, vp],
                              ctypes.c_int),
    "nntile_b200_gemm_bf16": ([vp, ctypes.c_int, ctypes.c_int] + [i64]*4 + [f32, vp, vp, f32, vp],
                              ctypes.c_int),
    "nntile_b200_flash_sdpa_read_status": ([vp, vp, ctypes.POINTER(ctypes.c_uint)], ctypes.c_int),
    "nntile_b200_test_arm_wait_timeout": ([], None),
    "nntile_b200_transpose_rope_bf16": ([vp] + [i64]*4 + [vp]*4, ctypes.c_int),
    "nntile_b200_transpose_bias_bf16": ([vp] + [i64]*4 + [vp]*3, ctypes.c_int),
    "nntile_b200_transpose_heads_back_bf16": ([vp] + [i64]*4 + [vp]*2, ctypes.c_int),
}
for _name in ("flash_sdpa_fwd", "flash_sdpa_bwd", "flash_sdpa_fwd_gqa", "flash_sdpa_bwd_gqa",
              "tensor_flash_sdpa_fwd", "tensor_flash_sdpa_bwd", "tensor_flash_sdpa_fwd_gqa",
              "tensor_flash_sdpa_bwd_gqa"):
    SIGNATURES[f"nntile_b200_{_name}_fp16"] = SIGNATURES[f"nntile_b200_{_name}_bf16"]
for _name, _args in _TYPED.items():
    for _sfx in ("fp32", "bf16"):
        SIGNATURES[f"nntile_b200_{_name}_{_sfx}"] = (_args, ctypes.c_int)


class LibraryMissing(RuntimeError):
    pass


_lib = None


def load() -> ctypes.CDLL:
    """Load the CUDA library; raise (never fall back) when it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} not found: build it with `python -m nntile_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (args, res) in SIGNATURES.items():
            fn = getattr(lib, name)       # AttributeError if the ABI is incomplete
            fn.argtypes = args
            fn.restype = res
        _lib = lib
    return _lib


class StatusError(RuntimeError):
    def __init__(self, fn: str, status: int):
        self.status = status
        text = load().nntile_b200_status_string(status).decode()
        super().__init__(f"{fn} returned {status} ({text})")


def check(fn: str, status: int) -> None:
    if status != 0:
        raise StatusError(fn, status)
