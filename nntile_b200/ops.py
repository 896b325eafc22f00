"""Kernel-level operations on torch CUDA tensors.

Each function mirrors one ``nntile::kernel::<op>::cuda<T>`` entry point of the
reference (same name, same argument order, sizes first) and only enqueues work
on the current torch stream.  Tensors are raw buffers: what matters is their
memory, which must hold the Fortran-order array the sizes describe (a Fortran
array of shape [a, b, c] is a contiguous torch tensor of shape (c, b, a)).
dtype float32 selects the fp32 kernels, bfloat16 the bf16 ones.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    if t is None:
        return ctypes.c_void_p(0)
    if not t.is_cuda:
        raise ValueError("nntile_b200 ops need CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("nntile_b200 ops need contiguous buffers")
    return ctypes.c_void_p(t.data_ptr())


def _sfx(t) -> str:
    if t.dtype == torch.float32:
        return "fp32"
    if t.dtype == torch.bfloat16:
        return "bf16"
    raise TypeError(f"unsupported dtype {t.dtype}")


def _sfx16(t) -> str:
    """Suffix of the fused-pair entry points: bfloat16 or IEEE half."""
    if t.dtype == torch.bfloat16:
        return "bf16"
    if t.dtype == torch.float16:
        return "fp16"
    raise TypeError(f"the fused path takes bfloat16 or float16, not {t.dtype}")


def _call(name, *args):
    fn = getattr(_lib.load(), name)
    _lib.check(name, fn(*args))


def mask_scalar(nrows, ncols, mask, val, data):
    """mask: uint8/bool buffer of nrows entries (true = keep)."""
    if mask.dtype == torch.bool:
        mask = mask.view(torch.uint8)
    _call(f"nntile_b200_mask_scalar_{_sfx(data)}", _stream(), nrows, ncols, _ptr(mask),
          float(val), _ptr(data))


def maxsumexp(m, n, k, src, maxsumexp_):
    _call(f"nntile_b200_maxsumexp_{_sfx(src)}", _stream(), m, n, k, _ptr(src), _ptr(maxsumexp_))


def softmax_inplace(m, n, k, maxsumexp_, alpha, dst):
    _call(f"nntile_b200_softmax_inplace_{_sfx(dst)}", _stream(), m, n, k, _ptr(maxsumexp_),
          float(alpha), _ptr(dst))


def sumprod_slice(m, n, k, alpha, src1, src2, beta, dst):
    _call(f"nntile_b200_sumprod_slice_{_sfx(dst)}", _stream(), m, n, k, float(alpha),
          _ptr(src1), _ptr(src2), float(beta), _ptr(dst))


def add_slice_inplace(m, n, k, alpha, src, beta, dst):
    _call(f"nntile_b200_add_slice_inplace_{_sfx(dst)}", _stream(), m, n, k, float(alpha),
          _ptr(src), float(beta), _ptr(dst))


def multiply_inplace(nelems, alpha, src, dst):
    _call(f"nntile_b200_multiply_inplace_{_sfx(dst)}", _stream(), nelems, float(alpha),
          _ptr(src), _ptr(dst))


def add_inplace(nelems, alpha, src, beta, dst):
    _call(f"nntile_b200_add_inplace_{_sfx(dst)}", _stream(), nelems, float(alpha), _ptr(src),
          float(beta), _ptr(dst))


def fill(val, dst):
    _call("nntile_b200_fill_fp32", _stream(), dst.numel(), float(val), _ptr(dst))


def clear(dst):
    _call("nntile_b200_clear", _stream(), dst.numel()*dst.element_size(), _ptr(dst))


def accumulate_attn_output(head, seq, batch, src_lse, src_attn, dst_lse, dst_attn):
    _call(f"nntile_b200_accumulate_attn_output_{_sfx(dst_attn)}", _stream(), head, seq, batch,
          _ptr(src_lse), _ptr(src_attn), _ptr(dst_lse), _ptr(dst_attn))


def gemm(transA, transB, m, n, k, batch, alpha, A, B, beta, C):
    """Batched column-major C = alpha*op(A)*op(B) + beta*C with packed leading
    dimensions - the contract and argument order of nntile::kernel::cublas::gemm<T>
    (src/kernel/cublas.cc:35-164), through the C ABI.  A library GEMM in the
    reference and here (cublasGemmStridedBatchedEx, fp32 compute, no TF32); the
    handle is torch's cuBLAS handle for the current stream, the stand-in for the
    StarPU worker's handle."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False     # the handle's math mode follows this
    try:
        handle = torch.cuda.current_blas_handle()
        _call(f"nntile_b200_gemm_{_sfx(C)}", ctypes.c_void_p(handle), int(bool(transA)),
              int(bool(transB)), m, n, k, batch, float(alpha), _ptr(A), _ptr(B), float(beta),
              _ptr(C))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def transpose_rope(lead, head, seq, batch, sin, cos, src, dst):
    """dst[head, seq, batch, lead] = RoPE(src[lead, head, seq, batch]); sin = cos = None
    changes the layout only."""
    _call("nntile_b200_transpose_rope_bf16", _stream(), lead, head, seq, batch, _ptr(sin),
          _ptr(cos), _ptr(src), _ptr(dst))


def transpose_bias(lead, head, seq, batch, bias, src, dst):
    """dst[head, seq, batch, lead] = src[lead, head, seq, batch] + bias[head, lead]."""
    _call("nntile_b200_transpose_bias_bf16", _stream(), lead, head, seq, batch, _ptr(bias),
          _ptr(src), _ptr(dst))


def transpose_heads_back(lead, head, seq, batch, src, dst):
    """dst[lead, head, seq, batch] = src[head, seq, batch, lead]."""
    _call("nntile_b200_transpose_heads_back_bf16", _stream(), lead, head, seq, batch,
          _ptr(src), _ptr(dst))


def flash_sdpa_read_status(scratch) -> int:
    """Status word of the tcgen05 kernels kept at the start of `scratch`
    (synchronises the current stream)."""
    code = ctypes.c_uint(0)
    _call("nntile_b200_flash_sdpa_read_status", _stream(), _ptr(scratch), ctypes.byref(code))
    return int(code.value)


def flash_sdpa_fwd(seq, head, batch, K, Q, mask, scratch_lse, V, scratch_A, lse, A):
    """Pointer order of flash_sdpa_fwd_cudnn::execute_graph."""
    _call(f"nntile_b200_flash_sdpa_fwd_{_sfx16(Q)}", _stream(), seq, head, batch, _ptr(K), _ptr(Q),
          _ptr(mask), _ptr(scratch_lse), _ptr(V), _ptr(scratch_A), _ptr(lse), _ptr(A))


def flash_sdpa_bwd(seq, head, batch, K, Q, V, A, dA, mask, lse, scratch_dK, scratch_dQ,
                   scratch_dV, dK, dQ, dV):
    """Pointer order of flash_sdpa_bwd_cudnn::execute_graph."""
    _call(f"nntile_b200_flash_sdpa_bwd_{_sfx16(Q)}", _stream(), seq, head, batch, _ptr(K), _ptr(Q),
          _ptr(V), _ptr(A), _ptr(dA), _ptr(mask), _ptr(lse), _ptr(scratch_dK),
          _ptr(scratch_dQ), _ptr(scratch_dV), _ptr(dK), _ptr(dQ), _ptr(dV))


def flash_sdpa_gqa_scratch_bytes(seq, head, batch, group, kv_heads) -> int:
    return int(_lib.load().nntile_b200_flash_sdpa_gqa_scratch_bytes(seq, head, batch, group,
                                                                    kv_heads))


def flash_sdpa_fwd_gqa(seq, head, batch, group, kv_heads, K, Q, mask, V, lse, A, scratch):
    """K, V un-replicated [head, seq, batch, kv_heads]; Q, A with the group index."""
    _call(f"nntile_b200_flash_sdpa_fwd_gqa_{_sfx16(Q)}", _stream(), seq, head, batch, group, kv_heads,
          _ptr(K), _ptr(Q), _ptr(mask), _ptr(V), _ptr(lse), _ptr(A), _ptr(scratch),
          scratch.numel()*scratch.element_size())


def flash_sdpa_bwd_gqa(seq, head, batch, group, kv_heads, K, Q, V, A, dA, mask, lse, dK, dQ, dV,
                       scratch):
    _call(f"nntile_b200_flash_sdpa_bwd_gqa_{_sfx16(Q)}", _stream(), seq, head, batch, group, kv_heads,
          _ptr(K), _ptr(Q), _ptr(V), _ptr(A), _ptr(dA), _ptr(mask), _ptr(lse), _ptr(dK),
          _ptr(dQ), _ptr(dV), _ptr(scratch), scratch.numel()*scratch.element_size())


def flash_sdpa_path(seq, head, batch, backward=False) -> int:
    lib = _lib.load()
    fn = lib.nntile_b200_flash_sdpa_bwd_path if backward else lib.nntile_b200_flash_sdpa_fwd_path
    return int(fn(seq, head, batch))


def kv_cache_append(head, max_seq, batch, kv_heads, cache_len, new_seq, src, cache):
    _call("nntile_b200_kv_cache_append_bf16", _stream(), head, max_seq, batch, kv_heads,
          cache_len, new_seq, _ptr(src), _ptr(cache))


def decode_workspace_bytes(head, length, batch, group, kv_heads) -> int:
    return int(_lib.load().nntile_b200_decode_sdpa_workspace_bytes(head, length, batch, group,
                                                                   kv_heads))


def decode_sdpa(head, max_seq, length, batch, group, kv_heads, q, Kcache, Vcache, out,
                lse_out, workspace):
    _call("nntile_b200_decode_sdpa_bf16", _stream(), head, max_seq, length, batch, group,
          kv_heads, _ptr(q), _ptr(Kcache), _ptr(Vcache), _ptr(out), _ptr(lse_out),
          _ptr(workspace), workspace.numel()*workspace.element_size())
