"""CPU oracle for the tiled SDPA path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package; the shipped library must never do so.

Two arithmetic back ends sit behind the same Python functions:

``port``  ``libsdpa_oracle.so`` built from ``sdpa_oracle.c`` - a plain-C
          restatement of the reference kernels (each function cites the
          reference file:line it follows).
``ref``   ``_ref/libnntile_ref_cpu.so`` - the reference's own
          ``src/kernel/<op>/cpu.cc`` and ``src/kernel/cblas.cc`` compiled in place
          (fp32 sgemm from OpenBLAS, as the reference's CPU codelets run it).

On top of them this module restates the StarPU-bound host logic that cannot be
compiled here: the (m, n, k) derivations of the tile layer, the tile loops of
the tensor layer, and the order of operations of ``nntile.layer.Sdpa``.

Arrays are numpy, Fortran order.  dtype float32 is fp32; dtype float16 is IEEE half
(the fused pair only); dtype uint16 holds
bfloat16 bit patterns (round to nearest even, the reference's CUDA build).
"""
from __future__ import annotations

import ctypes
import itertools
import math
import os

import numpy as np

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_vp = ctypes.c_void_p


def _load(path):
    return ctypes.CDLL(path) if path and os.path.exists(path) else None


def _ensure_port():
    try:
        return _load(_build.build_port())
    except Exception:  # compiler missing: use a prebuilt copy if there is one
        return _load(_build.PORT_SO)


port = _ensure_port()
if port is None:
    raise ImportError("oracle: libsdpa_oracle.so is missing and could not be built")
ref = _load(_build.REF_SO)
if ref is not None:
    ref.ref_bf16_rounds_to_nearest.restype = ctypes.c_int


def have_ref() -> bool:
    return ref is not None


def ref_gpu():
    """The reference's own GPU wrappers of the fused pair (cuDNN graph + merge /
    add_inplace kernels, oracle/_ref_gpu), loaded on demand; None when the library
    was not built or cuDNN cannot be loaded.  Needs a GPU to call."""
    global _ref_gpu
    if _ref_gpu is False:
        try:
            _ref_gpu = _load(_build.REF_GPU_SO)
        except OSError:
            _ref_gpu = None
        if _ref_gpu is not None:
            vp, i64 = ctypes.c_void_p, ctypes.c_int64
            for sfx in ("bf16", "fp16"):
                getattr(_ref_gpu, f"refgpu_flash_sdpa_fwd_{sfx}").argtypes = [vp, i64, i64, i64] + [vp]*8
                getattr(_ref_gpu, f"refgpu_flash_sdpa_bwd_{sfx}").argtypes = [vp, i64, i64, i64] + [vp]*13
    return _ref_gpu


_ref_gpu = False


def _p(a: np.ndarray):
    assert a.flags.f_contiguous or a.flags.c_contiguous
    return _vp(a.ctypes.data)


def _sfx(a: np.ndarray) -> str:
    if a.dtype == np.float32:
        return "f32"
    if a.dtype == np.uint16:
        return "bf16"
    if a.dtype == np.float16:
        return "f16"
    raise TypeError(f"oracle: unsupported dtype {a.dtype}")


def _fn(backend: str, name: str, sfx: str):
    if backend == "ref" and sfx == "f16":
        backend = "port"      # oracle/_ref carries the fp32 and bf16 instantiations
    if backend == "ref":
        if ref is None:
            raise RuntimeError("oracle: _ref library not built")
        f = getattr(ref, f"ref_{name}_{sfx}")
    else:
        f = getattr(port, f"orc_{name}_{sfx}")
    f.restype = None
    return f


# --------------------------------------------------------------------------
# dtype helpers
# --------------------------------------------------------------------------
def to_bf16(x) -> np.ndarray:
    """float32 array -> uint16 bfloat16 bits (round to nearest even)."""
    x = np.asarray(x, dtype=np.float32)
    xf = np.asfortranarray(x)
    out = np.empty(xf.shape, dtype=np.uint16, order="F")
    port.orc_f32_to_bf16(_i64(xf.size), _p(xf), _p(out))
    return out


def from_bf16(u) -> np.ndarray:
    u = np.asfortranarray(np.asarray(u, dtype=np.uint16))
    out = np.empty(u.shape, dtype=np.float32, order="F")
    port.orc_bf16_to_f32(_i64(u.size), _p(u), _p(out))
    return out


def as_f32(a) -> np.ndarray:
    return from_bf16(a) if a.dtype == np.uint16 else np.asfortranarray(a, dtype=np.float32)


def cast(x_f32, like_dtype) -> np.ndarray:
    if np.dtype(like_dtype) == np.uint16:
        return to_bf16(x_f32)
    if np.dtype(like_dtype) == np.float16:
        return np.asfortranarray(x_f32, dtype=np.float16)      # round to nearest even
    return np.asfortranarray(x_f32, dtype=np.float32)


def zeros(shape, dtype) -> np.ndarray:
    return np.zeros(shape, dtype=dtype, order="F")  # bf16 +0.0 is 0x0000


def full(shape, value, dtype) -> np.ndarray:
    return cast(np.full(shape, value, dtype=np.float32, order="F"), dtype)


# --------------------------------------------------------------------------
# kernel-level ops (in place on Fortran arrays); argument order follows
# include/nntile/kernel/<op>/cpu.hh of the reference
# --------------------------------------------------------------------------
def gemm(transA, transB, m, n, k, batch, alpha, A, B, beta, C, backend="port"):
    sfx = _sfx(C)
    if backend == "ref" and sfx != "f32":
        backend = "port"  # the reference has no CPU bf16 gemm (src/starpu/gemm.cc:38-45)
    _fn(backend, "gemm", sfx)(ctypes.c_int(int(transA)), ctypes.c_int(int(transB)),
                             _i64(m), _i64(n), _i64(k), _i64(batch), _f32(alpha),
                             _p(A), _p(B), _f32(beta), _p(C))


def mask_scalar(nrows, ncols, mask, val, data, backend="port"):
    mask = np.asfortranarray(mask, dtype=np.uint8)
    _fn(backend, "mask_scalar", _sfx(data))(_i64(nrows), _i64(ncols), _p(mask),
                                            _f32(val), _p(data))


def maxsumexp(m, n, k, src, dst, backend="port"):
    _fn(backend, "maxsumexp", _sfx(src))(_i64(m), _i64(n), _i64(k), _p(src), _p(dst))


def softmax_inplace(m, n, k, mse, alpha, dst, backend="port"):
    _fn(backend, "softmax_inplace", _sfx(dst))(_i64(m), _i64(n), _i64(k), _p(mse),
                                               _f32(alpha), _p(dst))


def sumprod_slice(m, n, k, alpha, a, b, beta, dst, backend="port"):
    _fn(backend, "sumprod_slice", _sfx(dst))(_i64(m), _i64(n), _i64(k), _f32(alpha),
                                             _p(a), _p(b), _f32(beta), _p(dst))


def add_slice_inplace(m, n, k, alpha, src, beta, dst, backend="port"):
    _fn(backend, "add_slice_inplace", _sfx(dst))(_i64(m), _i64(n), _i64(k),
                                                 _f32(alpha), _p(src), _f32(beta),
                                                 _p(dst))


def multiply_inplace(nelems, alpha, src, dst, backend="port"):
    _fn(backend, "multiply_inplace", _sfx(dst))(_i64(nelems), _f32(alpha), _p(src),
                                                _p(dst))


def add_inplace(nelems, alpha, src, beta, dst, backend="port"):
    _fn(backend, "add_inplace", _sfx(dst))(_i64(nelems), _f32(alpha), _p(src),
                                           _f32(beta), _p(dst))


def accumulate_attn_output(head, seq, batch, src_lse, src_attn, dst_lse, dst_attn,
                           cuda_rules=True, backend="port"):
    """``cuda_rules`` selects accumulate_attn_output/cuda.cu semantics (the ones
    the fused path runs); the ``ref`` back end only has the CPU-build rules."""
    if backend == "ref":
        _fn("ref", "accumulate_attn_output", _sfx(dst_attn))(
            _i64(head), _i64(seq), _i64(batch), _p(src_lse), _p(src_attn),
            _p(dst_lse), _p(dst_attn))
    else:
        _fn("port", "accumulate_attn_output", _sfx(dst_attn))(
            _i64(head), _i64(seq), _i64(batch), _p(src_lse), _p(src_attn),
            _p(dst_lse), _p(dst_attn), ctypes.c_int(1 if cuda_rules else 0))


def transpose(m, n, alpha, src, dst, backend="port"):
    """dst[i*n + j] = alpha*src[i + j*m] (include/nntile/kernel/transpose/cpu.hh:24)."""
    _fn(backend, "transpose", _sfx(dst))(_i64(m), _i64(n), _f32(alpha), _p(src), _p(dst))


def rope(m, n, sin, cos, src, dst, backend="port"):
    """include/nntile/kernel/rope/cpu.hh:23."""
    _fn(backend, "rope", _sfx(dst))(_i64(m), _i64(n), _p(sin), _p(cos), _p(src), _p(dst))


def add_fiber_inplace(m, n, k, batch, alpha, src, beta, dst, backend="port"):
    """include/nntile/kernel/add_fiber_inplace/cpu.hh:24."""
    _fn(backend, "add_fiber_inplace", _sfx(dst))(_i64(m), _i64(n), _i64(k), _i64(batch),
                                                 _f32(alpha), _p(src), _f32(beta), _p(dst))


def rope_sin_cos(head, positions, theta=10000.0):
    """sin, cos float32 [head/2, seq, batch] as LlamaAttention._fill_sin_cos builds
    them (wrappers/python/nntile/model/llama_attention.py:1122-1134); `positions`
    is [batch, seq]."""
    tmp = np.arange(0, head, 2, dtype=np.float32)
    inv_freq = 1.0/(theta**(tmp/head))
    frame = np.empty((head//2, positions.shape[1], positions.shape[0]))
    for i in range(positions.shape[0]):
        frame[:, :, i] = np.outer(inv_freq, positions[i, :])
    return (np.sin(frame).astype(np.float32, order="F"),
            np.cos(frame).astype(np.float32, order="F"))


def attention_prologue(proj, sin=None, cos=None, bias=None, backend="port"):
    """What the reference's attention layers run between a projection and the SDPA
    layer: transpose_async of [lead..., head, seq, batch] into [head, seq, batch,
    lead...] (the lead axes flattened here), then rope_async (Llama,
    llama_attention.py:592-610) or add_fiber_inplace_async of a [head, lead] bias
    (GPT-2, gpt2_attention.py:258-269).  `proj` is a Fortran array
    [lead, head, seq, batch]; returns [head, seq, batch, lead]."""
    lead, head, seq, batch = proj.shape
    out = zeros((head, seq, batch, lead), proj.dtype)
    transpose(lead, head*seq*batch, 1.0, proj, out, backend=backend)
    if sin is not None:
        rot = zeros(out.shape, proj.dtype)
        rope((head//2)*seq*batch, lead, sin, cos, out, rot, backend=backend)
        out = rot
    if bias is not None:
        add_fiber_inplace(1, seq*batch, head, lead, 1.0, bias, 1.0, out, backend=backend)
    return out


def attention_epilogue(attn, backend="port"):
    """transpose_async(1.0, A, At, 3) behind the SDPA layer (llama_attention.py:
    620-623): [head, seq, batch, lead] -> [lead, head, seq, batch]."""
    head, seq, batch, lead = attn.shape
    out = zeros((lead, head, seq, batch), attn.dtype)
    transpose(head*seq*batch, lead, 1.0, attn, out, backend=backend)
    return out


def flash_sdpa_fwd_tile(seq, head, batch, K, Q, mask, V, lse, A):
    """One fused-forward tile task (src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:145-202);
    ``lse`` and ``A`` are updated in place."""
    s_lse = np.empty(seq * batch, dtype=np.float32)
    s_A = np.empty(seq * head * batch, dtype=A.dtype)
    _fn("port", "flash_sdpa_fwd_tile", _sfx(A))(
        _i64(seq), _i64(head), _i64(batch), _p(K), _p(Q), _p(mask), _p(s_lse),
        _p(V), _p(s_A), _p(lse), _p(A))


def flash_sdpa_bwd_tile(seq, head, batch, K, Q, V, A, dA, mask, lse, dK, dQ, dV):
    """One fused-backward tile task (src/kernel/flash_sdpa_bwd_cudnn/cuda.cc:171-218);
    ``dK, dQ, dV`` are incremented in place."""
    n = seq * head * batch
    sk, sq, sv = (np.empty(n, dtype=dK.dtype) for _ in range(3))
    _fn("port", "flash_sdpa_bwd_tile", _sfx(dK))(
        _i64(seq), _i64(head), _i64(batch), _p(K), _p(Q), _p(V), _p(A), _p(dA),
        _p(mask), _p(lse), _p(sk), _p(sq), _p(sv), _p(dK), _p(dQ), _p(dV))


# --------------------------------------------------------------------------
# tile bookkeeping (include/nntile/tile/traits.hh, tensor/traits.hh): a tensor
# is a grid of separately stored Fortran-order tiles of shape `basetile`
# (ragged at the upper edges)
# --------------------------------------------------------------------------
class Tiled:
    def __init__(self, array: np.ndarray, basetile):
        self.shape = tuple(array.shape)
        self.basetile = tuple(int(b) for b in basetile)
        assert len(self.basetile) == len(self.shape)
        self.grid = tuple(-(-s // b) for s, b in zip(self.shape, self.basetile))
        self.dtype = array.dtype
        self.tiles = {}
        for idx in itertools.product(*(range(g) for g in self.grid)):
            self.tiles[idx] = np.asfortranarray(array[self._slices(idx)].copy(order="F"))

    def _slices(self, idx):
        return tuple(slice(i * b, min((i + 1) * b, s))
                     for i, b, s in zip(idx, self.basetile, self.shape))

    def tile(self, idx) -> np.ndarray:
        return self.tiles[tuple(idx)]

    def gather(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=self.dtype, order="F")
        for idx, t in self.tiles.items():
            out[self._slices(idx)] = t
        return out


def _batch_grid(t: Tiled, first_batch_axis: int):
    return list(itertools.product(*(range(g) for g in t.grid[first_batch_axis:])))


# --------------------------------------------------------------------------
# nntile.layer.Sdpa, unfused chain (wrappers/python/nntile/layer/sdpa.py)
# --------------------------------------------------------------------------
def sdpa_scale(head_size: int) -> float:
    """sdpa.py:149 - the scale is rounded through float32."""
    return float(np.float32(1.0) / np.sqrt(np.float32(head_size)))


def vanilla_forward(Q, K, V, mask_bool, q_tile=None, k_tile=None, batch_tile=None,
                    backend="port"):
    """sdpa.py:407-455: gemm(QK^T) -> mask_scalar(-inf) -> maxsumexp ->
    softmax_inplace -> gemm(PV).  Q is [D, Sq, B, G, H]; K, V are
    [D, Sk, B, G, H]; mask_bool is [Sk, Sq] (true = keep) or None.
    Returns (Y, attn, attn_maxsumexp).  Tile loops follow
    src/tensor/gemm.cc:378-409, src/tensor/mask_scalar.cc:47-61,
    src/tensor/maxsumexp.cc:80-107, src/tensor/softmax_inplace.cc:80-112 and
    the (m, n, k) of src/tile/{gemm.cc:281-312, mask_scalar.cc:56-59,
    maxsumexp.cc:67-70, softmax_inplace.cc:64-69}."""
    D, Sq = Q.shape[0], Q.shape[1]
    Sk = K.shape[1]
    bshape = Q.shape[2:]
    q_tile = q_tile or Sq
    k_tile = k_tile or Sk
    batch_tile = tuple(batch_tile or bshape)
    dt = Q.dtype
    scale = sdpa_scale(D)
    tQ = Tiled(Q, (D, q_tile) + batch_tile)
    tK = Tiled(K, (D, k_tile) + batch_tile)
    tV = Tiled(V, (D, k_tile) + batch_tile)
    attn = Tiled(zeros((Sk, Sq) + bshape, dt), (k_tile, q_tile) + batch_tile)
    mse = Tiled(zeros((2, Sq) + bshape, dt), (2, q_tile) + batch_tile)
    Y = Tiled(zeros((D, Sq) + bshape, dt), (D, q_tile) + batch_tile)
    tM = None
    if mask_bool is not None:
        tM = Tiled(np.asfortranarray(mask_bool, dtype=np.uint8), (k_tile, q_tile))
    for bt in _batch_grid(tQ, 2):
        for qi in range(tQ.grid[1]):
            q = tQ.tile((0, qi) + bt)
            sq = q.shape[1]
            nb = int(np.prod(q.shape[2:]))
            for ki in range(tK.grid[1]):
                k = tK.tile((0, ki) + bt)
                sk = k.shape[1]
                a = attn.tile((ki, qi) + bt)
                gemm(1, 0, sk, sq, D, nb, scale, k, q, 0.0, a, backend)
                if tM is not None:
                    mask_scalar(sk * sq, nb, tM.tile((ki, qi)), -np.inf, a, backend)
            ms = mse.tile((0, qi) + bt)
            for ki in range(tK.grid[1]):
                a = attn.tile((ki, qi) + bt)
                maxsumexp(1, sq * nb, a.shape[0], a, ms, backend)
            for ki in range(tK.grid[1]):
                a = attn.tile((ki, qi) + bt)
                softmax_inplace(1, sq * nb, a.shape[0], ms, 1.0, a, backend)
            y = Y.tile((0, qi) + bt)
            for ki in range(tK.grid[1]):
                v = tV.tile((0, ki) + bt)
                a = attn.tile((ki, qi) + bt)
                gemm(0, 0, D, sq, a.shape[0], nb, 1.0, v, a,
                     0.0 if ki == 0 else 1.0, y, backend)
    return Y.gather(), attn.gather(), mse.gather()


def vanilla_backward(Q, K, V, Y, dY, attn, mask_bool, dQ, dK, dV, backend="port"):
    """sdpa.py:595-698 on a single tile per tensor: dA = V^T dY; dV += dY A^T;
    delta = sumprod_slice(Y, dY); dA -= delta; dA *= A; mask_scalar(0);
    dK += scale Q dA^T; dQ += scale K dA.  dQ, dK, dV are incremented."""
    D, Sq = Q.shape[0], Q.shape[1]
    Sk = K.shape[1]
    nb = int(np.prod(Q.shape[2:]))
    dt = Q.dtype
    scale = sdpa_scale(D)
    dA = zeros(attn.shape, dt)
    gemm(1, 0, Sk, Sq, D, nb, 1.0, V, dY, 0.0, dA, backend)
    gemm(0, 1, D, Sk, Sq, nb, 1.0, dY, attn, 1.0, dV, backend)
    delta = zeros((Sq,) + Q.shape[2:], dt)
    sumprod_slice(1, Sq * nb, D, 1.0, Y, dY, 0.0, delta, backend)
    add_slice_inplace(1, Sq * nb, Sk, -1.0, delta, 1.0, dA, backend)
    multiply_inplace(dA.size, 1.0, attn, dA, backend)
    if mask_bool is not None:
        mask_scalar(Sk * Sq, nb, mask_bool, 0.0, dA, backend)
    gemm(0, 1, D, Sk, Sq, nb, scale, Q, dA, 1.0, dK, backend)
    gemm(0, 0, D, Sq, Sk, nb, scale, K, dA, 1.0, dQ, backend)
    return dA


# --------------------------------------------------------------------------
# nntile.layer.Sdpa, fused chain
# --------------------------------------------------------------------------
def flash_forward(Q, K, V, mask_add, seq_tile=None, batch_tile=None):
    """sdpa.py:533-557 + src/tensor/flash_sdpa_fwd_cudnn.cc:221-274 +
    src/tile/flash_sdpa_fwd_cudnn.cc:170-173: lse=-inf, A=0, then for every
    output tile, for EVERY K/V sequence tile (masked ones included) one tile
    task.  Q, K, V are [D, S, B, G, H]; mask_add is the additive [Sk, Sq] mask in
    the tensors' dtype.  Returns (A, lse[S, B, G, H])."""
    D, S = Q.shape[0], Q.shape[1]
    bshape = Q.shape[2:]
    seq_tile = seq_tile or S
    batch_tile = tuple(batch_tile or bshape)
    dt = Q.dtype
    tQ = Tiled(Q, (D, seq_tile) + batch_tile)
    tK = Tiled(K, (D, seq_tile) + batch_tile)
    tV = Tiled(V, (D, seq_tile) + batch_tile)
    tM = Tiled(mask_add, (seq_tile, seq_tile))
    A = Tiled(zeros(Q.shape, dt), (D, seq_tile) + batch_tile)
    lse = Tiled(np.full((S,) + bshape, -np.inf, dtype=np.float32, order="F"),
                (seq_tile,) + batch_tile)
    for bt in _batch_grid(tQ, 2):
        for qi in range(tQ.grid[1]):
            q = tQ.tile((0, qi) + bt)
            sq = q.shape[1]
            nb = int(np.prod(q.shape[2:]))
            for ki in range(tK.grid[1]):
                k = tK.tile((0, ki) + bt)
                if k.shape[1] != sq:
                    raise RuntimeError("K tile sequence length mismatches Q tile")
                flash_sdpa_fwd_tile(sq, D, nb, k, q, tM.tile((ki, qi)),
                                    tV.tile((0, ki) + bt), lse.tile((qi,) + bt),
                                    A.tile((0, qi) + bt))
    return A.gather(), lse.gather()


def flash_backward(Q, K, V, A, dA, mask_add, lse, dQ, dK, dV, seq_tile=None,
                   batch_tile=None):
    """sdpa.py:559-593 + src/tensor/flash_sdpa_bwd_cudnn.cc:172-246: for every Q
    tile and every K/V tile one task that adds its share into dK, dQ, dV."""
    D, S = Q.shape[0], Q.shape[1]
    bshape = Q.shape[2:]
    seq_tile = seq_tile or S
    batch_tile = tuple(batch_tile or bshape)
    bt5 = (D, seq_tile) + batch_tile
    tQ, tK, tV, tA, tdA = (Tiled(x, bt5) for x in (Q, K, V, A, dA))
    tdQ, tdK, tdV = (Tiled(x, bt5) for x in (dQ, dK, dV))
    tM = Tiled(mask_add, (seq_tile, seq_tile))
    tL = Tiled(lse, (seq_tile,) + batch_tile)
    for bt in _batch_grid(tQ, 2):
        for qi in range(tQ.grid[1]):
            q = tQ.tile((0, qi) + bt)
            sq = q.shape[1]
            nb = int(np.prod(q.shape[2:]))
            for ki in range(tK.grid[1]):
                flash_sdpa_bwd_tile(
                    sq, D, nb, tK.tile((0, ki) + bt), q, tV.tile((0, ki) + bt),
                    tA.tile((0, qi) + bt), tdA.tile((0, qi) + bt),
                    tM.tile((ki, qi)), tL.tile((qi,) + bt),
                    tdK.tile((0, ki) + bt), tdQ.tile((0, qi) + bt),
                    tdV.tile((0, ki) + bt))
    return tdQ.gather(), tdK.gather(), tdV.gather()


# --------------------------------------------------------------------------
# decode: what the reference runs for one new token against a KV cache
# --------------------------------------------------------------------------
def decode_chain(q, Kc, Vc, length=None, backend="port"):
    """wrappers/python/nntile/model/llama_attention.py:533-616, 672-676: with a
    non-empty cache the fused path is off, K/V are replicated `kv_group_size`
    times and the unfused chain runs with one query position and no mask.
    q is [D, 1, B, G, H]; Kc, Vc are the caches [D, L, B, H]; only the first
    `length` positions are attended.  Returns Y [D, 1, B, G, H]."""
    D, _, B, G, H = q.shape
    L = Kc.shape[1] if length is None else int(length)
    Krep = np.asfortranarray(np.repeat(Kc[:, :L, :, None, :], G, axis=3))
    Vrep = np.asfortranarray(np.repeat(Vc[:, :L, :, None, :], G, axis=3))
    Y, _, _ = vanilla_forward(np.asfortranarray(q), Krep, Vrep, None, backend=backend)
    return Y


# --------------------------------------------------------------------------
# fp64 ground truth, the formulas of the reference's kernel tests
# (tests/kernel/flash_sdpa_fwd_cudnn.cc:83-175, flash_sdpa_bwd_cudnn.cc:174-263)
# --------------------------------------------------------------------------
def sdpa_fp64(Q, K, V, mask_add):
    """Q [D,Sq,...], K,V [D,Sk,...] (any dtype), mask_add [Sk,Sq] additive.
    Returns (A float64 [D,Sq,...], lse float64 [Sq,...])."""
    q = as_f32(Q).astype(np.float64)
    k = as_f32(K).astype(np.float64)
    v = as_f32(V).astype(np.float64)
    m = as_f32(mask_add).astype(np.float64)
    D = q.shape[0]
    s = np.einsum("hk...,hq...->kq...", k, q) / math.sqrt(D)
    s = s + m.reshape(m.shape + (1,) * (s.ndim - 2))
    top = np.max(s, axis=0, keepdims=True)
    top = np.where(np.isfinite(top), top, 0.0)
    p = np.exp(s - top)
    den = p.sum(axis=0, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        lse = (np.log(den) + top)[0]
        w = np.where(den > 0, p / den, 0.0)
    a = np.einsum("hk...,kq...->hq...", v, w)
    return a, lse


def sdpa_bwd_fp64(Q, K, V, A, dA, mask_add, lse):
    """Gradients from the GIVEN A and lse.  Returns (dQ, dK, dV) float64."""
    q, k, v, a, da = (as_f32(x).astype(np.float64) for x in (Q, K, V, A, dA))
    m = as_f32(mask_add).astype(np.float64)
    l64 = np.asarray(lse, dtype=np.float64)
    D = q.shape[0]
    sc = 1.0 / math.sqrt(D)
    s = np.einsum("hk...,hq...->kq...", k, q) * sc
    s = s + m.reshape(m.shape + (1,) * (s.ndim - 2))
    with np.errstate(invalid="ignore"):
        p = np.where(np.isneginf(s), 0.0, np.exp(s - l64[None]))
    delta = (a * da).sum(axis=0)
    dp = np.einsum("hk...,hq...->kq...", v, da)
    ds = p * (dp - delta[None])
    dv = np.einsum("kq...,hq...->hk...", p, da)
    dq = np.einsum("kq...,hk...->hq...", ds, k) * sc
    dk = np.einsum("kq...,hq...->hk...", ds, q) * sc
    return dq, dk, dv


def rel_err(actual, reference) -> float:
    """Frobenius-relative error, the norm the reference's tests use."""
    a = np.asarray(actual, dtype=np.float64)
    r = np.asarray(reference, dtype=np.float64)
    den = np.linalg.norm(r)
    return float(np.linalg.norm(a - r) / (den if den != 0 else 1.0))


def kv_cache_append(cache, cache_len, partial):
    """wrappers/python/nntile/layer/cache_utils.py:146-176: KVCache.append copies
    k_partial / v_partial [D, n, B, H] into the preallocated cache [D, L, B, H] at
    sequence offset `cache_len` (copy_intersection_async).  In place; returns the
    new length."""
    n = partial.shape[1]
    if cache_len + n > cache.shape[1]:
        raise ValueError("append past the end of the cache")
    cache[:, cache_len:cache_len + n] = partial
    return cache_len + n
