"""Host-side mirror of ``nntile.layer.Sdpa`` for the path (reference:
wrappers/python/nntile/layer/sdpa.py).

Tensors are torch CUDA buffers holding NNTile's Fortran-order arrays: an NNTile
tensor of shape [head, seq, batch, group, kv_heads] is a contiguous torch tensor
of shape (kv_heads, group, batch, seq, head).  ``from_fortran`` / ``to_fortran``
convert from and to numpy Fortran arrays (bf16 as uint16 bit patterns).

``Sdpa`` issues the same operations in the same order as the reference layer:
the unfused chain (gemm -> mask_scalar -> maxsumexp -> softmax_inplace -> gemm
and its backward, sdpa.py:407-455, 595-698) or the fused tile tasks (fill/clear
prologue + flash forward, flash backward, sdpa.py:533-593) with the reference's
tile loops run by the C library.
"""
from __future__ import annotations

import ctypes
import itertools
import math

import numpy as np
import torch

from . import _lib, ops


def from_fortran(arr: np.ndarray, device="cuda") -> torch.Tensor:
    """numpy Fortran array (float32, float16, or uint16 = bf16 bits) -> torch buffer."""
    a = np.asfortranarray(arr)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.T.view(np.int16).copy()).view(torch.bfloat16).to(device)
    if a.dtype == np.bool_:
        return torch.from_numpy(a.T.copy()).to(device)
    return torch.from_numpy(a.T.copy()).to(device)


def to_fortran(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return np.asfortranarray(t.view(torch.int16).numpy().view(np.uint16).T)
    return np.asfortranarray(t.numpy().T)


def sdpa_scale(head_size: int) -> float:
    """sdpa.py:149."""
    return float(np.float32(1.0)/np.sqrt(np.float32(head_size)))


class TiledBuffer:
    """A tensor cut into separately stored Fortran-order tiles, the storage model
    of nntile::tensor::Tensor (include/nntile/tensor/tensor.hh).  `shape` and
    `basetile` are in NNTile (Fortran) order."""

    def __init__(self, full: torch.Tensor, basetile):
        self.shape = tuple(reversed(full.shape))
        self.basetile = tuple(int(b) for b in basetile)
        self.grid = tuple(-(-s//b) for s, b in zip(self.shape, self.basetile))
        self.dtype = full.dtype
        self.tiles = []
        # Fortran order of the tile grid: first index fastest
        for idx in itertools.product(*(range(g) for g in reversed(self.grid))):
            idx = tuple(reversed(idx))
            self.tiles.append(full[self._slices(idx)].contiguous())

    def _slices(self, idx):
        sl = [slice(i*b, min((i + 1)*b, s)) for i, b, s in zip(idx, self.basetile, self.shape)]
        return tuple(reversed(sl))

    def pointers(self):
        arr = (ctypes.c_void_p*len(self.tiles))(*[t.data_ptr() for t in self.tiles])
        return arr

    def gather(self) -> torch.Tensor:
        out = torch.empty(tuple(reversed(self.shape)), dtype=self.dtype,
                          device=self.tiles[0].device)
        for n, idx in enumerate(itertools.product(*(range(g) for g in reversed(self.grid)))):
            out[self._slices(tuple(reversed(idx)))] = self.tiles[n]
        return out


def _i64arr(vals):
    return (ctypes.c_int64*len(vals))(*[int(v) for v in vals])


def _tensor_call(name, shape5, base5, tiled, scratch_holder=None):
    """Run one tensor-level C entry point on lists of TiledBuffer."""
    lib = _lib.load()
    nbytes = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(_i64arr(shape5), _i64arr(base5))
    dev = tiled[0].tiles[0].device
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    keep = [t.pointers() for t in tiled]
    st = getattr(lib, name)(
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), _i64arr(shape5),
        _i64arr(base5), *[ctypes.cast(p, ctypes.POINTER(ctypes.c_void_p)) for p in keep],
        ctypes.c_void_p(scratch.data_ptr()), nbytes)
    _lib.check(name, st)
    if scratch_holder is not None:
        scratch_holder.append(scratch)
    return scratch


def flash_sdpa_fwd_async(K, Q, mask, lse, V, A, seq_tile=None, batch_tile=None, scratch_out=None):
    """nntile.functions.flash_sdpa_fwd_cudnn_async on whole tensors: cuts them into
    tiles like the reference's traits do, runs the C tensor-level loops, gathers A
    and lse back in place.  Q, A: (H, G, B, S, D) bf16; K, V: the same shape, or
    (H, B, S, D) = [head, seq, batch, kv_heads] not replicated over the group
    (grouped-query form); mask: additive (Sq, Sk) bf16 buffer = Fortran [Sk, Sq];
    lse: (H, G, B, S) fp32."""
    H, G, B, S, D = Q.shape
    gqa = K.dim() == 4
    seq_tile = seq_tile or S
    bt = tuple(batch_tile or (B, G, H))
    base5 = (D, seq_tile) + bt
    kv_base = (D, seq_tile, bt[0], bt[2]) if gqa else base5
    tK, tV = TiledBuffer(K, kv_base), TiledBuffer(V, kv_base)
    tQ, tA = TiledBuffer(Q, base5), TiledBuffer(A, base5)
    tM = TiledBuffer(mask, (seq_tile, seq_tile))
    tL = TiledBuffer(lse, (seq_tile,) + bt)
    name = f"nntile_b200_tensor_flash_sdpa_fwd{'_gqa' if gqa else ''}_{ops._sfx16(Q)}"
    _tensor_call(name, (D, S, B, G, H), base5, [tK, tQ, tM, tL, tV, tA], scratch_out)
    A.copy_(tA.gather())
    lse.copy_(tL.gather())


def flash_sdpa_bwd_async(K, Q, V, A, dA, mask, lse, dK, dQ, dV, seq_tile=None,
                         batch_tile=None, scratch_out=None):
    """nntile.functions.flash_sdpa_bwd_cudnn_async on whole tensors (K, V, dK, dV
    5-D like Q, or 4-D un-replicated for the grouped-query form)."""
    H, G, B, S, D = Q.shape
    gqa = K.dim() == 4
    seq_tile = seq_tile or S
    bt = tuple(batch_tile or (B, G, H))
    base5 = (D, seq_tile) + bt
    kv_base = (D, seq_tile, bt[0], bt[2]) if gqa else base5
    tK, tV, tdK, tdV = (TiledBuffer(x, kv_base) for x in (K, V, dK, dV))
    tQ, tA, tdA, tdQ = (TiledBuffer(x, base5) for x in (Q, A, dA, dQ))
    tM = TiledBuffer(mask, (seq_tile, seq_tile))
    tL = TiledBuffer(lse, (seq_tile,) + bt)
    name = f"nntile_b200_tensor_flash_sdpa_bwd{'_gqa' if gqa else ''}_{ops._sfx16(Q)}"
    _tensor_call(name, (D, S, B, G, H), base5, [tK, tQ, tV, tA, tdA, tM, tL, tdK, tdQ, tdV],
                 scratch_out)
    dK.copy_(tdK.gather())
    dQ.copy_(tdQ.gather())
    dV.copy_(tdV.gather())


class _TiledChain:
    """Tile loops of the unfused chain: what nntile::tensor::gemm_async
    (src/tensor/gemm.cc:344-410: every output tile, contraction tiles accumulated
    with beta = 1 after the first), maxsumexp_async (src/tensor/maxsumexp.cc:80-107:
    the K tiles of a fibre accumulate into the same (max, sum) pair),
    softmax_inplace_async (src/tensor/softmax_inplace.cc:80-112), mask_scalar_async
    (src/tensor/mask_scalar.cc:26-62), sumprod_slice_async, add_slice_inplace_async
    and multiply_inplace_async do on tiled tensors, in the order
    nntile.layer.Sdpa issues them (sdpa.py:407-455, 595-698).  Tensors are cut along
    the sequence axis (queries and keys separately) and the three batch axes; the
    head axis is one tile."""

    def __init__(self, layer, q_tile, k_tile, batch_tile):
        self.L = layer
        H, G, B, Sq, D = layer.q.shape
        Sk = layer.k.shape[3]
        self.bt = tuple(batch_tile or (B, G, H))
        self.qt, self.kt = int(q_tile or Sq), int(k_tile or Sk)
        self.D, self.Sq, self.Sk = D, Sq, Sk
        self.nq, self.nk = -(-Sq//self.qt), -(-Sk//self.kt)
        self.nb = tuple(-(-s//t) for s, t in zip((B, G, H), self.bt))
        self.batch_tiles = self.nb[0]*self.nb[1]*self.nb[2]
        dev, dt = layer.q.device, layer.q.dtype
        self.attn_full = torch.empty((H, G, B, Sq, Sk), dtype=dt, device=dev)
        self.attn = TiledBuffer(self.attn_full, (self.kt, self.qt) + self.bt)
        self.mse = TiledBuffer(torch.empty((H, G, B, Sq, 2), dtype=dt, device=dev),
                               (2, self.qt) + self.bt)
        self.sps = TiledBuffer(torch.empty((H, G, B, Sq), dtype=dt, device=dev),
                               (self.qt,) + self.bt)
        self.mask = None if layer.mask is None else TiledBuffer(layer.mask, (self.kt, self.qt))

    def _cut(self, x, seq_tile):
        return TiledBuffer(x, (self.D, seq_tile) + self.bt)

    @staticmethod
    def _nbatch(t):
        return t.shape[0]*t.shape[1]*t.shape[2]

    def forward(self):
        L = self.L
        q, k, v = self._cut(L.q, self.qt), self._cut(L.k, self.kt), self._cut(L.v, self.kt)
        y = self._cut(L.y, self.qt)
        nq, nk = self.nq, self.nk
        for b in range(self.batch_tiles):
            for qi in range(nq):
                tq, ty, tm = q.tiles[qi + nq*b], y.tiles[qi + nq*b], self.mse.tiles[qi + nq*b]
                nbat, sq = self._nbatch(tq), tq.shape[3]
                ops.clear(tm)
                for ki in range(nk):
                    tk = k.tiles[ki + nk*b]
                    ta = self.attn.tiles[ki + nk*(qi + nq*b)]
                    sk = tk.shape[3]
                    ops.gemm(True, False, sk, sq, self.D, nbat, L.scale, tk, tq, 0.0, ta)
                    if self.mask is not None:
                        ops.mask_scalar(sk*sq, nbat, self.mask.tiles[ki + nk*qi], L.val, ta)
                    ops.maxsumexp(1, sq*nbat, sk, ta, tm)
                for ki in range(nk):
                    ta = self.attn.tiles[ki + nk*(qi + nq*b)]
                    sk = ta.shape[4]
                    ops.softmax_inplace(1, sq*nbat, sk, tm, 1.0, ta)
                    ops.gemm(False, False, self.D, sq, sk, nbat, 1.0, v.tiles[ki + nk*b], ta,
                             0.0 if ki == 0 else 1.0, ty)
        L.y.copy_(y.gather())
        L.attn = self.attn.gather()
        L.attn_maxsumexp = self.mse.gather()

    def backward(self, dy, dq, dk, dv):
        L = self.L
        q, k, v = self._cut(L.q, self.qt), self._cut(L.k, self.kt), self._cut(L.v, self.kt)
        y, tdy = self._cut(L.y, self.qt), self._cut(dy, self.qt)
        tdq, tdk, tdv = self._cut(dq, self.qt), self._cut(dk, self.kt), self._cut(dv, self.kt)
        nq, nk = self.nq, self.nk
        for b in range(self.batch_tiles):
            for qi in range(nq):
                tq, ty, tg = q.tiles[qi + nq*b], y.tiles[qi + nq*b], tdy.tiles[qi + nq*b]
                tsp = self.sps.tiles[qi + nq*b]
                nbat, sq = self._nbatch(tq), tq.shape[3]
                ops.sumprod_slice(1, sq*nbat, self.D, 1.0, ty, tg, 0.0, tsp)
                for ki in range(nk):
                    tk, tv = k.tiles[ki + nk*b], v.tiles[ki + nk*b]
                    ta = self.attn.tiles[ki + nk*(qi + nq*b)]
                    sk = tk.shape[3]
                    da = torch.empty_like(ta)
                    ops.gemm(True, False, sk, sq, self.D, nbat, 1.0, tv, tg, 0.0, da)
                    ops.gemm(False, True, self.D, sk, sq, nbat, 1.0, tg, ta, 1.0,
                             tdv.tiles[ki + nk*b])
                    ops.add_slice_inplace(1, sq*nbat, sk, -1.0, tsp, 1.0, da)
                    ops.multiply_inplace(da.numel(), 1.0, ta, da)
                    if self.mask is not None:
                        ops.mask_scalar(sk*sq, nbat, self.mask.tiles[ki + nk*qi], 0.0, da)
                    ops.gemm(False, True, self.D, sk, sq, nbat, L.scale, tq, da, 1.0,
                             tdk.tiles[ki + nk*b])
                    ops.gemm(False, False, self.D, sq, sk, nbat, L.scale, tk, da, 1.0,
                             tdq.tiles[qi + nq*b])
        dq.copy_(tdq.gather())
        dk.copy_(tdk.gather())
        dv.copy_(tdv.gather())


class Sdpa:
    """Mirror of nntile.layer.Sdpa on tensors that are one tile or are cut along
    the sequence and batch axes (``seq_tile`` for queries and keys alike, or
    ``q_tile`` / ``k_tile`` separately for the unfused chain; ``batch_tile`` =
    (batch, group, kv_heads) extents of a tile).

    q, k, v: (H, G, B, S, D) buffers; for the fused path k and v may also be
    (H, B, S, D), not replicated over the group (grouped-query form).  ``mask``:
    for the unfused chain a bool (Sq, Sk) buffer = Fortran [Sk, Sq] (true = keep);
    for the fused path the additive mask in the tensors' dtype (0 / -inf), as
    sdpa.py:457-531 prepares.
    """

    def __init__(self, q, k, v, mask=None, flash_attention=False, seq_tile=None,
                 batch_tile=None, q_tile=None, k_tile=None):
        self.q, self.k, self.v, self.mask = q, k, v, mask
        self.flash_attention = flash_attention
        self.seq_tile, self.batch_tile = seq_tile, batch_tile
        self.q_tile, self.k_tile = q_tile or seq_tile, k_tile or seq_tile
        H, G, B, S, D = q.shape
        self.head, self.n_seq = D, S
        self.n_seq_k = k.shape[-2]
        self.batch = H*G*B
        self.scale = sdpa_scale(D)
        self.val = -math.inf
        dev, dt = q.device, q.dtype
        self.y = torch.zeros_like(q)
        if flash_attention:
            if dt not in (torch.bfloat16, torch.float16):
                raise TypeError("the fused path takes bf16 or fp16 (fp32 is rejected by the "
                                "reference as well, flash_sdpa_fwd_cudnn/cuda.cc:60-63)")
            self.flash_logsumexp = torch.empty((H, G, B, S), dtype=torch.float32, device=dev)
            if mask is None:
                self.mask = torch.zeros((S, S), dtype=dt, device=dev)
        elif self._tiled():
            self._chain = _TiledChain(self, self.q_tile, self.k_tile, batch_tile)
        else:
            self.attn = torch.empty((H, G, B, S, self.n_seq_k), dtype=dt, device=dev)
            self.attn_maxsumexp = torch.empty((H, G, B, S, 2), dtype=dt, device=dev)
            self.attn_sumprod_slice = torch.empty((H, G, B, S), dtype=dt, device=dev)

    def _tiled(self) -> bool:
        H, G, B, S, D = self.q.shape
        return bool((self.q_tile and self.q_tile < S)
                    or (self.k_tile and self.k_tile < self.n_seq_k)
                    or (self.batch_tile and tuple(self.batch_tile) != (B, G, H)))

    # ---- forward ----------------------------------------------------------
    def forward_async(self):
        if self.flash_attention:
            ops.fill(-math.inf, self.flash_logsumexp)          # sdpa.py:538
            ops.clear(self.y)                                   # sdpa.py:539
            flash_sdpa_fwd_async(self.k, self.q, self.mask, self.flash_logsumexp, self.v,
                                 self.y, self.seq_tile, self.batch_tile)
            return self.y
        if self._tiled():
            self._chain.forward()
            return self.y
        D, Sq, Sk, nb = self.head, self.n_seq, self.n_seq_k, self.batch
        ops.gemm(True, False, Sk, Sq, D, nb, self.scale, self.k, self.q, 0.0, self.attn)
        ops.clear(self.attn_maxsumexp)
        if self.mask is not None:
            ops.mask_scalar(Sk*Sq, nb, self.mask, self.val, self.attn)
        ops.maxsumexp(1, Sq*nb, Sk, self.attn, self.attn_maxsumexp)
        ops.softmax_inplace(1, Sq*nb, Sk, self.attn_maxsumexp, 1.0, self.attn)
        ops.gemm(False, False, D, Sq, Sk, nb, 1.0, self.v, self.attn, 0.0, self.y)
        return self.y

    def forward_dynamic(self, q, k, v, mask=None, kv_cache=None):
        """nntile.layer.Sdpa.forward_dynamic (sdpa.py:170-306): forward on tensors
        handed in at call time - the key/value sequence may be longer than the query
        sequence (generation against a cache) - with temporaries allocated on the
        fly; no backward.  As there, the fused path runs only when the two sequence
        lengths agree; otherwise the unfused chain.  ``mask`` is what the
        constructor takes for the chosen path.

        Beyond the reference: with ``kv_cache`` (a KVCache holding the un-replicated
        keys and values) and a single query position, the split-KV decode kernel
        reads the filled part of the cache in place; k and v are then ignored."""
        H, G, B, Sq, D = q.shape
        if kv_cache is not None and Sq == 1 and len(kv_cache) > 0:
            return kv_cache.decode(q)
        Sk = k.shape[3]
        mask_local = mask if mask is not None else self.mask
        y = torch.zeros_like(q)
        nb = H*G*B
        if self.flash_attention and Sk == Sq:
            lse = torch.full((H, G, B, Sq), -math.inf, dtype=torch.float32, device=q.device)
            if mask_local is None:
                mask_local = torch.zeros((Sq, Sq), dtype=q.dtype, device=q.device)
            flash_sdpa_fwd_async(k, q, mask_local, lse, v, y, self.seq_tile, self.batch_tile)
            return y
        attn = torch.empty((H, G, B, Sq, Sk), dtype=q.dtype, device=q.device)
        attn_max = torch.zeros((H, G, B, Sq, 2), dtype=q.dtype, device=q.device)
        ops.gemm(True, False, Sk, Sq, D, nb, sdpa_scale(D), k, q, 0.0, attn)
        if mask_local is not None:
            ops.mask_scalar(Sk*Sq, nb, mask_local, self.val, attn)
        ops.maxsumexp(1, Sq*nb, Sk, attn, attn_max)
        ops.softmax_inplace(1, Sq*nb, Sk, attn_max, 1.0, attn)
        ops.gemm(False, False, D, Sq, Sk, nb, 1.0, v, attn, 0.0, y)
        return y

    # ---- backward: dq, dk, dv are INCREMENTED, as in the reference -----------
    def backward_async(self, dy, dq, dk, dv):
        if self.flash_attention:
            flash_sdpa_bwd_async(self.k, self.q, self.v, self.y, dy, self.mask,
                                 self.flash_logsumexp, dk, dq, dv, self.seq_tile,
                                 self.batch_tile)
            return
        if self._tiled():
            self._chain.backward(dy, dq, dk, dv)
            return
        D, Sq, Sk, nb = self.head, self.n_seq, self.n_seq_k, self.batch
        dattn = torch.empty_like(self.attn)
        ops.gemm(True, False, Sk, Sq, D, nb, 1.0, self.v, dy, 0.0, dattn)
        ops.gemm(False, True, D, Sk, Sq, nb, 1.0, dy, self.attn, 1.0, dv)
        ops.sumprod_slice(1, Sq*nb, D, 1.0, self.y, dy, 0.0, self.attn_sumprod_slice)
        ops.add_slice_inplace(1, Sq*nb, Sk, -1.0, self.attn_sumprod_slice, 1.0, dattn)
        ops.multiply_inplace(dattn.numel(), 1.0, self.attn, dattn)
        if self.mask is not None:
            ops.mask_scalar(Sk*Sq, nb, self.mask, 0.0, dattn)
        ops.gemm(False, True, D, Sk, Sq, nb, self.scale, self.q, dattn, 1.0, dk)
        ops.gemm(False, False, D, Sq, Sk, nb, self.scale, self.k, dattn, 1.0, dq)


def decode_sdpa(q, Kcache, Vcache, length=None, out=None, lse_out=None, workspace=None):
    """One new token against the cache.  q: (H, G, B, 1, D) bf16; caches:
    (H, B, L, D) bf16 = Fortran [D, L, B, H].  Returns out shaped like q."""
    H, G, B, one, D = q.shape
    L = Kcache.shape[2]
    length = L if length is None else int(length)
    if out is None:
        out = torch.empty_like(q)
    if workspace is None:
        n = ops.decode_workspace_bytes(D, length, B, G, H)
        workspace = torch.empty(max(n, 16), dtype=torch.uint8, device=q.device)
    ops.decode_sdpa(D, L, length, B, G, H, q, Kcache, Vcache, out, lse_out, workspace)
    return out


class KVCache:
    """Preallocated key/value cache of one attention layer, filled in place.

    Mirrors nntile.layer.cache_utils.KVCache (wrappers/python/nntile/layer/
    cache_utils.py:118-228): ``append(k_partial, v_partial)``, ``len()``,
    ``clear()``, attributes ``k`` and ``v``.  Differences, all on purpose: the
    buffers hold the kv heads only (the reference stores what the attention layer
    has already replicated ``group`` times), ``append`` writes into the buffer at
    the current length (one kernel, no re-allocation), and there is no
    ``k_partial`` / ``v_partial`` copy of the filled part per step: ``decode``
    hands the whole buffer and the current length to the split-KV kernel.

    Torch shapes: k, v (kv_heads, batch, max_seq, head) = Fortran
    [head, max_seq, batch, kv_heads]; k_partial, v_partial (kv_heads, batch, new_seq,
    head); q (kv_heads, group, batch, 1, head)."""

    def __init__(self, max_cache_size: int, kv_heads: int, batch: int, head: int,
                 device="cuda"):
        self.max_cache_size = int(max_cache_size)
        self.k = torch.zeros((kv_heads, batch, self.max_cache_size, head), dtype=torch.bfloat16,
                             device=device)
        self.v = torch.zeros_like(self.k)
        self.k_cache_size = 0
        self.v_cache_size = 0
        self._workspace = None

    def append(self, k_partial: torch.Tensor, v_partial: torch.Tensor):
        H, B, L, D = self.k.shape
        if k_partial.shape != v_partial.shape or k_partial.shape[:2] != (H, B) \
                or k_partial.shape[3] != D:
            raise ValueError("k_partial / v_partial do not match the cache")
        n = k_partial.shape[2]
        ops.kv_cache_append(D, L, B, H, self.k_cache_size, n, k_partial.contiguous(), self.k)
        ops.kv_cache_append(D, L, B, H, self.v_cache_size, n, v_partial.contiguous(), self.v)
        self.k_cache_size += n
        self.v_cache_size += n

    def decode(self, q: torch.Tensor, out=None, lse_out=None):
        """Attention of one new query token per (batch, head) over the filled part."""
        H, G, B, one, D = q.shape
        need = ops.decode_workspace_bytes(D, max(self.k_cache_size, 1), B, G, H)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
        return decode_sdpa(q, self.k, self.v, length=self.k_cache_size, out=out,
                           lse_out=lse_out, workspace=self._workspace)

    def clear(self):
        self.k_cache_size = 0
        self.v_cache_size = 0

    def __len__(self):
        return self.k_cache_size
