"""GPU parity of the split-KV decode kernel, through the C ABI, against the chain
the reference runs for one new token on a non-empty cache (K/V replication +
unfused chain, restated by oracle.decode_chain) and against fp64.  bf16 storage
with fp32 accumulation: <= 2e-2 relative."""
import numpy as np
import pytest
import torch

import oracle as O
from nntile_b200 import ops
from nntile_b200.sdpa import decode_sdpa, from_fortran, to_fortran

pytestmark = pytest.mark.gpu
F = np.asfortranarray


def fp64_decode(q, Kc, Vc, length):
    G = q.shape[3]
    Kr = np.repeat(O.from_bf16(Kc)[:, :length, :, None, :], G, axis=3)
    Vr = np.repeat(O.from_bf16(Vc)[:, :length, :, None, :], G, axis=3)
    return O.sdpa_fp64(O.from_bf16(q), Kr, Vr, np.zeros((length, 1), np.float32))


@pytest.mark.parametrize("D,L,length,B,G,H", [
    (128, 512, 512, 2, 4, 2),      # the fast kernel, GQA group 4
    (128, 1024, 777, 3, 4, 1),     # cache only partly filled, ragged last step
    (64, 300, 300, 2, 8, 1),       # head 64, group 8
    (128, 64, 5, 1, 1, 2),         # shorter than one warp step
    (128, 2048, 2048, 1, 2, 1),    # several chunks
    (32, 200, 150, 3, 4, 2),       # generic kernel (head 32)
    (128, 96, 96, 2, 12, 1),       # generic kernel (group > 8)
])
def test_decode_against_reference_chain(D, L, length, B, G, H):
    rng = np.random.default_rng(D + L + G)
    q = O.to_bf16(rng.standard_normal((D, 1, B, G, H)).astype(np.float32))
    Kc, Vc = (O.to_bf16(rng.standard_normal((D, L, B, H)).astype(np.float32)) for _ in range(2))
    # poison the unused tail of the cache: it must never be read into the result
    if length < L:
        Kc[:, length:] = 0x7FC0
        Vc[:, length:] = 0x7FC0
    want = O.decode_chain(q, Kc, Vc, length=length)
    a64, l64 = fp64_decode(q, Kc, Vc, length)
    lse = torch.empty((H, G, B), dtype=torch.float32, device="cuda")
    out = decode_sdpa(from_fortran(q), from_fortran(Kc), from_fortran(Vc), length, lse_out=lse)
    torch.cuda.synchronize()
    got = O.from_bf16(to_fortran(out))
    assert O.rel_err(got, O.from_bf16(want)) <= 2e-2
    assert O.rel_err(got, a64) <= 1e-2
    assert np.allclose(to_fortran(lse), l64[0], rtol=1e-3, atol=1e-3)


def test_decode_split_invariance_and_linearity():
    """Size-independent properties at a larger size: doubling V doubles the
    output; a cache whose V rows are all equal returns that row."""
    rng = np.random.default_rng(1)
    D, L, B, G, H = 128, 4096, 4, 4, 2
    q = from_fortran(O.to_bf16(rng.standard_normal((D, 1, B, G, H)).astype(np.float32)))
    Kc = from_fortran(O.to_bf16(rng.standard_normal((D, L, B, H)).astype(np.float32)))
    Vn = rng.standard_normal((D, L, B, H)).astype(np.float32)
    V1, V2 = from_fortran(O.to_bf16(Vn)), from_fortran(O.to_bf16(2*Vn))
    o1 = decode_sdpa(q, Kc, V1).float()
    o2 = decode_sdpa(q, Kc, V2).float()
    assert torch.allclose(o2, 2*o1, rtol=2e-2, atol=1e-3)
    row = rng.standard_normal(D).astype(np.float32)
    Vc = from_fortran(O.to_bf16(np.broadcast_to(row[:, None, None, None], (D, L, B, H)).copy()))
    oc = decode_sdpa(q, Kc, Vc).float()
    want = torch.from_numpy(O.from_bf16(O.to_bf16(row))).cuda()
    assert torch.allclose(oc, want.expand_as(oc), rtol=1e-2, atol=1e-2)


def test_decode_rejects_small_workspace():
    q = torch.zeros((1, 4, 1, 1, 128), dtype=torch.bfloat16, device="cuda")
    Kc = torch.zeros((1, 1, 1024, 128), dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(16, dtype=torch.uint8, device="cuda")
    from nntile_b200 import _lib
    with pytest.raises(_lib.StatusError) as e:
        decode_sdpa(q, Kc, Kc, workspace=ws)
    assert e.value.status == -4


def test_kv_cache_prefill_append_decode_loop():
    """KVCache: prefill append, then token-by-token append + decode, against the
    reference's cache semantics (append = copy at the current length) and its
    decode chain on the filled part.  Bit-exact for the cache contents."""
    from nntile_b200.sdpa import KVCache
    D, L, B, G, H = 128, 640, 2, 4, 2
    rng = np.random.default_rng(11)
    dev = torch.device("cuda", 0)
    cache = KVCache(L, H, B, D, device=dev)
    Kref = O.to_bf16(np.zeros((D, L, B, H), dtype=np.float32, order="F"))
    Vref = Kref.copy(order="F")
    n_ref = 0

    def new_kv(n):
        k = O.to_bf16(np.asfortranarray(rng.standard_normal((D, n, B, H)).astype(np.float32)))
        v = O.to_bf16(np.asfortranarray(rng.standard_normal((D, n, B, H)).astype(np.float32)))
        return k, v

    for n in (300, 1, 1, 7, 1):                  # prefill, then decode steps
        k, v = new_kv(n)
        cache.append(from_fortran(k, dev), from_fortran(v, dev))
        O.kv_cache_append(Kref, n_ref, k)
        n_ref = O.kv_cache_append(Vref, n_ref, v)
        assert len(cache) == n_ref
        assert np.array_equal(to_fortran(cache.k).view(np.uint16), Kref.view(np.uint16))
        assert np.array_equal(to_fortran(cache.v).view(np.uint16), Vref.view(np.uint16))
        q = O.to_bf16(np.asfortranarray(
            rng.standard_normal((D, 1, B, G, H)).astype(np.float32)))
        got = O.from_bf16(to_fortran(cache.decode(from_fortran(q, dev))))
        want = O.from_bf16(O.decode_chain(q, Kref, Vref, length=n_ref))
        assert O.rel_err(got, want) <= 2e-2      # bf16 storage, fp32 accumulation
    cache.clear()
    assert len(cache) == 0


def test_kv_cache_append_rejects_overflow_and_odd_shapes():
    from nntile_b200 import _lib
    D, L, B, H = 24, 10, 3, 2                    # rows of 48 bytes: element-wise path
    dev = torch.device("cuda", 0)
    cache = torch.zeros((H, B, L, D), dtype=torch.bfloat16, device=dev)
    src = torch.randn((H, B, 4, D), device=dev).to(torch.bfloat16)
    ops.kv_cache_append(D, L, B, H, 3, 4, src, cache)
    torch.cuda.synchronize()
    assert torch.equal(cache[:, :, 3:7], src)
    assert float(cache[:, :, :3].abs().sum()) == 0.0 and float(cache[:, :, 7:].abs().sum()) == 0.0
    with pytest.raises(_lib.StatusError):
        ops.kv_cache_append(D, L, B, H, 8, 4, src, cache)
