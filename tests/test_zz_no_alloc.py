"""The allocation-free decode-attention entry point gives the same answer as the regular one.

Some users of the library cannot allocate device memory at the moment they attend (the KV pool owns all of HBM, or the call
sits in a section where the allocator must not be entered).  vx_sdpa_paged_decode_f16_noalloc keeps its split-K scratch in a
fixed array inside the library; this test calls it through the C ABI twice in a row on different inputs -- the array keeps
the first call's contents -- and compares with vx_sdpa_paged_decode_f16 and with the CPU oracle's paged attention.  It is
collected last so that a run stopping at the first failure has already run every other test, and it needs nothing from
the other tests.
"""
import math

import numpy as np
import pytest

from oracle import oracle as O
from vexel_b200 import capi

pytestmark = pytest.mark.gpu


def _case(be, rng, hq, hkv, d, kv_len, bs=16):
    nb = (kv_len + bs - 1) // bs
    n_phys = nb + 3
    table = rng.permutation(n_phys)[:nb].astype(np.int32)
    pool = ((rng.random(n_phys * 2 * bs * hkv * d, dtype=np.float32) - 0.5) * 0.5).astype(np.float16)
    q = ((rng.random(hq * d, dtype=np.float32) - 0.5) * 2).astype(np.float32)
    dpool, dq, dt = be.upload(pool, permanent=True), be.upload(q, permanent=True), be.upload(table, permanent=True)
    d_ref, d_new = be.AllocPermanent(hq * d * 4), be.AllocPermanent(hq * d * 4)
    scale = np.float32(1 / math.sqrt(d))
    til = kv_len - (nb - 1) * bs
    be.SDPAPagedDecodeF16(dq, dpool, dt, d_ref, nb, bs, hq, hkv, d, scale, til)
    be.SDPAPagedDecodeF16NoAlloc(dq, dpool, dt, d_new, nb, bs, hq, hkv, d, scale, til)
    ref, new = be.download(d_ref, hq * d), be.download(d_new, hq * d)
    for p in (dpool, dq, dt, d_ref, d_new):
        be.Free(p)
    want = O.sdpa_paged(q, pool.view(np.uint16), table, 0, kv_len, bs, hq, hkv, d, float(scale))
    return ref, new, want


def test_noalloc_matches_regular_entry_point_twice():
    be = capi.Backend(0)        # its own context: the test must pass alone in a fresh process and after the others
    rng = np.random.default_rng(123)
    # two calls in a row; the second is smaller, so stale work items and partials of the first stay in the array
    for hq, hkv, d, kv_len in [(32, 8, 128, 1500), (8, 2, 64, 70)]:
        ref, new, want = _case(be, rng, hq, hkv, d, kv_len)
        assert np.isfinite(new).all()
        assert np.max(np.abs(new - ref)) < 1e-5 and np.linalg.norm(new - ref) / np.linalg.norm(ref) < 1e-5
        assert np.linalg.norm(new - want) / np.linalg.norm(want) < 1e-5          # and both agree with the CPU oracle
    # shapes outside the fast kernels (32-token pages; head_dim 96) take the generic kernel over the same fixed scratch
    for hq, hkv, d, kv_len, bs in [(8, 2, 64, 333, 32), (6, 3, 96, 200, 16)]:
        ref, new, want = _case(be, rng, hq, hkv, d, kv_len, bs)
        assert np.linalg.norm(new - ref) / np.linalg.norm(ref) < 1e-5
        assert np.linalg.norm(new - want) / np.linalg.norm(want) < 1e-5
    # a block table beyond the stated maximum (65536 blocks) is refused with a clear error, not truncated
    with pytest.raises(capi.VxError) as e:
        be.SDPAPagedDecodeF16NoAlloc(1, 1, 1, 1, 70000, 16, 8, 2, 64, 1.0, 1)
    assert e.value.code == capi.E_BAD_ARG
    # so is a head configuration whose single split-K chunk would not fit the fixed array, and an oversize page
    with pytest.raises(capi.VxError) as e:
        be.SDPAPagedDecodeF16NoAlloc(1, 1, 1, 1, 4, 16, 8192, 1, 256, 1.0, 1)
    assert e.value.code == capi.E_BAD_ARG and "scratch" in str(e.value)
    with pytest.raises(capi.VxError) as e:
        be.SDPAPagedDecodeF16NoAlloc(1, 1, 1, 1, 4, 32768, 8, 2, 64, 1.0, 1)
    assert e.value.code == capi.E_BAD_ARG
    be.close()
