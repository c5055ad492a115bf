"""Parity of the interface-level CUDA kernels (through the C ABI) against the CPU oracle.

Shapes and tolerances follow the reference's kernel tests: exact scatter (backend/metal/paged_test.go),
paged == contiguous within 1e-3 (backend/metal/paged_sdpa_test.go:23-37, 186-322), batched == per-sequence
(backend/metal/paged_batched_test.go), quantised matvec against a CPU reference (backend/metal/q4_kernel_test.go).
Dequantisation and indexing are checked bit-exactly; float reductions within the stated tolerance.
"""
import ctypes as C
import math

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import rel_l2
from vexel_b200 import capi, gguf_synth as gs

pytestmark = pytest.mark.gpu


def rnd(rng, *shape, s=0.2):
    return ((rng.random(shape, dtype=np.float32) - 0.5) * s).astype(np.float32)


# ------------------------------------------------------------------ dequantisation: bit-exact
@pytest.mark.parametrize("type_id,quant,k", [(capi.T_Q4_0, gs.quantize_q4_0, 4096), (capi.T_Q4_K, gs.quantize_q4_k, 4096),
                                             (capi.T_Q6_K, gs.quantize_q6_k, 2048)])
def test_dequantize_bit_exact(be, type_id, quant, k):
    rng = np.random.default_rng(0)
    w = rng.standard_normal((37, k)).astype(np.float32) * 0.02
    raw = quant(w)
    d_raw = be.upload(raw); d_out = be.Alloc(w.size * 4)
    be.Dequantize(type_id, d_raw, d_out, w.size)
    got = be.download(d_out, w.size)
    want = O.dequant(type_id, raw, w.size)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    be.ResetPool()


def test_dequantize_random_bytes_bit_exact(be):
    """Arbitrary block bytes (all scale bit patterns except Inf/NaN exponents) decode to the oracle's bits."""
    rng = np.random.default_rng(1)
    for type_id, bpb, epb in [(capi.T_Q4_0, 18, 32), (capi.T_Q4_K, 144, 256), (capi.T_Q6_K, 210, 256)]:
        nb = 512
        raw = rng.integers(0, 256, (nb, bpb), dtype=np.uint8)
        for off in ([0] if type_id == capi.T_Q4_0 else [0, 2] if type_id == capi.T_Q4_K else [208]):
            hi = raw[:, off + 1]
            raw[:, off + 1] = np.where((hi & 0x7C) == 0x7C, hi & 0xBF, hi)    # keep scales finite
        d_raw = be.upload(raw); d_out = be.Alloc(nb * epb * 4)
        be.Dequantize(type_id, d_raw, d_out, nb * epb)
        got = be.download(d_out, nb * epb)
        want = O.dequant(type_id, raw, nb * epb)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), type_id
        be.ResetPool()


# ------------------------------------------------------------------ elementwise / norms / rope
def test_elementwise_ops(be):
    rng = np.random.default_rng(2)
    n = 5000
    a, b = rnd(rng, n, s=8), rnd(rng, n, s=8)
    da, db, do = be.upload(a), be.upload(b), be.Alloc(n * 4)
    for name, fn, ref, exact in [("SiLU", lambda: be.SiLU(da, do, n), O.silu(a), False),
                                 ("GELU", lambda: be.GELU(da, do, n), O.gelu(a), False),
                                 ("SiLUMul", lambda: be.SiLUMul(da, db, do, n), O.silu_mul(a, b), False),
                                 ("GELUMul", lambda: be.GELUMul(da, db, do, n), O.gelu_mul(a, b), False),
                                 ("Add", lambda: be.Add(da, db, do, n), O.add(a, b), True),
                                 ("Mul", lambda: be.Mul(da, db, do, n), O.mul(a, b), True)]:
        fn()
        got = be.download(do, n)
        if exact:
            assert np.array_equal(got, ref), name
        else:   # float64 transcendental rounded once on both sides: at most 1 ulp apart
            assert np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1e-30)) < 3e-7, name
    be.ScaleBuffer(da, 1.5, n)
    assert np.array_equal(be.download(da, n), a * np.float32(1.5))
    be.ResetPool()


def test_rmsnorm_and_softmax(be):
    rng = np.random.default_rng(3)
    x = rnd(rng, 7, 2048, s=4); w = rnd(rng, 2048, s=2) + 1
    dx, dw, do = be.upload(x), be.upload(w), be.Alloc(x.nbytes)
    be.RMSNorm(dx, dw, do, 7, 2048, 1e-5)
    assert rel_l2(be.download(do, x.shape), O.rmsnorm(x, w, 1e-5)) < 1e-6
    # reference KAT (backend/cpu/rmsnorm_test.go:8-43)
    k = np.float32([[1, 2, 3, 4], [2, 2, 2, 2]]); dk = be.upload(k); dw4 = be.upload(np.ones(4, np.float32)); dk2 = be.Alloc(32)
    be.RMSNorm(dk, dw4, dk2, 2, 4, 1e-5)
    assert abs(be.download(dk2, (2, 4))[0, 0] - np.float32(1.0 / 2.73861278)) < 1e-4
    be.Softmax(dx, do, 7, 2048)
    assert rel_l2(be.download(do, x.shape), O.softmax(x)) < 1e-6
    be.ResetPool()


@pytest.mark.parametrize("neox", [False, True])
def test_rope(be, neox):
    rng = np.random.default_rng(4)
    hd, nh, nkv, T, start = 64, 8, 2, 5, 37
    q, k = rnd(rng, T * nh * hd, s=2), rnd(rng, T * nkv * hd, s=2)
    dq, dk = be.upload(q), be.upload(k)
    be.RoPE(dq, dk, hd, nh, nkv, T, start, 0, 10000.0, neox)
    wq, wk = O.rope(q, k, hd, nh, nkv, T, start, 0, 10000.0, neox)
    assert np.max(np.abs(be.download(dq, q.size) - wq)) < 1e-6 and np.max(np.abs(be.download(dk, k.size) - wk)) < 1e-6
    # partial rotation leaves the tail untouched (backend/cpu/rope_test.go:33-45); nil k is allowed
    dq2 = be.upload(np.float32([1, 0, 1, 0]))
    be.RoPE(dq2, 0, 4, 1, 0, 1, 1, 2, 10000.0, False)
    r = be.download(dq2, 4)
    assert r[2] == 1.0 and r[3] == 0.0 and not (r[0] == 1.0 and r[1] == 0.0)
    freqs = (1.0 / 10000.0 ** (np.arange(hd // 2) * 2.0 / hd)).astype(np.float32) * np.float32(0.5)
    dq3, dk3, df = be.upload(q), be.upload(k), be.upload(freqs)
    be.RoPEWithFreqs(dq3, dk3, df, hd, nh, nkv, T, start, neox)
    wq3, _ = O.rope_freqs(q, k, freqs, hd, nh, nkv, T, start, neox)
    assert np.max(np.abs(be.download(dq3, q.size) - wq3)) < 1e-6
    be.ResetPool()


def test_embedding_and_argmax(be):
    rng = np.random.default_rng(5)
    table = rnd(rng, 50, 64)
    ids = np.int32([3, 49, 0, 77, -1])
    init = np.full((5, 64), 7.0, np.float32)
    dt, di, do = be.upload(table), be.upload(ids), be.upload(init)
    be.Embedding(di, 5, dt, do, 50, 64)
    assert np.array_equal(be.download(do, (5, 64)), O.embedding(ids, table, init))   # out-of-range rows untouched
    x = rnd(rng, 32000); x[[100, 20000]] = 9.0                                        # tie: first index wins
    dx = be.upload(x)
    assert be.Argmax(dx, 32000) == 100 == O.argmax(x)
    rows = rnd(rng, 6, 1000); rows[2, 5] = rows[2, 900] = 3.0
    dr, dout = be.upload(rows), be.Alloc(24)
    be.ArgmaxRows(dr, 6, 1000, dout)
    assert list(be.download(dout, 6, np.int32)) == [O.argmax(r) for r in rows]
    be.ResetPool()


def test_matmul_f32(be):
    a = np.float32([[1, 2, 3], [4, 5, 6]]); b = np.float32([[7, 8], [9, 1], [2, 3]])
    da, db, do = be.upload(a), be.upload(b), be.Alloc(16)
    be.MatMul(da, db, do, 2, 2, 3)
    assert np.array_equal(be.download(do, 4), np.float32([31, 19, 85, 55]))          # backend/cpu/kernels_test.go:8-59
    rng = np.random.default_rng(6)
    A, B = rnd(rng, 5, 300), rnd(rng, 17, 300)
    dA, dB, dO = be.upload(A), be.upload(B), be.Alloc(5 * 17 * 4)
    be.MatMulTransposed(dA, dB, dO, 5, 17, 300)
    assert rel_l2(be.download(dO, (5, 17)), O.matmul_transposed(A, B, 5, 17, 300)) < 1e-6
    be.ResetPool()


# ------------------------------------------------------------------ quantised projections
@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (1, 4096, 4096), (3, 1000, 512), (8, 2560, 2048), (13, 384, 1024),
                                   (32, 512, 4096), (64, 1024, 11008), (100, 300, 160), (1, 32000, 2048),
                                   # thin batches on the register-streaming kernel: odd row counts, a K that is not a whole
                                   # number of 128-weight groups, more groups than one staged chunk, both tile modes
                                   (2, 4096, 11008), (4, 12288, 4096), (5, 1000, 1184), (7, 200, 4096), (8, 22016, 4096), (1, 70, 32)])
def test_matmul_q4_0(be, m, n, k):
    rng = np.random.default_rng(m * 1000 + n)
    w = rng.standard_normal((n, k)).astype(np.float32) * 0.02
    raw = gs.quantize_q4_0(w)
    a = rng.standard_normal((m, k)).astype(np.float32)
    a[0, : min(k, 7)] *= 300.0           # wide dynamic range inside a row
    da, dw, do = be.upload(a), be.upload(raw), be.Alloc(m * n * 4)
    be.MatMulQ4_0(da, dw, do, m, n, k)
    got = be.download(do, (m, n))
    want = O.matmul_q4_0(a, raw, m, n, k)
    assert rel_l2(got, want) < 1e-5, rel_l2(got, want)     # two float32 summation orders over k terms; the bar for hidden states is 1e-3
    be.ResetPool()


def test_matmul_quant_reuses_and_drops_repacked_weights(be):
    """Weights in a permanent buffer are repacked once; overwriting them through the API must be seen by the next call."""
    rng = np.random.default_rng(77)
    m, n, k = 3, 512, 1024
    a = rng.standard_normal((m, k)).astype(np.float32)
    raw1 = gs.quantize_q4_0(rng.standard_normal((n, k)).astype(np.float32) * 0.02)
    raw2 = gs.quantize_q4_0(rng.standard_normal((n, k)).astype(np.float32) * 0.02)
    dw = be.AllocPermanent(raw1.nbytes)
    be.ToDevice(dw, raw1)
    da, do = be.upload(a), be.Alloc(m * n * 4)
    want1, want2 = O.matmul_q4_0(a, raw1, m, n, k), O.matmul_q4_0(a, raw2, m, n, k)
    for _ in range(3):                                  # the second and third call run on the kept copy
        be.MatMulQ4_0(da, dw, do, m, n, k)
        assert rel_l2(be.download(do, (m, n)), want1) < 1e-5
    be.ToDevice(dw, raw2)                               # new bytes at the same address
    be.MatMulQ4_0(da, dw, do, m, n, k)
    assert rel_l2(be.download(do, (m, n)), want2) < 1e-5
    be.lib.vx_set_repack_cache(be.h, 0)                 # and with the cache off
    be.MatMulQ4_0(da, dw, do, m, n, k)
    assert rel_l2(be.download(do, (m, n)), want2) < 1e-5
    be.lib.vx_set_repack_cache(be.h, 1)
    be.Free(dw)
    be.ResetPool()


@pytest.mark.parametrize("m,n,k", [(64, 12288, 4096), (40, 22016, 4096), (17, 12300, 4096), (64, 4096, 11008)])
def test_matmul_q4_0_split_modes(be, m, n, k):
    """The persistent projection kernel with tile-aligned split-K slices (mode 1) and with the stages of all tiles cut into
    one run per CTA (mode 2, the default where the cost model prefers it): both against the oracle, at the benchmark's
    matrix shapes and with a row count that is not a multiple of the 128-row tile."""
    rng = np.random.default_rng(m + n)
    w = rng.standard_normal((n, k)).astype(np.float32) * 0.02
    raw = gs.quantize_q4_0(w)
    a = rng.standard_normal((m, k)).astype(np.float32)
    want = O.matmul_q4_0(a, raw, m, n, k)
    da, dw, do = be.upload(a), be.upload(raw), be.Alloc(m * n * 4)
    try:
        for mode in (1, 2):
            be.lib.vx_set_persistent_projections(mode)
            be.MatMulQ4_0(da, dw, do, m, n, k)
            got = be.download(do, (m, n))
            assert rel_l2(got, want) < 1e-5, (mode, rel_l2(got, want))
    finally:
        be.lib.vx_set_persistent_projections(2)
    be.ResetPool()


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (3, 200, 1024), (8, 1000, 4096), (20, 130, 512), (70, 384, 2048),
                                   # 33-64 rows: both K-quant formats on the persistent tcgen05 kernel (aligned and stream splits,
                                   # a row count that is not a multiple of the 128-row tile, the benchmark's gate/up shape)
                                   (40, 384, 2048), (64, 1000, 4096), (33, 12300, 4096), (64, 28672, 4096)])
@pytest.mark.parametrize("type_id,quant,fn", [(capi.T_Q4_K, gs.quantize_q4_k, "MatMulQ4_K"), (capi.T_Q6_K, gs.quantize_q6_k, "MatMulQ6_K")])
def test_matmul_kquants(be, type_id, quant, fn, m, n, k):
    rng = np.random.default_rng(7 + m)
    w = rng.standard_normal((n, k)).astype(np.float32) * 0.02
    raw = quant(w); a = rng.standard_normal((m, k)).astype(np.float32) + np.float32(0.3)   # non-zero mean exercises the Q4_K minima
    da, dw, do = be.upload(a), be.upload(raw), be.Alloc(m * n * 4)
    getattr(be, fn)(da, dw, do, m, n, k)
    want = O.matmul_transposed(a, O.dequant(type_id, raw, n * k).reshape(n, k), m, n, k)   # the reference's CPU route for K-quants
    assert rel_l2(be.download(do, (m, n)), want) < 1e-5
    be.ResetPool()


# ------------------------------------------------------------------ contiguous SDPA (Backend.SDPA / SDPAPrefill / SoftCap)
def test_sdpa_kats_and_random(be):
    sc = np.float32(0.5)
    def run(q, k, v, kv_len, hq, hkv, d, scale, cap=0.0):
        dq, dk, dv, do = be.upload(np.float32(q)), be.upload(np.float32(k)), be.upload(np.float32(v)), be.Alloc(hq * d * 4)
        if cap: be.SDPASoftCap(dq, dk, dv, do, kv_len, hq, hkv, d, scale, cap, kv_len * d)
        else: be.SDPA(dq, dk, dv, do, kv_len, hq, hkv, d, scale, kv_len * d)
        return be.download(do, hq * d)
    assert np.allclose(run([1, 0, 0, 0], [1, 0, 0, 0], [0.5, 0.6, 0.7, 0.8], 1, 1, 1, 4, sc), [0.5, 0.6, 0.7, 0.8], atol=1e-5)
    assert np.allclose(run([1, 0, 0, 0], [1, 0, 0, 0, 0, 1, 0, 0], [1, 1, 1, 1, 0, 0, 0, 0], 2, 1, 1, 4, sc),
                       math.exp(0.5) / (math.exp(0.5) + 1.0), atol=1e-4)
    rng = np.random.default_rng(8)
    hq, hkv, d, kv = 8, 2, 64, 300
    q, k, v = rnd(rng, hq * d, s=2), rnd(rng, hkv * kv * d, s=2), rnd(rng, hkv * kv * d, s=2)
    for cap in (0.0, 5.0):
        assert rel_l2(run(q, k, v, kv, hq, hkv, d, np.float32(1 / 8), cap), O.sdpa(q, k, v, kv, hq, hkv, d, np.float32(1 / 8), cap)) < 1e-5
    T = 70
    q, k, v = rnd(rng, T * hq * d, s=2), rnd(rng, T * hkv * d, s=2), rnd(rng, T * hkv * d, s=2)
    dq, dk, dv, do = be.upload(q), be.upload(k), be.upload(v), be.Alloc(q.nbytes)
    be.SDPAPrefill(dq, dk, dv, do, T, hq, hkv, d, np.float32(1 / 8))
    assert rel_l2(be.download(do, q.size), O.sdpa_prefill(q, k, v, T, hq, hkv, d, np.float32(1 / 8))) < 1e-5
    be.SDPAPrefillSoftCap(dq, dk, dv, do, T, hq, hkv, d, np.float32(1 / 8), 3.0)
    assert rel_l2(be.download(do, q.size), O.sdpa_prefill(q, k, v, T, hq, hkv, d, np.float32(1 / 8), 3.0)) < 1e-5
    be.ResetPool()


# ------------------------------------------------------------------ paged KV ops
def _fill_pool(be, rng, f16, n_phys, bs, hkv, d, kv_len, table):
    """Scatter kv_len tokens through ReshapePagedKV[F16]; returns (device pool, host oracle pool, k, v)."""
    k, v = rnd(rng, kv_len, hkv, d), rnd(rng, kv_len, hkv, d)
    elems = n_phys * 2 * bs * hkv * d
    host = np.zeros(elems, np.uint16 if f16 else np.float32)
    dpool = be.zeros(elems * (2 if f16 else 4))
    pos = np.arange(kv_len)
    blk, off = table[pos // bs].astype(np.int32), (pos % bs).astype(np.int32)
    dk, dv, dblk, doff = be.upload(k), be.upload(v), be.upload(blk), be.upload(off)
    fn = be.ReshapePagedKVF16 if f16 else be.ReshapePagedKV
    fn(dk, dpool, dblk, doff, kv_len, hkv, d, bs, False)
    fn(dv, dpool, dblk, doff, kv_len, hkv, d, bs, True)
    O.reshape_paged_kv(k, host, blk, off, hkv, d, bs, False)
    O.reshape_paged_kv(v, host, blk, off, hkv, d, bs, True)
    return dpool, host, k, v


@pytest.mark.parametrize("f16", [False, True])
def test_reshape_paged_kv_exact(be, f16):
    rng = np.random.default_rng(9)
    bs, hkv, d, kv_len, n_phys = 16, 4, 64, 45, 8
    table = rng.permutation(n_phys)[:3].astype(np.int32)
    dpool, host, _, _ = _fill_pool(be, rng, f16, n_phys, bs, hkv, d, kv_len, table)
    got = be.download(dpool, host.size, host.dtype)
    assert np.array_equal(got, host)        # exact scatter incl. round-to-nearest-even fp16 conversion
    be.Free(dpool); be.ResetPool()


PAGED_SHAPES = [  # (hq, hkv, d, kv_len) -- backend/metal/paged_sdpa_test.go:23-37 plus the benchmark head shapes
    (4, 4, 64, 16), (4, 4, 64, 17), (8, 2, 64, 100), (32, 8, 128, 100), (32, 32, 128, 333), (32, 4, 64, 255),
    (16, 8, 256, 70), (64, 8, 128, 2000), (32, 32, 128, 1), (12, 3, 96, 50), (8, 1, 128, 700)]


@pytest.mark.parametrize("f16", [True, False])
@pytest.mark.parametrize("hq,hkv,d,kv_len", PAGED_SHAPES)
def test_sdpa_paged_decode(be, f16, hq, hkv, d, kv_len):
    rng = np.random.default_rng(hq * 7 + kv_len)
    bs = 16; nb = (kv_len + bs - 1) // bs; n_phys = nb + 5
    table = rng.permutation(n_phys)[:nb].astype(np.int32)          # scattered blocks
    dpool, host, k, v = _fill_pool(be, rng, f16, n_phys, bs, hkv, d, kv_len, table)
    q = rnd(rng, hq * d, s=2)
    dq, dt, do = be.upload(q), be.upload(table), be.Alloc(hq * d * 4)
    scale = np.float32(1 / math.sqrt(d))
    fn = be.SDPAPagedDecodeF16 if f16 else be.SDPAPagedDecode
    fn(dq, dpool, dt, do, nb, bs, hq, hkv, d, scale, kv_len - (nb - 1) * bs)
    got = be.download(do, hq * d)
    want = O.sdpa_paged(q, host, table, 0, kv_len, bs, hq, hkv, d, scale)
    assert np.max(np.abs(got - want)) < 1e-5 and rel_l2(got, want) < 1e-5
    if not f16:   # paged == contiguous (the reference's own check, tolerance 1e-3)
        kh, vh = np.ascontiguousarray(k.transpose(1, 0, 2)), np.ascontiguousarray(v.transpose(1, 0, 2))
        assert np.max(np.abs(got - O.sdpa(q, kh, vh, kv_len, hq, hkv, d, scale))) < 1e-3
    be.Free(dpool); be.ResetPool()


def test_sdpa_paged_softcap_window_and_odd_block_size(be):
    rng = np.random.default_rng(10)
    hq, hkv, d, kv_len, bs = 16, 8, 256, 300, 16
    nb = (kv_len + bs - 1) // bs
    table = rng.permutation(nb + 2)[:nb].astype(np.int32)
    dpool, host, _, _ = _fill_pool(be, rng, True, nb + 2, bs, hkv, d, kv_len, table)
    q = rnd(rng, hq * d, s=4)
    dq, dt, do = be.upload(q), be.upload(table), be.Alloc(hq * d * 4)
    scale = np.float32(1 / 16)
    for kv_start, cap in [(0, 50.0), (300 - 128, 0.0), (173, 2.0), (299, 0.0)]:
        be.SDPAPagedDecodeEx(dq, dpool, dt, do, kv_start, kv_len, bs, hq, hkv, d, scale, cap, True)
        want = O.sdpa_paged(q, host, table, kv_start, kv_len, bs, hq, hkv, d, scale, cap)
        assert rel_l2(be.download(do, hq * d), want) < 1e-5, (kv_start, cap)
    be.Free(dpool)
    # block size 8 goes through the generic kernel
    bs = 8; nb = (kv_len + bs - 1) // bs
    table = rng.permutation(nb)[:nb].astype(np.int32)
    dpool, host, _, _ = _fill_pool(be, rng, True, nb, bs, hkv, d, kv_len, table)
    dt = be.upload(table)
    be.SDPAPagedDecodeF16(dq, dpool, dt, do, nb, bs, hq, hkv, d, scale, kv_len - (nb - 1) * bs)
    assert rel_l2(be.download(do, hq * d), O.sdpa_paged(q, host, table, 0, kv_len, bs, hq, hkv, d, scale)) < 1e-5
    be.Free(dpool); be.ResetPool()


def test_sdpa_paged_batched_equals_per_sequence(be):
    """backend/metal/paged_batched_test.go: a ragged batch through one call == each sequence alone."""
    rng = np.random.default_rng(11)
    hq, hkv, d, bs = 32, 8, 128, 16
    lens = [1, 16, 17, 100, 513, 64, 31]
    n_phys = sum((l + bs - 1) // bs for l in lens) + 4
    perm = rng.permutation(n_phys).astype(np.int32)
    elems = n_phys * 2 * bs * hkv * d
    host = np.zeros(elems, np.uint16); dpool = be.zeros(elems * 2)
    tables, dts, used = [], [], 0
    for l in lens:
        nb = (l + bs - 1) // bs
        t = perm[used:used + nb].copy(); used += nb
        k, v = rnd(rng, l, hkv, d), rnd(rng, l, hkv, d)
        pos = np.arange(l); blk, off = t[pos // bs].astype(np.int32), (pos % bs).astype(np.int32)
        dk, dv, db_, do_ = be.upload(k), be.upload(v), be.upload(blk), be.upload(off)
        be.ReshapePagedKVF16(dk, dpool, db_, do_, l, hkv, d, bs, False); be.ReshapePagedKVF16(dv, dpool, db_, do_, l, hkv, d, bs, True)
        O.reshape_paged_kv(k, host, blk, off, hkv, d, bs, False); O.reshape_paged_kv(v, host, blk, off, hkv, d, bs, True)
        tables.append(t); dts.append(be.upload(t, permanent=True))
    B = len(lens)
    q = rnd(rng, B, hq * d, s=2)
    dq, do = be.upload(q), be.Alloc(q.nbytes)
    scale = np.float32(1 / math.sqrt(d))
    be.SDPAPagedDecodeBatched(dq, dpool, dts, do, B, max(len(t) for t in tables), bs, hq, hkv, d, scale, lens, True)
    got = be.download(do, q.shape)
    d1 = be.Alloc(hq * d * 4)
    for i, l in enumerate(lens):
        want = O.sdpa_paged(q[i], host, tables[i], 0, l, bs, hq, hkv, d, scale)
        assert rel_l2(got[i], want) < 1e-5, i
        nb = len(tables[i])
        be.SDPAPagedDecodeF16(dq + i * hq * d * 4, dpool, dts[i], d1, nb, bs, hq, hkv, d, scale, l - (nb - 1) * bs)   # offset pointers are honoured
        assert np.max(np.abs(be.download(d1, hq * d) - got[i])) < 1e-5
    for p in dts: be.Free(p)
    be.Free(dpool); be.ResetPool()


def test_sdpa_paged_multiquery(be):
    """Per-query causal lengths (speculative verify): query i sees kvLens[i] positions."""
    rng = np.random.default_rng(12)
    hq, hkv, d, bs, kv_len, Q = 8, 2, 128, 16, 77, 5
    nb = (kv_len + bs - 1) // bs
    table = rng.permutation(nb + 1)[:nb].astype(np.int32)
    dpool, host, _, _ = _fill_pool(be, rng, True, nb + 1, bs, hkv, d, kv_len, table)
    q = rnd(rng, Q, hq * d, s=2)
    kv_lens = np.int32([kv_len - Q + i + 1 for i in range(Q)])
    dq, dt, dkl, do = be.upload(q), be.upload(table), be.upload(kv_lens), be.Alloc(q.nbytes)
    scale = np.float32(1 / math.sqrt(d))
    be.SDPAPagedDecodeMultiquery(dq, dpool, dt, do, dkl, nb, bs, hq, hkv, d, scale, Q, True)
    got = be.download(do, q.shape)
    for i in range(Q):
        assert rel_l2(got[i], O.sdpa_paged(q[i], host, table, 0, int(kv_lens[i]), bs, hq, hkv, d, scale)) < 1e-5
    be.Free(dpool); be.ResetPool()


def test_bad_arguments_are_reported_not_crashed(be):
    with pytest.raises(capi.VxError) as e:
        be.MatMulQ4_0(1, 2, 3, 1, 8, 33)
    assert e.value.code == capi.E_BAD_ARG
    with pytest.raises(capi.VxError):
        be.SDPAPagedDecodeF16(0, 0, 0, 0, 1, 16, 4, 4, 64, 1.0, 1)
    assert be.Alloc(0) == 0     # Alloc(<=0) yields a nil pointer
    p = be.Alloc(1024); be.ResetPool(); p2 = be.Alloc(1024)
    assert p == p2              # pooled buffers are recycled by ResetPool
    be.ResetPool()


# ------------------------------------------------------------------ sampler (pkg/sampler/sampler.go:49-218)
def _sample_params(rows):
    return np.zeros(rows, capi.SAMPLE_DTYPE)


def test_sampler_reference_cases(be):
    """The reference's own sampler tests (pkg/sampler/sampler_test.go:20-100) replayed with explicit draws."""
    logits = np.array([0.1, 0.5, 0.2, 0.9, 0.3], np.float32)
    draws = np.random.default_rng(42).random(64).astype(np.float32)
    for (t, k, p, ok) in [(0.0, 0, 0.0, {3}), (1.0, 2, 0.0, {1, 3}), (1.0, 0, 0.5, None), (1.0, 0, 0.0, None)]:
        rows = draws.size
        par = _sample_params(rows); par["temperature"] = t; par["top_k"] = k; par["top_p"] = p; par["u"] = draws
        d = be.upload(np.tile(logits, (rows, 1)))
        got = be.SampleRows(d, rows, logits.size, par)
        want = np.array([O.sample(logits, t, k, p, float(u)) for u in draws], np.int32)
        assert np.array_equal(got, want)
        if ok is not None:
            assert set(got.tolist()) <= ok
        be.ResetPool()


@pytest.mark.parametrize("n", [1000, 32000, 128256])
def test_sampler_matches_oracle(be, n):
    rng = np.random.default_rng(n)
    rows = 48
    logits = (rng.standard_normal((rows, n)) * 2.5).astype(np.float32)
    par = _sample_params(rows)
    par["temperature"] = rng.choice([0.0, 0.7, 1.0, 1.3], rows).astype(np.float32)
    par["top_k"] = rng.choice([0, 1, 40, 200, n, n + 5], rows)
    par["top_p"] = rng.choice([0.0, 0.3, 0.9, 0.95, 1.0], rows).astype(np.float32)
    par["u"] = rng.random(rows).astype(np.float32)
    par["u"][0] = 0.0
    d = be.upload(logits)
    got = be.SampleRows(d, rows, n, par)
    want = np.array([O.sample(logits[i], float(par["temperature"][i]), int(par["top_k"][i]), float(par["top_p"][i]), float(par["u"][i]))
                     for i in range(rows)], np.int32)
    assert np.array_equal(got, want), (got, want, par)
    # the rows now hold the filtered, renormalised distribution
    probs = be.download(d, rows * n).reshape(rows, n)
    for i in range(rows):
        if par["temperature"][i] == 0:
            continue
        assert abs(float(probs[i].astype(np.float64).sum()) - 1.0) < 2e-3     # float32 running sums, as in the reference
        k = int(par["top_k"][i])
        if 0 < k < n and not (0 < par["top_p"][i] < 1):
            assert np.count_nonzero(probs[i]) == k          # continuous logits: no ties at the threshold
    # the largest draw: float32 (reference) and float64 (here) running sums end a few ulps apart, so only the property
    # is compared: the pick sits where the running sum has reached the draw, or is the last-index fallback (sampler.go:216-217)
    par["u"] = np.float32(1.0) - np.float32(2.0 ** -24)
    d = be.upload(logits)
    got = be.SampleRows(d, rows, n, par)
    probs = be.download(d, rows * n).reshape(rows, n).astype(np.float64)
    for i in range(rows):
        if par["temperature"][i] == 0:
            assert got[i] == O.argmax(logits[i])
            continue
        cdf = np.cumsum(probs[i])
        assert (probs[i][got[i]] > 0 and cdf[got[i]] >= 1.0 - 1e-5) or got[i] == n - 1, (i, got[i])
    be.ResetPool()


def test_sampler_topk_keeps_ties(be):
    """Every value equal to the k-th largest survives top-k (sampler.go:127-136 compares with '<')."""
    n = 4096
    rng = np.random.default_rng(5)
    logits = rng.integers(0, 6, (8, n)).astype(np.float32)          # six levels, hundreds of ties each
    par = _sample_params(8); par["temperature"] = 1.0; par["top_k"] = 10; par["u"] = rng.random(8).astype(np.float32)
    d = be.upload(logits)
    got = be.SampleRows(d, 8, n, par)
    want = np.array([O.sample(logits[i], 1.0, 10, 0.0, float(par["u"][i])) for i in range(8)], np.int32)
    assert np.array_equal(got, want)
    probs = be.download(d, 8 * n).reshape(8, n)
    for i in range(8):
        assert np.count_nonzero(probs[i]) == np.count_nonzero(logits[i] == 5.0)
    # top-p over ties: the kept set is the top level only partly; its size is what the running sum dictates
    par["top_k"] = 0; par["top_p"] = 0.05
    d = be.upload(logits)
    got = be.SampleRows(d, 8, n, par)
    probs = be.download(d, 8 * n).reshape(8, n)
    for i in range(8):
        e = np.exp((logits[i] - 5.0).astype(np.float64)); p = (e / e.sum())
        top = p.max(); need = int(math.floor(0.05 / top)) + 1
        kept = np.nonzero(probs[i])[0]
        assert abs(kept.size - need) <= 1 and np.all(logits[i][kept] == 5.0)
        assert logits[i][got[i]] == 5.0 and probs[i][got[i]] > 0
    be.ResetPool()


def test_bounded_wait_gives_up_and_context_survives(be):
    """Failure handling of device-side waits: a kernel that waits (2 ms limit) on a barrier nobody signals returns by itself,
    the next synchronisation reports the timeout status, and the context keeps working afterwards."""
    reached = C.c_int(0)
    be._ck(be.lib.vx_selftest_bounded_wait(be.h, 2000, C.byref(reached)))
    assert reached.value == 1
    with pytest.raises(capi.VxError) as ei:
        be.Sync()
    assert ei.value.code == 6 and "wait gave up" in str(ei.value)         # VX_E_TIMEOUT
    be.Sync()                                                              # the status word was cleared: no sticky failure
    x = np.arange(1024, dtype=np.float32)
    d = be.upload(x); o = be.Alloc(4096)
    be.Add(d, d, o, 1024)
    assert np.array_equal(be.download(o, 1024), x + x)
    be.ResetPool()
