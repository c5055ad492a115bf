"""Pins the CPU oracle to the known-answer tests the reference holds for this path.

Vectors transcribed from the reference's own tests (paths relative to the reference root):
  inference/pkg/gguf/dequant_test.go:9-36     float16 table
  inference/pkg/gguf/dequant_test.go:83-119   Q4_0 nibble placement
  inference/backend/cpu/sdpa_test.go:19-164   SDPA single position / two positions / GQA / range
  inference/backend/cpu/rmsnorm_test.go:8-43  RMSNorm
  inference/backend/cpu/kernels_test.go:8-59  2x3 @ 3x2 matmul
  inference/backend/cpu/rope_test.go:10-46    RoPE styles, partial rotation
  inference/kv/paged_test.go, inference/runtime/gpu_block_pool.go:114-219  allocation order, truncate, refcounts
  inference/backend/metal/q4k_kernel_test.go:32-80, q6k_kernel_test.go:19-70  K-quant block builders
"""
import math

import numpy as np
import pytest

from oracle import oracle as O
from vexel_b200 import gguf_synth as gs


def test_f16_table():
    L = O.lib()
    for h, want in [(0x0000, 0.0), (0x3C00, 1.0), (0x4000, 2.0), (0x3800, 0.5), (0xBC00, -1.0)]:
        assert L.vo_f16_to_f32(h) == want
    assert math.isinf(L.vo_f16_to_f32(0x7C00)) and L.vo_f16_to_f32(0x7C00) > 0
    assert math.isinf(L.vo_f16_to_f32(0xFC00)) and L.vo_f16_to_f32(0xFC00) < 0
    # every finite half agrees with numpy's conversion, subnormals included
    bits = np.arange(0, 0x7C00, dtype=np.uint16)
    got = np.array([L.vo_f16_to_f32(int(b)) for b in bits[::7]], np.float32)
    assert np.array_equal(got, bits[::7].view(np.float16).astype(np.float32))


def test_f32_to_f16_rne_matches_ieee():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 6, 4000)).astype(np.float32)
    x = np.concatenate([x, np.float32([0, -0.0, 65504, 65520, 1e-8, 6e-8, 2.0 ** -24, 2.0 ** -25, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11])])
    assert np.array_equal(O.f32_to_f16_bits(x), x.astype(np.float16).view(np.uint16))


def test_q4_0_nibble_placement():
    data = np.zeros(18, np.uint8)
    data[0:2] = np.array([0x3C00], np.uint16).view(np.uint8)   # scale 1.0
    data[2] = 0x98; data[3] = 0xBA
    r = O.dequant(O.Q4_0, data, 32)
    assert r[0] == 0.0 and r[1] == 2.0 and r[16] == 1.0 and r[17] == 3.0
    assert r.size == 32


def test_q4_0_matmul_equals_dequant_then_dot_order():
    rng = np.random.default_rng(1)
    w = rng.standard_normal((5, 64)).astype(np.float32) * 0.02
    raw = gs.quantize_q4_0(w)
    a = rng.standard_normal((3, 64)).astype(np.float32)
    got = O.matmul_q4_0(a, raw, 3, 5, 64)
    deq = O.dequant(O.Q4_0, raw, 5 * 64).reshape(5, 64)
    # same products, interleaved low/high order (cpu.go:881-904): compare against that order in float32
    want = np.zeros((3, 5), np.float32)
    for i in range(3):
        for j in range(5):
            s = np.float32(0)
            for blk in range(2):
                for bi in range(16):
                    s = np.float32(s + np.float32(a[i, blk * 32 + bi] * deq[j, blk * 32 + bi]))
                    s = np.float32(s + np.float32(a[i, blk * 32 + bi + 16] * deq[j, blk * 32 + bi + 16]))
            want[i, j] = s
    assert np.array_equal(got, want)


def _q6k_block_ref(raw):
    """Python restatement of dequantizeQ6_KRef (backend/metal/q6k_kernel_test.go:73-131) for one block."""
    ql, qh, sc = raw[0:128], raw[128:192], raw[192:208].view(np.int8)
    d = np.float32(raw[208:210].view(np.float16)[0])
    out = np.zeros(256, np.float32)
    for n in range(2):
        for l in range(32):
            is_ = l // 16
            q1 = np.int8((ql[n * 64 + l] & 0xF) | (((qh[n * 32 + l] >> 0) & 3) << 4)) - 32
            q2 = np.int8((ql[n * 64 + l + 32] & 0xF) | (((qh[n * 32 + l] >> 2) & 3) << 4)) - 32
            q3 = np.int8((ql[n * 64 + l] >> 4) | (((qh[n * 32 + l] >> 4) & 3) << 4)) - 32
            q4 = np.int8((ql[n * 64 + l + 32] >> 4) | (((qh[n * 32 + l] >> 6) & 3) << 4)) - 32
            for j, q in enumerate((q1, q2, q3, q4)):
                out[n * 128 + l + 32 * j] = np.float32(np.float32(d * np.float32(sc[n * 8 + is_ + 2 * j])) * np.float32(q))
    return out


def test_q6_k_block_builder_roundtrip():
    # createQ6_KBlock (q6k_kernel_test.go:19-70): values[i] with scales 1 and d=1 dequantise to themselves
    values = ((np.arange(256) % 64) - 32).astype(np.float32)
    raw = gs.quantize_q6_k(values[None, :] * 1.0)
    got = O.dequant(O.Q6_K, raw, 256)
    assert np.array_equal(got, _q6k_block_ref(raw.ravel()))
    assert np.max(np.abs(got - values)) <= 0.6   # own encoder: within one step of the source


def test_q4_k_scale_unpack_and_dequant():
    # getScaleMinK4 round trip over all 6-bit pairs positions (dequant.go:400-409)
    rng = np.random.default_rng(2)
    sc = rng.integers(0, 64, (10, 8)).astype(np.uint8); mn = rng.integers(0, 64, (10, 8)).astype(np.uint8)
    packed = gs._pack_scales_k4(sc, mn)
    L = O.lib()
    import ctypes as C
    for r in range(10):
        for j in range(8):
            a, b = C.c_uint8(), C.c_uint8()
            L.vo_scale_min_k4(j, packed[r].ctypes.data_as(C.c_void_p), C.byref(a), C.byref(b))
            assert (a.value, b.value) == (sc[r, j], mn[r, j])
    # dequantised Q4_K reproduces N(0, 0.02) weights to the format's resolution
    w = rng.standard_normal((4, 512)).astype(np.float32) * 0.02
    deq = O.dequant(O.Q4_K, gs.quantize_q4_k(w), w.size).reshape(w.shape)
    assert np.sqrt(np.mean((deq - w) ** 2)) < 0.15 * 0.02
    # element formula d1*q - dm1 with two roundings (dequant.go:376-388)
    raw = gs.quantize_q4_k(w)[0, :144]
    d = np.float32(raw[0:2].view(np.float16)[0]); dmin = np.float32(raw[2:4].view(np.float16)[0])
    s0, m0 = raw[4] & 63, raw[8] & 63
    q0 = raw[16] & 0xF
    want = np.float32(np.float32(np.float32(d * np.float32(s0)) * np.float32(q0)) - np.float32(dmin * np.float32(m0)))
    assert deq[0, 0] == want


def test_rmsnorm_kat():
    x = np.float32([[1, 2, 3, 4], [2, 2, 2, 2]])
    out = O.rmsnorm(x, np.ones(4, np.float32), 1e-5)
    assert abs(out[0, 0] - np.float32(1.0 / 2.73861278)) < 1e-4
    assert abs(out[1, 0] - 1.0) < 1e-4


def test_matmul_kat():
    a = np.float32([[1, 2, 3], [4, 5, 6]]); b = np.float32([[7, 8], [9, 1], [2, 3]])
    assert np.array_equal(O.matmul(a, b, 2, 2, 3).ravel(), np.float32([31, 19, 85, 55]))
    assert np.array_equal(O.matmul_transposed(a, b.T.copy(), 2, 2, 3).ravel(), np.float32([31, 19, 85, 55]))


def test_rope_kat():
    q, _ = O.rope(np.float32([1, 0, 1, 0]), None, 4, 1, 0, 1, 1, 0, 10000.0, False)
    assert not (q[0] == 1.0 and q[1] == 0.0)
    assert abs(q[0] - math.cos(1.0)) < 1e-6 and abs(q[1] - math.sin(1.0)) < 1e-6       # pair 0: freq 1
    assert abs(q[2] - math.cos(0.01)) < 1e-6 and abs(q[3] - math.sin(0.01)) < 1e-6     # pair 1: freq 1e4^-0.5
    qn, _ = O.rope(np.float32([1, 1, 0, 0]), None, 4, 1, 0, 1, 1, 4, 10000.0, True)
    assert not (qn[0] == 1.0 and qn[2] == 0.0)
    qp, _ = O.rope(np.float32([1, 0, 1, 0]), None, 4, 1, 0, 1, 1, 2, 10000.0, False)
    assert qp[2] == 1.0 and qp[3] == 0.0 and not (qp[0] == 1.0 and qp[1] == 0.0)


def test_sdpa_kats():
    sc = np.float32(1.0 / math.sqrt(4))
    out = O.sdpa([1, 0, 0, 0], [1, 0, 0, 0], [0.5, 0.6, 0.7, 0.8], 1, 1, 1, 4, sc)
    assert np.allclose(out, [0.5, 0.6, 0.7, 0.8], atol=1e-5)
    out = O.sdpa([1, 0, 0, 0], [1, 0, 0, 0, 0, 1, 0, 0], [1, 1, 1, 1, 0, 0, 0, 0], 2, 1, 1, 4, sc)
    assert np.allclose(out, math.exp(0.5) / (math.exp(0.5) + 1.0), atol=1e-4)
    out = O.sdpa([1, 0, 0, 0, 0, 1, 0, 0], [1, 1, 0, 0], [0.1, 0.2, 0.3, 0.4], 1, 2, 1, 4, sc)
    assert np.allclose(out.reshape(2, 4), [[0.1, 0.2, 0.3, 0.4]] * 2, atol=1e-5)
    out = O.sdpa([1, 1], [1, 0, 0, 1, 1, 1], [1, 0, 0, 1, 0.5, 0.5], 3, 1, 1, 2, np.float32(1 / math.sqrt(2)))
    assert np.all(out >= 0) and np.all(out <= 1)


def test_argmax_first_max_wins():
    assert O.argmax(np.float32([1, 5, 5, 2])) == 1
    assert O.argmax(np.float32([-1, -1])) == 0


def test_paged_equals_contiguous():
    # the reference's paged-vs-contiguous check (backend/metal/paged_sdpa_test.go:23-37 shapes, GQA 4:1, partial last block)
    rng = np.random.default_rng(3)
    for (hq, hkv, d, kv_len) in [(4, 4, 64, 16), (8, 2, 64, 37), (32, 8, 128, 100), (4, 1, 32, 1)]:
        bs = 16; nb = (kv_len + bs - 1) // bs
        k = (rng.random((kv_len, hkv, d), dtype=np.float32) - 0.5) * 0.2
        v = (rng.random((kv_len, hkv, d), dtype=np.float32) - 0.5) * 0.2
        q = (rng.random((hq, d), dtype=np.float32) - 0.5) * 0.2
        table = rng.permutation(nb + 3)[:nb].astype(np.int32)       # scattered physical blocks
        pool = np.zeros((nb + 3) * 2 * bs * hkv * d, np.float32)
        pos = np.arange(kv_len)
        O.reshape_paged_kv(k, pool, table[pos // bs], pos % bs, hkv, d, bs, False)
        O.reshape_paged_kv(v, pool, table[pos // bs], pos % bs, hkv, d, bs, True)
        scale = np.float32(1 / math.sqrt(d))
        got = O.sdpa_paged(q, pool, table, 0, kv_len, bs, hq, hkv, d, scale)
        kh = np.ascontiguousarray(k.transpose(1, 0, 2)); vh = np.ascontiguousarray(v.transpose(1, 0, 2))
        want = O.sdpa(q, kh, vh, kv_len, hq, hkv, d, scale)
        assert np.array_equal(got, want)     # same arithmetic, only the addressing differs


def test_block_pool_allocation_order():
    # runtime/gpu_block_pool.go:114-116, 200-219: ascending free list popped from the end, LIFO reuse
    p = O.Pool(2, 1, 8, 16, 10, f16=True)
    p.create_seq(1)
    k = np.zeros((17, 8), np.float32)
    assert p.store_kv(0, 1, 0, k, k, 17) == 0
    assert list(p.table(0, 1)) == [9, 8]
    assert p.free_blocks(0) == 8 and p.free_blocks(1) == 10 and p.seq_len(1) == 17
    p.create_seq(2)
    assert p.store_kv(0, 2, 0, k, k, 1) == 0 and list(p.table(0, 2)) == [7]
    p.truncate(1, 16)                      # drops logical block 1 (physical 8)
    assert list(p.table(0, 1)) == [9] and p.seq_len(1) == 16
    assert p.store_kv(0, 2, 1, k, k, 16) == 0 and list(p.table(0, 2)) == [7, 8]   # freed block comes back first
    p.delete_seq(2)                        # released in table order: 7 then 8 -> next pops 8, then 7
    p.create_seq(3)
    assert p.store_kv(0, 3, 0, k, k, 17) == 0 and list(p.table(0, 3)) == [8, 7]
    # exhaustion is an error, not a crash (gpu_block_pool.go:200-204)
    p.create_seq(4)
    big = np.zeros((16 * 8, 8), np.float32)
    assert p.store_kv(0, 4, 0, big, big, 16 * 8) == -2
    # prefix sharing bumps refcounts (gpu_block_pool.go:572-607): deleting one owner keeps the block
    p2 = O.Pool(1, 1, 8, 16, 4)
    p2.create_seq(1); p2.create_seq(2)
    p2.store_kv(0, 1, 0, k, k, 16)
    assert p2.share(1, 2, 16) == 0 and list(p2.table(0, 2)) == [3] and p2.seq_len(2) == 16
    p2.delete_seq(1)
    assert p2.free_blocks(0) == 3
    p2.delete_seq(2)
    assert p2.free_blocks(0) == 4


def test_f16_pool_store_rounds_to_nearest_even():
    p = O.Pool(1, 1, 8, 16, 2, f16=True)
    p.create_seq(1)
    k = np.float32([[1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11, 0.1, -0.1, 65504, 1e-8, 0, -0.0]])
    p.store_kv(0, 1, 0, k, k, 1)
    data = p.layer_data(0)
    base = 1 * 2 * 16 * 8      # block 1 (first pop), K part, offset 0
    assert np.array_equal(data[base:base + 8], k.astype(np.float16).view(np.uint16).ravel())


def test_sampler_semantics():
    logits = np.float32([0.0, 1.0, 2.0, 3.0])
    assert O.sample(logits, 0.0, 0, 0.0, 0.5) == 3                       # temperature 0 = greedy
    assert O.sample(logits, 1.0, 1, 0.0, 0.999) == 3                     # top-1
    p = np.exp(logits - 3); p /= p.sum()
    assert O.sample(logits, 1.0, 0, 0.0, 0.0) == 0                       # r < p[0]
    assert O.sample(logits, 1.0, 0, 0.0, float(p[0] + p[1] / 2)) == 1    # inverse CDF in index order
    assert O.sample(logits, 1.0, 0, 0.5, 0.0) == 3                       # nucleus {3} (p3=0.64 > 0.5)


def test_q4_0_quantiser_rule():
    x = np.zeros(32, np.float32); x[5] = -0.8; x[6] = 0.35
    raw = gs.quantize_q4_0(x)
    d = np.float32(raw[0:2].view(np.float16)[0])
    assert d == np.float32(0.1).astype(np.float16)                       # -0.8 / -8
    deq = O.dequant(O.Q4_0, raw, 32)
    assert deq[5] == np.float32(d * np.float32(-8)) and abs(deq[6] - 0.35) <= 0.05 + 1e-3 and deq[0] == 0


@pytest.mark.parametrize("T", [1, 5])
def test_model_forward_runs_and_is_deterministic(T):
    from tests.helpers import build_pair
    spec = gs.scaled(gs.C1_TINYLLAMA, 2, 128, 4, 2, 32, 256, 512)
    om, _ = build_pair(None, spec, 0, 16, gpu=False)
    toks = np.arange(T, dtype=np.int32) + 3
    a, ha = om.forward(1, toks, 0, want_hidden=True)
    om2, _ = build_pair(None, spec, 0, 16, gpu=False)
    b, hb = om2.forward(1, toks, 0, want_hidden=True)
    assert np.array_equal(a, b) and np.array_equal(ha, hb) and np.isfinite(a).all()
    assert om.pool.seq_len(1) == T and list(om.pool.table(0, 1)) == [15]
