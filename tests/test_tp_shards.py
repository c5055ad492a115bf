"""Tensor-parallel sharding arithmetic on the CPU: slices of the GGUF bytes dequantise to slices of the matrix, the row-split
projections concatenate and the column-split ones sum to the whole product."""
import dataclasses

import numpy as np
import pytest

from oracle import oracle as O
from vexel_b200 import capi, gguf_synth as gs, tp


def _dq(t, raw, n, k):
    return O.dequant(t, raw, n * k).reshape(n, k) if t != capi.T_F32 else np.asarray(raw, np.float32).reshape(n, k)


@pytest.mark.parametrize("t,k", [(capi.T_Q4_0, 128), (capi.T_Q4_K, 1024), (capi.T_Q6_K, 1024), (capi.T_F32, 64)])
@pytest.mark.parametrize("world", [2, 4])
def test_slices_of_the_bytes_are_slices_of_the_matrix(t, k, world):
    rng = np.random.default_rng(1)
    n = 8 * world
    w = rng.standard_normal((n, k), dtype=np.float32)
    raw = gs._QUANT[t](w) if t != capi.T_F32 else w
    full = _dq(t, raw, n, k)
    x = rng.standard_normal(k).astype(np.float32)
    rows, partial = [], np.zeros(n, np.float64)
    for r in range(world):
        a = _dq(t, tp.shard_rows(raw, r, world), n // world, k)
        assert np.array_equal(a, full[r * n // world:(r + 1) * n // world])
        rows.append(a.astype(np.float64) @ x)
        b = _dq(t, tp.shard_cols(raw, t, r, world), n, k // world)
        assert np.array_equal(b, full[:, r * k // world:(r + 1) * k // world])
        partial += b.astype(np.float64) @ x[r * k // world:(r + 1) * k // world]
    ref = full.astype(np.float64) @ x
    assert np.allclose(np.concatenate(rows), ref, rtol=0, atol=1e-12)
    assert np.allclose(partial, ref, rtol=1e-12, atol=1e-9)


def test_local_spec_and_refusals():
    spec = gs.scaled(gs.C5_LLAMA3_70B, 2, 1024, 16, 8, 128, 4096, 2048)
    loc = tp.local_spec(spec, 8)
    assert (loc.n_heads, loc.n_kv_heads, loc.ffn, loc.vocab, loc.hidden) == (2, 1, 512, 256, 1024)
    with pytest.raises(ValueError):
        tp.local_spec(spec, 16)                                   # 8 KV heads over 16 ranks
    with pytest.raises(ValueError):
        tp.local_spec(dataclasses.replace(spec, ffn=4096 + 256), 8)   # 544 columns of W2 are not whole 256-weight blocks
    # the benchmark's 70B shape splits cleanly over 8 ranks
    tp.check_divisible(gs.C5_LLAMA3_70B, 8)


def test_shard_tensor_routes_every_slot():
    spec = gs.scaled(gs.C2_LLAMA2_7B, 1, 256, 4, 4, 64, 512, 512)
    seen = {}
    for layer, slot, t, raw in gs.synth_tensors(spec, 0):
        s = tp.shard_tensor(layer, slot, t, raw, 1, 2)
        seen[(layer, slot)] = (np.asarray(raw).nbytes, np.asarray(s).nbytes)
    for (layer, slot), (whole, part) in seen.items():
        split = (layer < 0 and slot == capi.G_OUTPUT) or (layer >= 0 and slot in tp.ROW_SPLIT + tp.COL_SPLIT)
        assert part == (whole // 2 if split else whole), (layer, slot)
