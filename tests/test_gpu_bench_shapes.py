"""Parity of the batched decode step at the shapes the benchmark times, against the CPU oracle.

The other model tests use narrow layers (hidden 256) so that the oracle can run many steps; these build one or two layers
at the real widths of the benchmark configurations -- the Llama-2-7B shape with 64 sequences at contexts ~U[128, 2048] on
shuffled physical blocks is exactly what bench.py times -- and compare ONE full step: block tables and slot mapping
bit-exact, per-layer hidden states and logits within rel-L2 1e-3, greedy tokens >= 99 %.  Weights come from the
benchmark's own device generator (the oracle is handed the same GGUF bytes), the KV cache from its synthetic fill (the
oracle stores the same fp16 values through its own allocator, after being given the same free-list order).
"""
import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import oracle_config, rel_l2
from vexel_b200 import capi, gguf_synth as gs

pytestmark = pytest.mark.gpu

HIDDEN_TOL = 1e-3


def build_pair_like_the_benchmark(be, spec, seed, ctx, shuffle_seed, max_rows, extra_tokens=8):
    """(oracle model, gpu model) with device-generated weights, a shuffled free list and ctx[i] tokens of synthetic KV."""
    B = len(ctx)
    per_seq = int(max(ctx) + extra_tokens) // 16 + 2
    max_blocks = int(sum((int(c) + extra_tokens) // 16 + 2 for c in ctx) + 8)
    gm = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs=B, max_batch_tokens=max_rows, max_blocks_per_seq=per_seq))
    om = O.Model(oracle_config(spec, max_blocks))

    def sink(layer, slot, t, raw):
        if layer < 0: om.set_global(slot, t, raw)
        else: om.set_layer(layer, slot, t, raw)

    gs.synth_weights_on_device(be, gm, spec, seed, sink=sink)
    gm.shuffle_free_list(shuffle_seed)
    om.pool.set_free_list(gm.free_list())                       # both sides now hand out blocks in the same (shuffled) order
    for i in range(B):
        gm.seq_fill_synthetic(i + 1, int(ctx[i]), seed=1000 + i)
    kvd = spec.n_kv_heads * spec.head_dim
    tables = [gm.block_table(i + 1) for i in range(B)]
    for i in range(B):
        om.pool.create_seq(i + 1)
    for layer in range(spec.n_layers):
        p, nbytes = gm.pool_layer(layer)
        dev = be.download(p, nbytes // 2, np.uint16).reshape(max_blocks, 2 * 16 * kvd)
        ora = om.pool.layer_data(layer).reshape(max_blocks, 2 * 16 * kvd)
        for i in range(B):
            assert om.pool.store_kv(layer, i + 1, 0, None, None, int(ctx[i])) == 0     # the oracle's own allocator picks the pages
            t = om.pool.table(layer, i + 1)
            assert np.array_equal(t, tables[i])                                        # ... the same ones, in the same order
            ora[t] = dev[t]                                                            # fp16 pages copied bit for bit
        del dev
    return om, gm


def check_step(be, spec, om, gm, ids, q_lens, positions, rng):
    """One packed step against the oracle fed the same tokens sequence by sequence."""
    toks = [rng.integers(0, spec.vocab, q).astype(np.int32) for q in q_lens]
    gm.set_capture(True)
    out, logits = gm.decode_step(ids, np.concatenate(toks), positions, q_lens=q_lens, want_logits=True)
    rows = int(sum(q_lens))
    h = gm.get_capture(rows)
    cu, slot_map, kv_len = gm.get_packing(len(ids), rows)
    assert list(cu) == list(np.concatenate([[0], np.cumsum(q_lens)]))
    worst_h = worst_l = 0.0
    agree = 0
    row = 0
    for s, q, t, p0 in zip(ids, q_lens, toks, positions):
        wl, wh = om.forward(int(s), t, int(p0), all_logits=True, want_hidden=True)
        if spec.final_softcap > 0:
            O.lib().vo_final_softcap(wl.ctypes.data, wl.size, spec.final_softcap)
        for l in range(spec.n_layers + 1):
            worst_h = max(worst_h, rel_l2(h[l, row:row + q], wh[l]))
        worst_l = max(worst_l, rel_l2(logits[row:row + q], wl))
        agree += sum(int(out[row + j]) == O.argmax(wl[j]) for j in range(q))
        tab = om.pool.table(0, int(s))
        assert np.array_equal(gm.block_table(int(s)), tab)                      # block tables bit-exact, new pages included
        for j in range(q):
            pos = p0 + j
            assert slot_map[row + j] == tab[pos // 16] * 16 + pos % 16          # slot mapping bit-exact
            assert kv_len[row + j] == pos + 1
        row += q
    assert worst_h < HIDDEN_TOL and worst_l < HIDDEN_TOL, (worst_h, worst_l)
    assert agree / rows >= 0.99, (agree, rows)
    gm.set_capture(False)
    return worst_h, worst_l


def test_llama2_7b_shape_b64_step(be):
    """Two layers of the headline configuration: hidden 4096, 32/32 heads of 128, FFN 11008, vocab 32000, Q4_0, 64 sequences
    at contexts ~U[128, 2048], shuffled blocks: the tcgen05 projections with their split-K, the CUDA-core paged attention
    with its work list and fused merge, packing and KV append exactly as the benchmark runs them."""
    spec = gs.scaled(gs.C2_LLAMA2_7B, 2, 4096, 32, 32, 128, 11008, 32000)
    rng = np.random.default_rng(2)
    ctx = rng.integers(128, 2049, 64)
    ctx[:4] = [128, 2048, 1023, 1024]                                           # extremes and both sides of a page boundary
    om, gm = build_pair_like_the_benchmark(be, spec, seed=0, ctx=ctx, shuffle_seed=3, max_rows=64)
    ids = np.arange(1, 65, dtype=np.int64)
    wh, wl = check_step(be, spec, om, gm, ids, [1] * 64, [int(c) for c in ctx], rng)
    # a second step (teacher-forced with fresh tokens): sequence 4 has just opened a new page
    wh2, wl2 = check_step(be, spec, om, gm, ids, [1] * 64, [int(c) + 1 for c in ctx], rng)
    print(f"llama2-7b shape, B=64: worst per-layer hidden rel-L2 {max(wh, wh2):.2e}, logits {max(wl, wl2):.2e}")
    gm.close()


def test_llama3_8b_shape_b64_step(be):
    """One layer of the grouped-query Q4_K_M configuration: 32/8 heads of 128, FFN 14336, vocab 128256 (Q4_K projections with
    attn_v / ffn_down / output in Q6_K), 64 sequences at contexts ~U[128, 2048]: the tensor-core attention for groups of four
    and both K-quant projection kernels at their real widths."""
    spec = gs.scaled(gs.C3_LLAMA3_8B, 1, 4096, 32, 8, 128, 14336, 128256)
    rng = np.random.default_rng(5)
    ctx = rng.integers(128, 2049, 64)
    om, gm = build_pair_like_the_benchmark(be, spec, seed=1, ctx=ctx, shuffle_seed=7, max_rows=64)
    wh, wl = check_step(be, spec, om, gm, np.arange(1, 65, dtype=np.int64), [1] * 64, [int(c) for c in ctx], rng)
    print(f"llama3-8b shape, B=64: worst per-layer hidden rel-L2 {wh:.2e}, logits {wl:.2e}")
    gm.close()


def test_gemma2_9b_shape_b32_step_with_verify_row(be):
    """Two layers (one global, one with the 4096-token window) of the Gemma-2 configuration: 16/8 heads of 256, GeGLU FFN
    14336, vocab 256000, Q6_K, soft-caps 50 / 30, post-norms; 32 sequences at contexts ~U[1024, 8192], one of which verifies
    five tokens at once (input + 4 drafts, runtime/decode.go:1446-1569)."""
    spec = gs.scaled(gs.C4_GEMMA2_9B, 2, 3584, 16, 8, 256, 14336, 256000)
    rng = np.random.default_rng(6)
    ctx = rng.integers(1024, 8193, 32)
    ctx[0], ctx[1] = 8192, 4090                                                 # the longest context; one that crosses the window in the step
    om, gm = build_pair_like_the_benchmark(be, spec, seed=2, ctx=ctx, shuffle_seed=9, max_rows=40)
    q_lens = [1] * 32; q_lens[1] = 5; q_lens[7] = 5
    wh, wl = check_step(be, spec, om, gm, np.arange(1, 33, dtype=np.int64), q_lens, [int(c) for c in ctx], rng)
    print(f"gemma2-9b shape, B=32 + verify rows: worst per-layer hidden rel-L2 {wh:.2e}, logits {wl:.2e}")
    gm.close()


def test_llama3_70b_shape_b32_step(be):
    """One layer of the 70B configuration: hidden 8192, 64/8 heads of 128, FFN 28672, vocab 128256, Q4_K_M; 32 sequences (one
    replica's share of the batch of 256) at contexts ~U[512, 8192]: groups of eight query heads per KV head."""
    spec = gs.scaled(gs.C5_LLAMA3_70B, 1, 8192, 64, 8, 128, 28672, 128256)
    rng = np.random.default_rng(7)
    ctx = rng.integers(512, 8193, 32)
    om, gm = build_pair_like_the_benchmark(be, spec, seed=3, ctx=ctx, shuffle_seed=11, max_rows=32)
    wh, wl = check_step(be, spec, om, gm, np.arange(1, 33, dtype=np.int64), [1] * 32, [int(c) for c in ctx], rng)
    print(f"llama3-70b shape, B=32: worst per-layer hidden rel-L2 {wh:.2e}, logits {wl:.2e}")
    gm.close()
