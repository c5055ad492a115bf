"""Shared test plumbing: build the same synthetic model in the CPU oracle and in the CUDA library."""
import numpy as np

from oracle import oracle as O
from vexel_b200 import capi, gguf_synth as gs


def rel_l2(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def oracle_config(spec, max_blocks):
    return O.Config(n_layers=spec.n_layers, hidden=spec.hidden, n_heads=spec.n_heads, n_kv_heads=spec.n_kv_heads,
                    head_dim=spec.head_dim, ffn=spec.ffn, vocab=spec.vocab, rms_eps=spec.rms_eps,
                    rope_theta=spec.rope_theta, rope_neox=0, geglu=int(spec.geglu), post_norms=int(spec.post_norms),
                    embed_scale=spec.embed_scale, attn_softcap=spec.attn_softcap, final_softcap=spec.final_softcap,
                    sliding_window=spec.sliding_window, window_alternating=int(spec.window_alternating),
                    max_blocks=max_blocks, kv_f16=1)


def build_pair(be, spec, seed, max_blocks, max_seqs=8, max_batch_tokens=256, max_blocks_per_seq=64, gpu=True, cpu=True):
    """Returns (oracle model or None, gpu model or None) holding identical weights."""
    om = O.Model(oracle_config(spec, max_blocks)) if cpu else None
    gm = capi.Model(be, gs.model_config(spec, max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq)) if gpu else None
    for layer, slot, t, raw in gs.synth_tensors(spec, seed):
        if om is not None:
            if layer < 0: om.set_global(slot, t, raw)
            else: om.set_layer(layer, slot, t, raw)
        if gm is not None:
            gm.set_tensor(layer, slot, t, raw)
    if gm is not None:
        gm.finalize()
    return om, gm
