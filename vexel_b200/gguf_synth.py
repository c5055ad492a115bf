"""Synthetic GGUF-format weights for the model shapes the benchmark and tests use.

Weights are seeded N(0, sigma) values quantised into GGUF block formats (the layouts that
inference/pkg/gguf/dequant.go decodes).  Q4_0 follows the rule the benchmark configuration states:
per 32-weight block d = (signed value of largest magnitude) / -8 stored as fp16, and
q = clamp(round(x / d) + 8, 0, 15).  Q4_K / Q6_K blocks come from this module's own encoder (a
per-sub-block affine / symmetric fit): any valid encoding serves, parity is defined on the bytes.
"""
from dataclasses import dataclass, field

import numpy as np

from . import capi

T_F32, T_Q4_0, T_Q4_K, T_Q6_K = capi.T_F32, capi.T_Q4_0, capi.T_Q4_K, capi.T_Q6_K


@dataclass
class ModelSpec:
    name: str
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 1e4
    arch: str = "llama"            # "llama" | "gemma2"
    sliding_window: int = 0
    attn_softcap: float = 0.0
    final_softcap: float = 0.0
    sigma: float = 0.02
    quant: str = "q4_0"            # "q4_0" | "q4_k_m" | "q6_k"
    extra: dict = field(default_factory=dict)

    @property
    def geglu(self): return self.arch == "gemma2"
    @property
    def post_norms(self): return self.arch == "gemma2"
    @property
    def embed_scale(self): return float(np.float32(np.sqrt(np.float64(self.hidden)))) if self.arch == "gemma2" else 0.0
    @property
    def window_alternating(self): return self.arch == "gemma2"

    def kv_bytes_per_token(self):
        return 2 * self.n_layers * self.n_kv_heads * self.head_dim * 2


# the five benchmark configurations
C1_TINYLLAMA = ModelSpec("tinyllama-1.1b-q4_0", 22, 2048, 32, 4, 64, 5632, 32000)
C2_LLAMA2_7B = ModelSpec("llama2-7b-q4_0", 32, 4096, 32, 32, 128, 11008, 32000)
C3_LLAMA3_8B = ModelSpec("llama3-8b-q4_k_m", 32, 4096, 32, 8, 128, 14336, 128256, rope_theta=5e5, quant="q4_k_m")
C4_GEMMA2_9B = ModelSpec("gemma2-9b-q6_k", 42, 3584, 16, 8, 256, 14336, 256000, rms_eps=1e-6, arch="gemma2",
                         sliding_window=4096, attn_softcap=50.0, final_softcap=30.0, quant="q6_k")
C5_LLAMA3_70B = ModelSpec("llama3-70b-q4_k_m", 80, 8192, 64, 8, 128, 28672, 128256, rope_theta=5e5, sigma=0.015,
                          quant="q4_k_m")


def scaled(spec: ModelSpec, n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, **kw) -> ModelSpec:
    """A small model with the architecture switches of `spec` (small enough for CPU-checked parity tests)."""
    d = dict(spec.__dict__)
    d.update(name=spec.name + "-scaled", n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads,
             head_dim=head_dim, ffn=ffn, vocab=vocab)
    d.update(kw)
    return ModelSpec(**d)


# ---------------------------------------------------------------------------- quantisers
def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """x: float32 [..., k] with k % 32 == 0 -> uint8 [..., k/32*18] GGUF Q4_0 bytes."""
    x = np.ascontiguousarray(x, np.float32)
    k = x.shape[-1]
    assert k % 32 == 0
    b = x.reshape(-1, 32)
    idx = np.argmax(np.abs(b), axis=1)
    vmax = b[np.arange(b.shape[0]), idx]
    d = (vmax / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0)).astype(np.float32)
    q = np.clip(np.floor(b * inv[:, None] + np.float32(8.5)), 0, 15).astype(np.uint8)
    out = np.empty((b.shape[0], 18), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(*x.shape[:-1], k // 32 * 18)


def _pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """sc, mn: uint8 [n, 8] 6-bit values -> [n, 12] packed as getScaleMinK4 (dequant.go:400-409) unpacks them."""
    out = np.zeros((sc.shape[0], 12), np.uint8)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def quantize_q4_k(x: np.ndarray) -> np.ndarray:
    """Own Q4_K encoder: per 32-weight sub-block w ~ d*sc*q - dmin*m, q in [0,15], sc/m 6-bit, d/dmin fp16."""
    x = np.ascontiguousarray(x, np.float32)
    k = x.shape[-1]
    assert k % 256 == 0
    sb = x.reshape(-1, 8, 32)
    lo = np.minimum(sb.min(axis=2), 0.0)                    # min <= 0 so that -dmin*m can represent it
    hi = sb.max(axis=2)
    scale = np.maximum((hi - lo) / 15.0, 1e-12)             # per sub-block step
    mins = -lo                                              # >= 0
    d = (scale.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    dmin = (mins.max(axis=1) / 63.0).astype(np.float16).astype(np.float32)
    d = np.where(d == 0, np.float32(1e-8), d); dmin_safe = np.where(dmin == 0, np.float32(1.0), dmin)
    sc = np.clip(np.rint(scale / d[:, None]), 0, 63).astype(np.uint8)
    mn = np.clip(np.rint(mins / dmin_safe[:, None]), 0, 63).astype(np.uint8)
    eff_d = d[:, None] * sc.astype(np.float32)
    eff_m = dmin[:, None] * mn.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff_d[:, :, None] > 0, np.rint((sb + eff_m[:, :, None]) / eff_d[:, :, None]), 0)
    q = np.clip(q, 0, 15).astype(np.uint8)
    nb = sb.shape[0]
    out = np.empty((nb, 144), np.uint8)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 4:16] = _pack_scales_k4(sc, mn)
    qs = q.reshape(nb, 4, 2, 32)                            # 64-element groups: low nibble = first 32, high = next 32
    out[:, 16:] = (qs[:, :, 0, :] | (qs[:, :, 1, :] << 4)).reshape(nb, 128)
    return out.reshape(*x.shape[:-1], k // 256 * 144)


def quantize_q6_k(x: np.ndarray) -> np.ndarray:
    """Own Q6_K encoder: per 16-weight sub-block w ~ d*sc*q, q in [-32,31], sc int8, d fp16 (layout dequant.go:272-331)."""
    x = np.ascontiguousarray(x, np.float32)
    k = x.shape[-1]
    assert k % 256 == 0
    sb = x.reshape(-1, 16, 16)
    amax = np.abs(sb).max(axis=2)
    sub = amax / 31.0
    d = (sub.max(axis=1) / 127.0).astype(np.float16).astype(np.float32)
    d = np.where(d == 0, np.float32(1e-8), d)
    sc = np.clip(np.rint(sub / d[:, None]), 1, 127).astype(np.int8)
    eff = d[:, None] * sc.astype(np.float32)
    q = np.clip(np.rint(sb / eff[:, :, None]), -32, 31).astype(np.int16) + 32      # 0..63
    nb = sb.shape[0]
    v = q.reshape(nb, 2, 4, 32).astype(np.uint8)           # [half n][chunk 0..3][l]
    out = np.empty((nb, 210), np.uint8)
    ql = np.empty((nb, 2, 64), np.uint8)
    ql[:, :, 0:32] = (v[:, :, 0, :] & 0xF) | ((v[:, :, 2, :] & 0xF) << 4)
    ql[:, :, 32:64] = (v[:, :, 1, :] & 0xF) | ((v[:, :, 3, :] & 0xF) << 4)
    qh = ((v[:, :, 0, :] >> 4) & 3) | (((v[:, :, 1, :] >> 4) & 3) << 2) | (((v[:, :, 2, :] >> 4) & 3) << 4) | (((v[:, :, 3, :] >> 4) & 3) << 6)
    out[:, 0:128] = ql.reshape(nb, 128)
    out[:, 128:192] = qh.reshape(nb, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    return out.reshape(*x.shape[:-1], k // 256 * 210)


_QUANT = {T_Q4_0: quantize_q4_0, T_Q4_K: quantize_q4_k, T_Q6_K: quantize_q6_k}


def tensor_types(spec: ModelSpec):
    """GGUF type per slot for the quantisation mix of `spec` (Q4_K_M: attn_v / ffn_down / output in Q6_K)."""
    if spec.quant == "q4_0":
        proj = {s: T_Q4_0 for s in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2)}
        return proj, T_Q4_0, T_Q4_0
    if spec.quant == "q6_k":
        proj = {s: T_Q6_K for s in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2)}
        return proj, T_Q6_K, T_Q6_K
    proj = {s: T_Q4_K for s in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2)}
    proj[capi.W_WV] = T_Q6_K; proj[capi.W_W2] = T_Q6_K
    return proj, T_Q4_K, T_Q6_K     # (projections, embedding, output head)


def slot_shape(spec: ModelSpec, slot):
    qd, kvd = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
    return {capi.W_WQ: (qd, spec.hidden), capi.W_WK: (kvd, spec.hidden), capi.W_WV: (kvd, spec.hidden),
            capi.W_WO: (spec.hidden, qd), capi.W_W1: (spec.ffn, spec.hidden), capi.W_W3: (spec.ffn, spec.hidden),
            capi.W_W2: (spec.hidden, spec.ffn)}[slot]


def synth_tensors(spec: ModelSpec, seed=0):
    """Yields (layer, slot, gguf_type, raw ndarray) in a fixed order; layer -1 = globals.  Norm vectors are 1."""
    rng = np.random.default_rng(seed)
    proj_types, emb_type, out_type = tensor_types(spec)

    def qmat(n, k, t):
        w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(spec.sigma)
        return _QUANT[t](w)

    ones = np.ones(spec.hidden, np.float32)
    yield -1, capi.G_EMBED, emb_type if emb_type == T_Q4_0 else T_F32, (
        qmat(spec.vocab, spec.hidden, T_Q4_0) if emb_type == T_Q4_0
        else rng.standard_normal((spec.vocab, spec.hidden), dtype=np.float32) * np.float32(spec.sigma))
    for layer in range(spec.n_layers):
        yield layer, capi.W_ATTN_NORM, T_F32, ones
        for slot in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO):
            n, k = slot_shape(spec, slot)
            yield layer, slot, proj_types[slot], qmat(n, k, proj_types[slot])
        if spec.post_norms:
            yield layer, capi.W_POST_ATTN_NORM, T_F32, ones
        yield layer, capi.W_FFN_NORM, T_F32, ones
        for slot in (capi.W_W1, capi.W_W3, capi.W_W2):
            n, k = slot_shape(spec, slot)
            yield layer, slot, proj_types[slot], qmat(n, k, proj_types[slot])
        if spec.post_norms:
            yield layer, capi.W_POST_FFN_NORM, T_F32, ones
    yield -1, capi.G_FINAL_NORM, T_F32, ones
    yield -1, capi.G_OUTPUT, out_type, qmat(spec.vocab, spec.hidden, out_type)


def synth_weights_on_device(be, model, spec, seed, sink=None, embed_vocab=None):
    """Random weights of the model's shape and block formats, generated by CUDA kernels straight into GGUF blocks (Q4_0 by the
    benchmark's quantisation rule from N(0, sigma) draws; Q4_K / Q6_K as valid blocks with hashed payload).  The token
    embedding is kept in Q4_0 for every workload: it is read B rows per step and is not part of the timed traffic.
    sink(layer, slot, type, raw) -- optional -- receives every tensor as host data too (uint8 GGUF bytes, or the float32
    norm vectors), so that a checker can be given the same model.  embed_vocab -- rows of the embedding table when they
    differ from spec.vocab (a tensor-parallel rank: local output head, whole embedding)."""
    ones = np.ones(spec.hidden, np.float32)
    proj_types, _, out_type = tensor_types(spec)
    per_elem = {capi.T_Q4_0: 18 / 32, capi.T_Q4_K: 144 / 256, capi.T_Q6_K: 210 / 256}
    embed_vocab = embed_vocab or spec.vocab
    big = max(embed_vocab * spec.hidden, spec.ffn * spec.hidden)
    d_tmp = be.AllocPermanent(int(big * max(per_elem.values())) + 256)
    n_t = 0

    def q(layer, slot, n, k, t):
        nonlocal n_t
        if t == capi.T_Q4_0:
            be.SynthQ4_0(d_tmp, n * k, seed * 100003 + n_t, spec.sigma)
        else:
            be.SynthKQuant(d_tmp, t, n * k, seed * 100003 + n_t, spec.sigma)
        nbytes = int(n * k * per_elem[t])
        model.set_tensor(layer, slot, t, (d_tmp, nbytes))
        if sink is not None:
            sink(layer, slot, t, be.download(d_tmp, nbytes, np.uint8))
        n_t += 1

    def norm(layer, slot):
        model.set_tensor(layer, slot, capi.T_F32, ones)
        if sink is not None:
            sink(layer, slot, capi.T_F32, ones)

    q(-1, capi.G_EMBED, embed_vocab, spec.hidden, capi.T_Q4_0)
    for layer in range(spec.n_layers):
        norm(layer, capi.W_ATTN_NORM); norm(layer, capi.W_FFN_NORM)
        if spec.post_norms:
            norm(layer, capi.W_POST_ATTN_NORM); norm(layer, capi.W_POST_FFN_NORM)
        for slot in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2):
            n, k = slot_shape(spec, slot)
            q(layer, slot, n, k, proj_types[slot])
    norm(-1, capi.G_FINAL_NORM)
    q(-1, capi.G_OUTPUT, spec.vocab, spec.hidden, out_type)
    be.Free(d_tmp)
    model.finalize()


def model_config(spec: ModelSpec, max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq) -> capi.ModelConfig:
    return capi.ModelConfig(
        n_layers=spec.n_layers, hidden=spec.hidden, n_heads=spec.n_heads, n_kv_heads=spec.n_kv_heads,
        head_dim=spec.head_dim, ffn=spec.ffn, vocab=spec.vocab, rms_eps=spec.rms_eps, rope_theta=spec.rope_theta,
        rope_neox=0, geglu=int(spec.geglu), post_norms=int(spec.post_norms), embed_scale=spec.embed_scale,
        attn_softcap=spec.attn_softcap, final_softcap=spec.final_softcap, sliding_window=spec.sliding_window,
        window_alternating=int(spec.window_alternating), max_blocks=max_blocks, max_seqs=max_seqs,
        max_batch_tokens=max_batch_tokens, max_blocks_per_seq=max_blocks_per_seq)


def weight_bytes(spec: ModelSpec) -> int:
    """GGUF bytes read once per decode step: projections + output head + norm vectors."""
    proj_types, _, out_type = tensor_types(spec)
    per = {T_Q4_0: 18 / 32, T_Q4_K: 144 / 256, T_Q6_K: 210 / 256, T_F32: 4.0}
    total = 0.0
    for slot, t in proj_types.items():
        n, k = slot_shape(spec, slot)
        total += n * k * per[t]
    total *= spec.n_layers
    total += spec.vocab * spec.hidden * per[out_type]
    total += (spec.n_layers * (4 if spec.post_norms else 2) + 1) * spec.hidden * 4
    return int(total)


# ---------------------------------------------------------------------------- GGUF v3 files
_GGUF_NAMES = {  # slot -> tensor suffix under blk.N. (GetLayerTensorName, inference/pkg/gguf/loader.go:132-229)
    capi.W_ATTN_NORM: "attn_norm.weight", capi.W_WQ: "attn_q.weight", capi.W_WK: "attn_k.weight", capi.W_WV: "attn_v.weight",
    capi.W_WO: "attn_output.weight", capi.W_POST_ATTN_NORM: "post_attention_norm.weight", capi.W_FFN_NORM: "ffn_norm.weight",
    capi.W_W1: "ffn_gate.weight", capi.W_W3: "ffn_up.weight", capi.W_W2: "ffn_down.weight", capi.W_POST_FFN_NORM: "post_ffw_norm.weight"}
_GGUF_GLOBALS = {capi.G_EMBED: "token_embd.weight", capi.G_FINAL_NORM: "output_norm.weight", capi.G_OUTPUT: "output.weight"}
_MT_U32, _MT_F32, _MT_STR, _MT_ARR = 4, 6, 8, 9


def gguf_tensor_name(layer, slot):
    return _GGUF_GLOBALS[slot] if layer < 0 else "blk.%d.%s" % (layer, _GGUF_NAMES[slot])


def _gstr(s):
    b = s.encode()
    return np.uint64(len(b)).tobytes() + b


def write_gguf(path, spec: ModelSpec, tensors, alignment=32, with_tokens=True, tie_output=False, version=3, meta_spec=None):
    """Writes `tensors` (an iterable of (layer, slot, ggml type, raw ndarray), e.g. synth_tensors(spec, seed)) as a GGUF
    file with the metadata keys inference/pkg/gguf/gguf.go:503-584 reads.  with_tokens adds a tokenizer.ggml.tokens
    array of spec.vocab placeholder strings (the reference takes the vocabulary size from its length);
    tie_output drops output.weight so that loaders fall back to the embedding; meta_spec (tests of error paths) lets
    the metadata describe a different model than the tensor shapes."""
    shape_spec, spec = spec, (meta_spec or spec)
    a = spec.arch
    kv = [("general.architecture", _MT_STR, a), ("general.alignment", _MT_U32, alignment),
          (a + ".block_count", _MT_U32, spec.n_layers), (a + ".embedding_length", _MT_U32, spec.hidden),
          (a + ".attention.head_count", _MT_U32, spec.n_heads), (a + ".attention.head_count_kv", _MT_U32, spec.n_kv_heads),
          (a + ".feed_forward_length", _MT_U32, spec.ffn), (a + ".context_length", _MT_U32, 8192),
          (a + ".rope.freq_base", _MT_F32, spec.rope_theta), (a + ".attention.layer_norm_rms_epsilon", _MT_F32, spec.rms_eps),
          (a + ".attention.key_length", _MT_U32, spec.head_dim), (a + ".attention.value_length", _MT_U32, spec.head_dim)]
    if spec.sliding_window:
        kv.append((a + ".attention.sliding_window", _MT_U32, spec.sliding_window))
    if spec.attn_softcap:
        kv.append((a + ".attn_logit_softcapping", _MT_F32, spec.attn_softcap))
    if spec.final_softcap:
        kv.append((a + ".final_logit_softcapping", _MT_F32, spec.final_softcap))
    items = []
    for layer, slot, t, raw in tensors:
        if tie_output and layer < 0 and slot == capi.G_OUTPUT:
            continue
        if layer < 0:
            n, k = (1, shape_spec.hidden) if slot == capi.G_FINAL_NORM else (shape_spec.vocab, shape_spec.hidden)
        else:
            n, k = (slot_shape(shape_spec, slot) if slot in (capi.W_WQ, capi.W_WK, capi.W_WV, capi.W_WO, capi.W_W1, capi.W_W3, capi.W_W2)
                    else (1, shape_spec.hidden))
        dims = (k,) if n == 1 and raw.ndim == 1 else (k, n)                      # ne[0] is the innermost dimension
        items.append((gguf_tensor_name(layer, slot), dims, t, np.ascontiguousarray(raw).view(np.uint8).reshape(-1)))
    head = bytearray()
    head += np.uint32(0x46554747).tobytes() + np.uint32(version).tobytes()
    head += np.uint64(len(items)).tobytes() + np.uint64(len(kv) + (1 if with_tokens else 0)).tobytes()
    for key, t, v in kv:
        head += _gstr(key) + np.uint32(t).tobytes()
        head += _gstr(v) if t == _MT_STR else (np.uint32(v).tobytes() if t == _MT_U32 else np.float32(v).tobytes())
    if with_tokens:
        head += _gstr("tokenizer.ggml.tokens") + np.uint32(_MT_ARR).tobytes() + np.uint32(_MT_STR).tobytes() + np.uint64(spec.vocab).tobytes()
        head += b"".join(_gstr("t%d" % i) for i in range(spec.vocab))
    off = 0
    offsets = []
    for name, dims, t, raw in items:
        offsets.append(off)
        off = (off + raw.size + alignment - 1) // alignment * alignment
    for (name, dims, t, raw), o in zip(items, offsets):
        head += _gstr(name) + np.uint32(len(dims)).tobytes() + b"".join(np.uint64(d).tobytes() for d in dims)
        head += np.uint32(t).tobytes() + np.uint64(o).tobytes()
    pad = (-len(head)) % alignment
    with open(path, "wb") as f:
        f.write(bytes(head) + b"\0" * pad)
        pos = 0
        for (name, dims, t, raw), o in zip(items, offsets):
            f.write(b"\0" * (o - pos)); f.write(raw.tobytes()); pos = o + raw.size
    return [(name, t, dims) for name, dims, t, raw in items]
