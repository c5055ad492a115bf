"""Host side of the GGUF path (no GPU): the parser against files written by the synthetic-model writer, following
pkg/gguf/gguf.go (header, metadata, tensor table, aligned data section) and runtime/config.go:388-507 (architecture switches)."""
import numpy as np
import pytest

from vexel_b200 import capi, gguf_synth as gs


def _small(arch="llama", quant="q4_0"):
    base = gs.C4_GEMMA2_9B if arch == "gemma2" else gs.C3_LLAMA3_8B
    kw = dict(sliding_window=24) if arch == "gemma2" else {}
    return gs.scaled(base, 2, 256, 4, 2, 64, 512, 320, quant=quant, **kw)


@pytest.mark.parametrize("alignment", [32, 64])
def test_tensor_table_and_data(tmp_path, alignment):
    spec = _small()
    tensors = list(gs.synth_tensors(spec, 3))
    path = str(tmp_path / "m.gguf")
    written = gs.write_gguf(path, spec, tensors, alignment=alignment)
    g = capi.GGUF(path)
    table = g.tensors()
    assert [(n, t, d) for n, t, d, _, _ in table] == written
    blob = open(path, "rb").read()
    for (name, t, dims, off, nbytes), (_, _, _, raw) in zip(table, tensors):
        assert off % alignment == 0
        raw = np.ascontiguousarray(raw).view(np.uint8).reshape(-1)
        assert nbytes == raw.size and blob[off:off + nbytes] == raw.tobytes(), name
    assert table[0][0] == "token_embd.weight" and table[0][2] == (spec.hidden, spec.vocab)      # ne[0] innermost
    assert g.meta("general.architecture") == "llama" and g.meta("llama.block_count") == "2"
    assert g.meta("tokenizer.ggml.tokens") == "[8;%d]" % spec.vocab and g.meta("no.such.key") is None
    g.close()


def test_config_llama_and_gemma2(tmp_path):
    spec = _small()
    p = str(tmp_path / "l.gguf"); gs.write_gguf(p, spec, gs.synth_tensors(spec, 1))
    g = capi.GGUF(p); cfg = g.model_config(64, 8, 128, 16); g.close()
    want = gs.model_config(spec, 64, 8, 128, 16)
    for f, _ in capi.ModelConfig._fields_:
        assert getattr(cfg, f) == getattr(want, f), f
    spec = _small("gemma2", "q6_k")
    p = str(tmp_path / "g.gguf"); gs.write_gguf(p, spec, gs.synth_tensors(spec, 1), tie_output=True)
    g = capi.GGUF(p); cfg = g.model_config(64, 8, 128, 16)
    want = gs.model_config(spec, 64, 8, 128, 16)
    for f, _ in capi.ModelConfig._fields_:
        assert getattr(cfg, f) == getattr(want, f), f
    assert cfg.geglu == 1 and cfg.post_norms == 1 and cfg.window_alternating == 1 and cfg.attn_softcap == 50.0 and cfg.final_softcap == 30.0
    assert abs(cfg.embed_scale - 16.0) < 1e-6 and cfg.sliding_window == 24
    assert "output.weight" not in [t[0] for t in g.tensors()]
    g.close()


def test_defaults_and_vocab_fallback(tmp_path):
    """No tokenizer section: the vocabulary comes from the embedding's outer dimension; missing keys take the reference's
    defaults (theta 10000 gguf.go:528-532, eps 1e-5 config.go:471-474, kv heads = heads gguf.go:516-520)."""
    spec = gs.scaled(gs.C2_LLAMA2_7B, 1, 128, 4, 4, 32, 256, 96)
    p = str(tmp_path / "d.gguf"); gs.write_gguf(p, spec, gs.synth_tensors(spec, 1), with_tokens=False)
    g = capi.GGUF(p); cfg = g.model_config(8, 2, 16, 4); g.close()
    assert cfg.vocab == 96 and cfg.n_kv_heads == 4 and cfg.head_dim == 32 and cfg.rope_theta == 10000.0
    p2 = str(tmp_path / "v2.gguf"); gs.write_gguf(p2, spec, gs.synth_tensors(spec, 1), version=2)
    capi.GGUF(p2).close()                                    # versions 2 and 3 are accepted (gguf.go:291-293)


def test_rejects_bad_files(tmp_path):
    spec = gs.scaled(gs.C2_LLAMA2_7B, 1, 128, 4, 4, 32, 256, 96)
    good = str(tmp_path / "ok.gguf"); gs.write_gguf(good, spec, gs.synth_tensors(spec, 1))
    blob = bytearray(open(good, "rb").read())

    def expect(data, text):
        p = str(tmp_path / "bad.gguf"); open(p, "wb").write(bytes(data))
        with pytest.raises(capi.GGUFError, match=text):
            capi.GGUF(p)

    b = bytearray(blob); b[0:4] = b"GGML"; expect(b, "invalid magic")
    b = bytearray(blob); b[4:8] = np.uint32(4).tobytes(); expect(b, "unsupported version")
    expect(blob[:200], "failed to read|runs past|truncated")
    expect(blob[:len(blob) - 4096], "runs past the end of the file")
    expect(blob[:10], "too short")
    with pytest.raises(capi.GGUFError, match="failed to open"):
        capi.GGUF(str(tmp_path / "missing.gguf"))
    spec_q = gs.scaled(gs.C2_LLAMA2_7B, 1, 128, 4, 4, 32, 256, 96, arch="qwen2")
    p = str(tmp_path / "q.gguf"); gs.write_gguf(p, spec_q, gs.synth_tensors(spec_q, 1))
    g = capi.GGUF(p)
    with pytest.raises(capi.GGUFError, match="qwen2"):
        g.model_config(8, 2, 16, 4)
    g.close()
