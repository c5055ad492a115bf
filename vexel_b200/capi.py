"""ctypes binding of include/vexel_cuda.h.

`Backend` mirrors the method names of the reference's backend interfaces
(inference/backend/backend.go: Backend, QuantizedMatMul, PagedKVOps, ArgmaxOps, ...), so tests written
against it read like the reference's own kernel tests.  `Model` wraps the batched decode fast path.
Nothing here computes: every call goes through the C ABI into CUDA kernels.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("VEXEL_CUDA_LIB") or os.path.join(_HERE, "libvexel_cuda.so")     # the override loads another build of the same library

OK, E_BAD_ARG, E_CUDA, E_OOM, E_OOM_BLOCKS, E_NO_SEQ, E_TIMEOUT, E_UNSUPPORTED = range(8)
T_F32, T_F16, T_Q4_0, T_Q4_K, T_Q6_K = 0, 1, 2, 12, 14
(W_ATTN_NORM, W_WQ, W_WK, W_WV, W_WO, W_POST_ATTN_NORM, W_FFN_NORM, W_W1, W_W3, W_W2, W_POST_FFN_NORM) = range(11)
G_EMBED, G_FINAL_NORM, G_OUTPUT = 0, 1, 2


class VxError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"vexel_cuda status {code}: {msg}")
        self.code = code


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("rope_neox", C.c_int), ("geglu", C.c_int),
        ("post_norms", C.c_int), ("embed_scale", C.c_float), ("attn_softcap", C.c_float),
        ("final_softcap", C.c_float), ("sliding_window", C.c_int), ("window_alternating", C.c_int),
        ("max_blocks", C.c_int), ("max_seqs", C.c_int), ("max_batch_tokens", C.c_int), ("max_blocks_per_seq", C.c_int)]


class SchedConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("max_batch_size", "max_sequences", "max_tokens", "eos_token")] + [
        ("temperature", C.c_float), ("top_k", C.c_int), ("top_p", C.c_float), ("seed", C.c_uint64)]


class SchedMetrics(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("active_sequences", "completed_sequences", "total_tokens", "prefill_tokens", "decode_tokens")] + [
        ("prefill_seconds", C.c_double), ("decode_seconds", C.c_double)]


_vp, _i, _i64, _f, _u64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64, C.c_size_t
_D = C.c_uint64  # vx_dptr

# name -> argtypes (every function returns int unless listed in _RESTYPE)
STEP_LAST_ROWS, STEP_PROMPT_ROWS = 1, 2
SAMPLE_DTYPE = np.dtype([("temperature", np.float32), ("top_k", np.int32), ("top_p", np.float32), ("u", np.float32)])

SIGNATURES = {
    "vx_init": [_i, C.POINTER(_vp)], "vx_destroy": [_vp], "vx_last_error": [_vp], "vx_device_index": [_vp],
    "vx_alloc": [_vp, _sz, C.POINTER(_D)], "vx_alloc_permanent": [_vp, _sz, C.POINTER(_D)], "vx_free": [_vp, _D],
    "vx_reset_pool": [_vp], "vx_h2d": [_vp, _D, _vp, _sz], "vx_d2h": [_vp, _vp, _D, _sz], "vx_d2d": [_vp, _D, _D, _sz],
    "vx_memset": [_vp, _D, _i, _sz], "vx_sync": [_vp],
    "vx_matmul_f32": [_vp, _D, _D, _D, _i, _i, _i], "vx_matmul_f32_t": [_vp, _D, _D, _D, _i, _i, _i],
    "vx_rmsnorm": [_vp, _D, _D, _D, _i, _i, _f],
    "vx_rope": [_vp, _D, _D, _i, _i, _i, _i, _i, _i, _f, _i],
    "vx_silu": [_vp, _D, _D, _i], "vx_silu_mul": [_vp, _D, _D, _D, _i], "vx_softmax": [_vp, _D, _D, _i, _i],
    "vx_add": [_vp, _D, _D, _D, _i], "vx_mul": [_vp, _D, _D, _D, _i],
    "vx_embedding": [_vp, _D, _i, _D, _D, _i, _i],
    "vx_sdpa": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _f, _i],
    "vx_sdpa_prefill": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _f],
    "vx_matmul_q4_0": [_vp, _D, _D, _D, _i, _i, _i], "vx_matmul_q4_k": [_vp, _D, _D, _D, _i, _i, _i],
    "vx_matmul_q6_k": [_vp, _D, _D, _D, _i, _i, _i],
    "vx_argmax": [_vp, _D, _i, C.POINTER(_i)], "vx_argmax_rows": [_vp, _D, _i, _i, _D],
    "vx_gelu": [_vp, _D, _D, _i], "vx_gelu_mul": [_vp, _D, _D, _D, _i], "vx_scale": [_vp, _D, _f, _i],
    "vx_sdpa_softcap": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _f, _f, _i],
    "vx_sdpa_prefill_softcap": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _f, _f],
    "vx_rope_freqs": [_vp, _D, _D, _D, _i, _i, _i, _i, _i, _i],
    "vx_dequantize": [_vp, _i, _D, _D, _i64],
    "vx_reshape_paged_kv": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i],
    "vx_reshape_paged_kv_f16": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i],
    "vx_sdpa_paged_decode": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i, _f, _i],
    "vx_sdpa_paged_decode_f16": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i, _f, _i],
    "vx_sdpa_paged_decode_f16_noalloc": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i, _f, _i],
    "vx_sdpa_paged_decode_batched": [_vp, _D, _D, C.POINTER(_D), _D, _i, _i, _i, _i, _i, _i, _f, C.POINTER(_i), _i],
    "vx_sdpa_paged_decode_multiquery": [_vp, _D, _D, _D, _D, _D, _i, _i, _i, _i, _i, _f, _i, _i],
    "vx_sdpa_paged_decode_ex": [_vp, _D, _D, _D, _D, _i, _i, _i, _i, _i, _i, _f, _f, _i],
    "vx_model_create": [_vp, C.POINTER(ModelConfig), C.POINTER(_vp)], "vx_model_destroy": [_vp],
    "vx_model_set_tensor": [_vp, _i, _i, _i, _vp, _sz, _i], "vx_model_finalize": [_vp],
    "vx_seq_create": [_vp, _i64], "vx_seq_delete": [_vp, _i64], "vx_seq_truncate": [_vp, _i64, _i],
    "vx_seq_share": [_vp, _i64, _i64, _i], "vx_seq_len": [_vp, _i64, C.POINTER(_i)],
    "vx_seq_block_table": [_vp, _i64, _vp, _i, C.POINTER(_i)],
    "vx_pool_stats": [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)],
    "vx_pool_layer_ptr": [_vp, _i, C.POINTER(_D), C.POINTER(_sz)],
    "vx_pool_free_list": [_vp, _vp, _i, C.POINTER(_i)],
    "vx_seq_fill_synthetic": [_vp, _i64, _i, C.c_uint32],
    "vx_decode_step": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "vx_decode_step_ex": [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp],
    "vx_model_get_config": [_vp, _vp],
    "vx_gguf_open": [C.c_char_p, C.POINTER(_vp)], "vx_gguf_close": [_vp], "vx_gguf_error": [_vp], "vx_gguf_tensor_count": [_vp],
    "vx_gguf_tensor_info": [_vp, _i, C.c_char_p, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_u64), C.POINTER(_u64), C.POINTER(_u64)],
    "vx_gguf_meta": [_vp, C.c_char_p, C.c_char_p, _i], "vx_gguf_model_config": [_vp, _vp], "vx_model_load_gguf": [_vp, _vp],
    "vx_decode_step_sampled": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp],
    "vx_sample_rows": [_vp, _D, _i, _i, _vp, _vp],
    "vx_prefill": [_vp, _i64, _vp, _i, _i, _vp, _vp],
    "vx_prefill_sampled": [_vp, _i64, _vp, _i, _i, _vp, _vp, _vp],
    "vx_decode_run": [_vp, _i, _vp, _vp, _vp, _i, _vp, C.POINTER(_f)],
    "vx_model_set_capture": [_vp, _i], "vx_model_get_capture": [_vp, _vp, _sz],
    "vx_model_get_packing": [_vp, _vp, _vp, _vp, _i, _i],
    "vx_model_counters": [_vp, C.POINTER(_u64), C.POINTER(_u64)],
    "vx_model_graph_stats": [_vp, C.POINTER(_u64), C.POINTER(_u64)],
    "vx_model_kernel_time": [_vp, _i, _i, C.POINTER(_f), C.POINTER(_u64)],
    "vx_synth_kquant": [_vp, _D, _i, _i64, _u64, _f],
    "vx_selftest_bounded_wait": [_vp, _i, C.POINTER(_i)],
    "vx_set_graphs": [_i],
    "vx_synth_q4_0": [_vp, _D, _i64, _u64, _f],
    "vx_synth_kquant": [_vp, _D, _i, _i64, _u64, _f],
    "vx_pool_shuffle_free_list": [_vp, C.c_uint32], "vx_model_weight_bytes": [_vp, C.POINTER(_u64)],
    "vx_set_persistent_projections": [_i], "vx_set_thin_batch_projections": [_i], "vx_debug_skip": [_i], "vx_set_repack_cache": [_vp, _i],
    "vx_tp_unique_id": [_vp, _i], "vx_tp_init": [_vp, _vp, _i, _i], "vx_tp_shutdown": [_vp], "vx_model_enable_tp": [_vp, _i],
    "vx_set_gemm_terms": [_i], "vx_set_tc_min_rows": [_i], "vx_set_dependent_launch": [_i], "vx_model_max_blocks": [_vp],
    "vx_sched_create": [_vp, C.POINTER(SchedConfig), C.POINTER(_vp)], "vx_sched_destroy": [_vp],
    "vx_sched_add_sequence": [_vp, _i64, _vp, _i, _i], "vx_sched_remove_sequence": [_vp, _i64],
    "vx_sched_step": [_vp, C.POINTER(_i)], "vx_sched_poll": [_vp, _i64, _vp, _i, C.POINTER(_i), C.POINTER(_i)],
    "vx_sched_get_metrics": [_vp, C.POINTER(SchedMetrics)],
    "vx_sched_get_pressure": [_vp, C.POINTER(_u64), C.POINTER(_u64)],
}
_RESTYPE = {"vx_last_error": C.c_char_p, "vx_gguf_error": C.c_char_p}


class Lib:
    """Loads libvexel_cuda.so (built by vexel_b200/build.py).  Raises if it is absent: no fallback."""
    _inst = None

    def __init__(self, path=LIB_PATH):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is missing: build it with `python -m vexel_b200.build` (nvcc, sm_100a)")
        self.dll = C.CDLL(path)
        for name, args in SIGNATURES.items():
            fn = getattr(self.dll, name)   # AttributeError if the library lacks a declared symbol
            fn.argtypes = args
            fn.restype = _RESTYPE.get(name, C.c_int)

    @classmethod
    def get(cls):
        if cls._inst is None:
            cls._inst = Lib()
        return cls._inst


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Backend:
    """Method-for-method mirror of the reference's backend interfaces over the C ABI.
    Device buffers are plain integers (device addresses), like DevicePtr.addr+offset."""

    def __init__(self, device=0):
        self.lib = Lib.get().dll
        h = C.c_void_p()
        rc = self.lib.vx_init(device, C.byref(h))
        if rc != OK:
            raise VxError(rc, "vx_init failed: no usable CUDA device (this backend has no CPU fallback)")
        self.h = h

    def close(self):
        if self.h:
            self.lib.vx_destroy(self.h); self.h = None

    def _ck(self, rc):
        if rc != OK:
            raise VxError(rc, self.lib.vx_last_error(self.h).decode())

    # ---- memory (Backend.Alloc/Free/ToDevice/ToHost/Sync, AllocPermanent, ResetPool, CopyBuffer)
    def Alloc(self, nbytes):
        p = _D(); self._ck(self.lib.vx_alloc(self.h, nbytes, C.byref(p))); return p.value

    def AllocPermanent(self, nbytes):
        p = _D(); self._ck(self.lib.vx_alloc_permanent(self.h, nbytes, C.byref(p))); return p.value

    def Free(self, p): self._ck(self.lib.vx_free(self.h, p))
    def ResetPool(self): self._ck(self.lib.vx_reset_pool(self.h))
    def Sync(self): self._ck(self.lib.vx_sync(self.h))

    def ToDevice(self, dst, arr):
        arr = np.ascontiguousarray(arr); self._ck(self.lib.vx_h2d(self.h, dst, _np_ptr(arr), arr.nbytes))

    def ToHost(self, arr, src):
        assert arr.flags["C_CONTIGUOUS"]; self._ck(self.lib.vx_d2h(self.h, _np_ptr(arr), src, arr.nbytes))

    def CopyBuffer(self, src, src_off, dst, dst_off, size):
        self._ck(self.lib.vx_d2d(self.h, dst + dst_off, src + src_off, size))

    # convenience for tests
    def upload(self, arr, permanent=False):
        arr = np.ascontiguousarray(arr)
        p = (self.AllocPermanent if permanent else self.Alloc)(max(arr.nbytes, 4)); self.ToDevice(p, arr); return p

    def download(self, p, shape, dtype=np.float32):
        out = np.empty(shape, dtype); self.ToHost(out, p); return out

    def zeros(self, nbytes, permanent=True):
        p = (self.AllocPermanent if permanent else self.Alloc)(nbytes); self._ck(self.lib.vx_memset(self.h, p, 0, nbytes)); return p

    # ---- Backend kernels
    def MatMul(self, a, b, out, m, n, k): self._ck(self.lib.vx_matmul_f32(self.h, a, b, out, m, n, k))
    def MatMulTransposed(self, a, b, out, m, n, k): self._ck(self.lib.vx_matmul_f32_t(self.h, a, b, out, m, n, k))
    def RMSNorm(self, x, w, out, rows, cols, eps): self._ck(self.lib.vx_rmsnorm(self.h, x, w, out, rows, cols, eps))

    def RoPE(self, q, k, head_dim, n_heads, n_kv_heads, seq_len, start_pos, rope_dim, theta, neox):
        self._ck(self.lib.vx_rope(self.h, q, k or 0, head_dim, n_heads, n_kv_heads, seq_len, start_pos, rope_dim, theta, int(neox)))

    def RoPEWithFreqs(self, q, k, freqs, head_dim, n_heads, n_kv_heads, seq_len, start_pos, neox):
        self._ck(self.lib.vx_rope_freqs(self.h, q, k or 0, freqs, head_dim, n_heads, n_kv_heads, seq_len, start_pos, int(neox)))

    def SiLU(self, x, out, n): self._ck(self.lib.vx_silu(self.h, x, out, n))
    def SiLUMul(self, g, u, out, n): self._ck(self.lib.vx_silu_mul(self.h, g, u, out, n))
    def GELU(self, x, out, n): self._ck(self.lib.vx_gelu(self.h, x, out, n))
    def GELUMul(self, g, u, out, n): self._ck(self.lib.vx_gelu_mul(self.h, g, u, out, n))
    def Softmax(self, x, out, rows, cols): self._ck(self.lib.vx_softmax(self.h, x, out, rows, cols))
    def Add(self, a, b, out, n): self._ck(self.lib.vx_add(self.h, a, b, out, n))
    def Mul(self, a, b, out, n): self._ck(self.lib.vx_mul(self.h, a, b, out, n))
    def ScaleBuffer(self, buf, s, n): self._ck(self.lib.vx_scale(self.h, buf, s, n))

    def Embedding(self, ids, n_tokens, table, out, vocab, dim):
        self._ck(self.lib.vx_embedding(self.h, ids, n_tokens, table, out, vocab, dim))

    def SDPA(self, q, k, v, out, kv_len, hq, hkv, d, scale, kv_head_stride):
        self._ck(self.lib.vx_sdpa(self.h, q, k, v, out, kv_len, hq, hkv, d, scale, kv_head_stride))

    def SDPAPrefill(self, q, k, v, out, seq_len, hq, hkv, d, scale):
        self._ck(self.lib.vx_sdpa_prefill(self.h, q, k, v, out, seq_len, hq, hkv, d, scale))

    def SDPASoftCap(self, q, k, v, out, kv_len, hq, hkv, d, scale, softcap, kv_head_stride):
        self._ck(self.lib.vx_sdpa_softcap(self.h, q, k, v, out, kv_len, hq, hkv, d, scale, softcap, kv_head_stride))

    def SDPAPrefillSoftCap(self, q, k, v, out, seq_len, hq, hkv, d, scale, softcap):
        self._ck(self.lib.vx_sdpa_prefill_softcap(self.h, q, k, v, out, seq_len, hq, hkv, d, scale, softcap))

    def Argmax(self, x, n):
        r = C.c_int(); self._ck(self.lib.vx_argmax(self.h, x, n, C.byref(r))); return r.value

    def SampleRows(self, logits, rows, n, params):
        """Sampler.Sample on `rows` device logits rows; params = array of (temperature, top_k, top_p, u) records."""
        params = np.ascontiguousarray(params, SAMPLE_DTYPE); out = np.empty(rows, np.int32)
        self._ck(self.lib.vx_sample_rows(self.h, logits, rows, n, _np_ptr(params), _np_ptr(out))); return out

    def ArgmaxRows(self, x, rows, cols, out): self._ck(self.lib.vx_argmax_rows(self.h, x, rows, cols, out))
    def MatMulQ4_0(self, a, b, out, m, n, k): self._ck(self.lib.vx_matmul_q4_0(self.h, a, b, out, m, n, k))
    def MatMulQ4_K(self, a, b, out, m, n, k): self._ck(self.lib.vx_matmul_q4_k(self.h, a, b, out, m, n, k))
    def MatMulQ6_K(self, a, b, out, m, n, k): self._ck(self.lib.vx_matmul_q6_k(self.h, a, b, out, m, n, k))
    def Dequantize(self, type_id, raw, out, n): self._ck(self.lib.vx_dequantize(self.h, type_id, raw, out, n))

    # ---- PagedKVOps
    def ReshapePagedKV(self, src, pool, page_table, block_offsets, n_tokens, hkv, d, bs, is_value):
        self._ck(self.lib.vx_reshape_paged_kv(self.h, src, pool, page_table, block_offsets, n_tokens, hkv, d, bs, int(is_value)))

    def ReshapePagedKVF16(self, src, pool, page_table, block_offsets, n_tokens, hkv, d, bs, is_value):
        self._ck(self.lib.vx_reshape_paged_kv_f16(self.h, src, pool, page_table, block_offsets, n_tokens, hkv, d, bs, int(is_value)))

    def SDPAPagedDecode(self, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last):
        self._ck(self.lib.vx_sdpa_paged_decode(self.h, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last))

    def SDPAPagedDecodeF16(self, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last):
        self._ck(self.lib.vx_sdpa_paged_decode_f16(self.h, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last))

    def SDPAPagedDecodeF16NoAlloc(self, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last):
        """vx_sdpa_paged_decode_f16 with its scratch in a fixed device array: the call allocates nothing."""
        self._ck(self.lib.vx_sdpa_paged_decode_f16_noalloc(self.h, q, pool, table, out, n_blocks, bs, hq, hkv, d, scale, tokens_in_last))

    def SDPAPagedDecodeBatched(self, q, pool, tables, out, batch, max_blocks, bs, hq, hkv, d, scale, seq_lens, f16=True):
        tb = (_D * batch)(*tables); sl = (_i * batch)(*seq_lens)
        self._ck(self.lib.vx_sdpa_paged_decode_batched(self.h, q, pool, tb, out, batch, max_blocks, bs, hq, hkv, d, scale, sl, int(f16)))

    def SDPAPagedDecodeMultiquery(self, q, pool, table, out, kv_lens, n_blocks, bs, hq, hkv, d, scale, query_len, f16=True):
        self._ck(self.lib.vx_sdpa_paged_decode_multiquery(self.h, q, pool, table, out, kv_lens, n_blocks, bs, hq, hkv, d, scale, query_len, int(f16)))

    def SDPAPagedDecodeEx(self, q, pool, table, out, kv_start, kv_len, bs, hq, hkv, d, scale, softcap, f16=True):
        self._ck(self.lib.vx_sdpa_paged_decode_ex(self.h, q, pool, table, out, kv_start, kv_len, bs, hq, hkv, d, scale, softcap, int(f16)))

    def SynthQ4_0(self, dst, n_elements, seed, sigma): self._ck(self.lib.vx_synth_q4_0(self.h, dst, n_elements, seed, sigma))

    def SynthKQuant(self, dst, type_id, n_elements, seed, sigma):
        self._ck(self.lib.vx_synth_kquant(self.h, dst, type_id, n_elements, seed, sigma))


class GGUFError(RuntimeError):
    pass


class GGUF:
    """A parsed GGUF file (gguf.Open, pkg/gguf/gguf.go:246): metadata, tensor table, architecture config.  Host only."""

    def __init__(self, path):
        self.lib = Lib.get().dll
        h = C.c_void_p()
        rc = self.lib.vx_gguf_open(os.fsencode(path), C.byref(h))
        self.h = h
        if rc != 0:
            msg = self.lib.vx_gguf_error(h).decode(); self.close()
            raise GGUFError(msg)

    def close(self):
        if self.h:
            self.lib.vx_gguf_close(self.h); self.h = None

    def _ck(self, rc):
        if rc != 0:
            raise GGUFError("%d: %s" % (rc, self.lib.vx_gguf_error(self.h).decode()))

    def tensors(self):
        """[(name, ggml type, dims in GGUF order, absolute file offset, bytes)]"""
        out = []
        for i in range(self.lib.vx_gguf_tensor_count(self.h)):
            name = C.create_string_buffer(256); t, nd = C.c_int(), C.c_int()
            ne = (C.c_uint64 * 4)(); off, nb = C.c_uint64(), C.c_uint64()
            self._ck(self.lib.vx_gguf_tensor_info(self.h, i, name, 256, C.byref(t), C.byref(nd), ne, C.byref(off), C.byref(nb)))
            out.append((name.value.decode(), t.value, tuple(ne[:nd.value]), off.value, nb.value))
        return out

    def meta(self, key):
        buf = C.create_string_buffer(4096)
        rc = self.lib.vx_gguf_meta(self.h, key.encode(), buf, 4096)
        return None if rc == 5 else buf.value.decode()

    def model_config(self, max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq) -> ModelConfig:
        cfg = ModelConfig(max_blocks=max_blocks, max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, max_blocks_per_seq=max_blocks_per_seq)
        self._ck(self.lib.vx_gguf_model_config(self.h, C.byref(cfg)))
        return cfg


class Model:
    """The batched decode fast path (vx_model_* / vx_seq_* / vx_decode_step / vx_prefill)."""

    def __init__(self, be: Backend, cfg: ModelConfig):
        self.be, self.lib, self.cfg = be, be.lib, cfg
        h = C.c_void_p()
        be._ck(self.lib.vx_model_create(be.h, C.byref(cfg), C.byref(h)))
        self.h = h

    @classmethod
    def from_gguf(cls, be: Backend, path, max_blocks, max_seqs=8, max_batch_tokens=256, max_blocks_per_seq=64):
        """initModel's load sequence (cmd/vexel/commands.go:35-142): parse, configure from metadata, stream weights to the device."""
        g = GGUF(path)
        try:
            m = cls(be, g.model_config(max_blocks, max_seqs, max_batch_tokens, max_blocks_per_seq))
            try:
                m._ck(m.lib.vx_model_load_gguf(m.h, g.h))
            except Exception:
                m.close(); raise
            return m
        finally:
            g.close()

    def close(self):
        if self.h:
            self.lib.vx_model_destroy(self.h); self.h = None

    def _ck(self, rc): self.be._ck(rc)

    def set_tensor(self, layer, slot, type_id, data):
        if isinstance(data, tuple):   # (device address, nbytes)
            self._ck(self.lib.vx_model_set_tensor(self.h, layer, slot, type_id, C.c_void_p(data[0]), data[1], 1))
        else:
            data = np.ascontiguousarray(data)
            self._ck(self.lib.vx_model_set_tensor(self.h, layer, slot, type_id, _np_ptr(data), data.nbytes, 0))

    def finalize(self): self._ck(self.lib.vx_model_finalize(self.h))
    def seq_create(self, s): self._ck(self.lib.vx_seq_create(self.h, s))
    def seq_delete(self, s): self._ck(self.lib.vx_seq_delete(self.h, s))
    def seq_truncate(self, s, n): self._ck(self.lib.vx_seq_truncate(self.h, s, n))
    def seq_share(self, a, b, n): self._ck(self.lib.vx_seq_share(self.h, a, b, n))
    def seq_fill_synthetic(self, s, n, seed=0): self._ck(self.lib.vx_seq_fill_synthetic(self.h, s, n, seed))
    def shuffle_free_list(self, seed): self._ck(self.lib.vx_pool_shuffle_free_list(self.h, seed))

    def seq_len(self, s):
        r = C.c_int(); self._ck(self.lib.vx_seq_len(self.h, s, C.byref(r))); return r.value

    def block_table(self, s):
        buf = np.zeros(self.cfg.max_blocks_per_seq, np.int32); n = C.c_int()
        self._ck(self.lib.vx_seq_block_table(self.h, s, _np_ptr(buf), buf.size, C.byref(n)))
        return buf[:n.value].copy()

    def pool_stats(self):
        a, b, c = C.c_int(), C.c_int(), C.c_int()
        self._ck(self.lib.vx_pool_stats(self.h, C.byref(a), C.byref(b), C.byref(c))); return a.value, b.value, c.value

    def free_list(self):
        """the per-layer free list, bottom of the stack first (the next block handed out is the last entry)"""
        buf = np.empty(self.cfg.max_blocks, np.int32); n = C.c_int()
        self._ck(self.lib.vx_pool_free_list(self.h, _np_ptr(buf), buf.size, C.byref(n))); return buf[:n.value].copy()

    def pool_layer(self, layer):
        p, n = _D(), C.c_size_t()
        self._ck(self.lib.vx_pool_layer_ptr(self.h, layer, C.byref(p), C.byref(n))); return p.value, n.value

    def decode_step(self, seq_ids, tokens, positions, q_lens=None, want_logits=False):
        seq_ids = np.ascontiguousarray(seq_ids, np.int64); tokens = np.ascontiguousarray(tokens, np.int32)
        positions = np.ascontiguousarray(positions, np.int32)
        ql = None if q_lens is None else np.ascontiguousarray(q_lens, np.int32)
        rows = tokens.size
        out = np.empty(rows, np.int32)
        logits = np.empty((rows, self.cfg.vocab), np.float32) if want_logits else None
        self._ck(self.lib.vx_decode_step(self.h, seq_ids.size, _np_ptr(seq_ids), _np_ptr(tokens), _np_ptr(positions),
                                        _np_ptr(ql), _np_ptr(out), _np_ptr(logits)))
        return (out, logits) if want_logits else out

    def decode_step_ex(self, seq_ids, tokens, positions, q_lens=None, last_rows=False, prompt_rows=False, params=None,
                       want_logits=False, want_hidden=False):
        """vx_decode_step_ex: returns (tokens, logits or None, post-final-norm hidden states or None) for the output rows --
        every packed row, or with last_rows the last row of each batch entry."""
        seq_ids = np.ascontiguousarray(seq_ids, np.int64); tokens = np.ascontiguousarray(tokens, np.int32)
        positions = np.ascontiguousarray(positions, np.int32)
        ql = None if q_lens is None else np.ascontiguousarray(q_lens, np.int32)
        rows = seq_ids.size if last_rows else tokens.size
        par = None if params is None else np.ascontiguousarray(params, SAMPLE_DTYPE)
        assert par is None or par.size == rows
        out = np.empty(rows, np.int32)
        logits = np.empty((rows, self.cfg.vocab), np.float32) if want_logits else None
        hidden = np.empty((rows, self.cfg.hidden), np.float32) if want_hidden else None
        flags = (STEP_LAST_ROWS if last_rows else 0) | (STEP_PROMPT_ROWS if prompt_rows else 0)
        self._ck(self.lib.vx_decode_step_ex(self.h, seq_ids.size, _np_ptr(seq_ids), _np_ptr(tokens), _np_ptr(positions), _np_ptr(ql),
                                           flags, _np_ptr(par), _np_ptr(out), _np_ptr(logits), _np_ptr(hidden)))
        return out, logits, hidden

    def decode_step_sampled(self, seq_ids, tokens, positions, params, q_lens=None, want_logits=False):
        """decode_step with one (temperature, top_k, top_p, u) record per packed row, sampled on the device."""
        seq_ids = np.ascontiguousarray(seq_ids, np.int64); tokens = np.ascontiguousarray(tokens, np.int32)
        positions = np.ascontiguousarray(positions, np.int32); params = np.ascontiguousarray(params, SAMPLE_DTYPE)
        ql = None if q_lens is None else np.ascontiguousarray(q_lens, np.int32)
        rows = tokens.size
        assert params.size == rows
        out = np.empty(rows, np.int32)
        logits = np.empty((rows, self.cfg.vocab), np.float32) if want_logits else None
        self._ck(self.lib.vx_decode_step_sampled(self.h, seq_ids.size, _np_ptr(seq_ids), _np_ptr(tokens), _np_ptr(positions),
                                                _np_ptr(ql), _np_ptr(params), _np_ptr(out), _np_ptr(logits)))
        return (out, logits) if want_logits else out

    def decode_run(self, seq_ids, tokens, positions, n_steps):
        """n_steps greedy steps with on-device token feedback; returns (tokens [n_steps, n_seqs], device ms)."""
        seq_ids = np.ascontiguousarray(seq_ids, np.int64); tokens = np.ascontiguousarray(tokens, np.int32)
        positions = np.ascontiguousarray(positions, np.int32)
        out = np.empty((n_steps, seq_ids.size), np.int32); ms = C.c_float()
        self._ck(self.lib.vx_decode_run(self.h, seq_ids.size, _np_ptr(seq_ids), _np_ptr(tokens), _np_ptr(positions), n_steps,
                                       _np_ptr(out), C.byref(ms)))
        return out, ms.value

    def prefill(self, seq, tokens, start_pos=0, want_logits=False):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty(1, np.int32)
        logits = np.empty((1, self.cfg.vocab), np.float32) if want_logits else None
        self._ck(self.lib.vx_prefill(self.h, seq, _np_ptr(tokens), tokens.size, start_pos, _np_ptr(out), _np_ptr(logits)))
        return (int(out[0]), logits) if want_logits else int(out[0])

    def set_capture(self, on): self._ck(self.lib.vx_model_set_capture(self.h, int(on)))

    def get_capture(self, rows):
        out = np.empty((self.cfg.n_layers + 1, rows, self.cfg.hidden), np.float32)
        self._ck(self.lib.vx_model_get_capture(self.h, _np_ptr(out), out.size)); return out

    def get_packing(self, n_seqs, n_rows):
        cu = np.empty(n_seqs + 1, np.int32); sm = np.empty(n_rows, np.int32); kl = np.empty(n_rows, np.int32)
        self._ck(self.lib.vx_model_get_packing(self.h, _np_ptr(cu), _np_ptr(sm), _np_ptr(kl), n_seqs, n_rows)); return cu, sm, kl

    def counters(self):
        a, b = C.c_uint64(), C.c_uint64(); self._ck(self.lib.vx_model_counters(self.h, C.byref(a), C.byref(b))); return a.value, b.value

    def graph_stats(self):
        a, b = C.c_uint64(), C.c_uint64(); self._ck(self.lib.vx_model_graph_stats(self.h, C.byref(a), C.byref(b))); return a.value, b.value

    def kernel_time(self, which, enable=-1):
        ms, n = C.c_float(), C.c_uint64()
        self._ck(self.lib.vx_model_kernel_time(self.h, which, enable, C.byref(ms), C.byref(n))); return ms.value, n.value

    def weight_bytes(self):
        b = C.c_uint64(); self._ck(self.lib.vx_model_weight_bytes(self.h, C.byref(b))); return b.value


class Scheduler:
    """vx_sched_*: the continuous-batching loop of inference/scheduler over the batched fast path."""

    def __init__(self, model: Model, max_batch_size, max_sequences=0, max_tokens=0, eos_token=-1, temperature=0.0, top_k=0, top_p=0.0, seed=0):
        self.m, self.lib = model, model.lib
        cfg = SchedConfig(max_batch_size, max_sequences, max_tokens, eos_token, temperature, top_k, top_p, seed)
        h = C.c_void_p()
        model._ck(self.lib.vx_sched_create(model.h, C.byref(cfg), C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.lib.vx_sched_destroy(self.h); self.h = None

    def AddSequence(self, seq_id, prompt, max_tokens=0):
        p = np.ascontiguousarray(prompt, np.int32)
        self.m._ck(self.lib.vx_sched_add_sequence(self.h, seq_id, _np_ptr(p), p.size, max_tokens))

    def RemoveSequence(self, seq_id): self.m._ck(self.lib.vx_sched_remove_sequence(self.h, seq_id))

    def step(self):
        n = C.c_int(); self.m._ck(self.lib.vx_sched_step(self.h, C.byref(n))); return n.value

    def poll(self, seq_id, cap=4096):
        buf = np.empty(cap, np.int32); n, fin = C.c_int(), C.c_int()
        self.m._ck(self.lib.vx_sched_poll(self.h, seq_id, _np_ptr(buf), cap, C.byref(n), C.byref(fin)))
        return buf[:n.value].copy(), bool(fin.value)

    def poll_status(self, seq_id, cap=4096):
        """(tokens, status): 0 running, 1 ended, 2 refused (the request could never fit the block pool)."""
        buf = np.empty(cap, np.int32); n, fin = C.c_int(), C.c_int()
        self.m._ck(self.lib.vx_sched_poll(self.h, seq_id, _np_ptr(buf), cap, C.byref(n), C.byref(fin)))
        return buf[:n.value].copy(), fin.value

    def Metrics(self):
        m = SchedMetrics(); self.m._ck(self.lib.vx_sched_get_metrics(self.h, C.byref(m))); return m

    def pressure(self):
        a, b = C.c_uint64(), C.c_uint64()
        self.m._ck(self.lib.vx_sched_get_pressure(self.h, C.byref(a), C.byref(b))); return a.value, b.value
