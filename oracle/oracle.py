"""ctypes view of the CPU oracle (oracle/vexel_oracle.c).  TEST INFRASTRUCTURE ONLY:
imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline leg."""
import ctypes as C
import numpy as np

from . import build as _build

F32, F16, Q4_0, Q4_K, Q6_K = 0, 1, 2, 12, 14
T_ATTN_NORM, T_WQ, T_WK, T_WV, T_WO, T_POST_ATTN_NORM, T_FFN_NORM, T_W1, T_W3, T_W2, T_POST_FFN_NORM = range(11)
G_EMBED, G_FINAL_NORM, G_OUTPUT = 0, 1, 2

_lib = None


class Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n_layers", "hidden", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab")] + [
        ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("rope_neox", C.c_int), ("geglu", C.c_int),
        ("post_norms", C.c_int), ("embed_scale", C.c_float), ("attn_softcap", C.c_float),
        ("final_softcap", C.c_float), ("sliding_window", C.c_int), ("window_alternating", C.c_int),
        ("max_blocks", C.c_int), ("kv_f16", C.c_int)]


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(_build.build())
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        sig = {
            "vo_f16_to_f32": (f32, [C.c_uint16]), "vo_f32_to_f16": (C.c_uint16, [f32]),
            "vo_type_row_bytes": (C.c_size_t, [i32, i64]),
            "vo_dequant": (None, [i32, vp, i64, vp]),
            "vo_scale_min_k4": (None, [i32, vp, vp, vp]),
            "vo_matmul": (None, [vp, vp, vp, i32, i32, i32]),
            "vo_matmul_transposed": (None, [vp, vp, vp, i32, i32, i32]),
            "vo_matmul_q4_0": (None, [vp, vp, vp, i32, i32, i32]),
            "vo_rmsnorm": (None, [vp, vp, vp, i32, i32, f32]),
            "vo_rope": (None, [vp, vp, i32, i32, i32, i32, i32, i32, f32, i32]),
            "vo_rope_freqs": (None, [vp, vp, vp, i32, i32, i32, i32, i32, i32]),
            "vo_silu": (None, [vp, vp, i32]), "vo_silu_mul": (None, [vp, vp, vp, i32]),
            "vo_gelu": (None, [vp, vp, i32]), "vo_gelu_mul": (None, [vp, vp, vp, i32]),
            "vo_softmax": (None, [vp, vp, i32, i32]),
            "vo_add": (None, [vp, vp, vp, i32]), "vo_mul": (None, [vp, vp, vp, i32]),
            "vo_scale": (None, [vp, f32, i32]),
            "vo_embedding": (None, [vp, i32, vp, vp, i32, i32]),
            "vo_sdpa": (None, [vp, vp, vp, vp, i32, i32, i32, i32, f32, f32, i32]),
            "vo_sdpa_prefill": (None, [vp, vp, vp, vp, i32, i32, i32, i32, f32, f32]),
            "vo_argmax": (i32, [vp, i32]), "vo_final_softcap": (None, [vp, i32, f32]),
            "vo_sample": (i32, [vp, i32, f32, i32, f32, f32]),
            "vo_reshape_paged_kv_f32": (None, [vp, vp, vp, vp, i32, i32, i32, i32, i32]),
            "vo_reshape_paged_kv_f16": (None, [vp, vp, vp, vp, i32, i32, i32, i32, i32]),
            "vo_sdpa_paged": (None, [vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, f32, f32]),
            "vo_pool_create": (vp, [i32] * 6), "vo_pool_destroy": (None, [vp]),
            "vo_pool_create_seq": (None, [vp, i64]), "vo_pool_delete_seq": (None, [vp, i64]),
            "vo_pool_truncate": (None, [vp, i64, i32]), "vo_pool_share": (i32, [vp, i64, i64, i32]),
            "vo_pool_store_kv": (i32, [vp, i32, i64, i32, vp, vp, i32]),
            "vo_pool_seq_len": (i32, [vp, i64]), "vo_pool_table": (i32, [vp, i32, i64, vp, i32]),
            "vo_pool_free_blocks": (i32, [vp, i32]), "vo_pool_layer_data": (vp, [vp, i32]),
            "vo_pool_set_free_list": (i32, [vp, vp, i32]),
            "vo_pool_attention": (i32, [vp, i32, i64, vp, vp, i32, f32, f32, i32, i32]),
            "vo_model_create": (vp, [C.POINTER(Config)]), "vo_model_destroy": (None, [vp]),
            "vo_model_set_layer_tensor": (i32, [vp, i32, i32, i32, vp]),
            "vo_model_set_global_tensor": (i32, [vp, i32, i32, vp]),
            "vo_model_pool": (vp, [vp]),
            "vo_model_forward": (i32, [vp, i64, vp, i32, i32, i32, vp, vp]),
            "vo_set_threads": (None, [i32]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def dequant(type_id, raw, n):
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty(n, np.float32)
    lib().vo_dequant(type_id, _p(raw), n, _p(out))
    return out


def f32_to_f16_bits(x):
    L = lib()
    return np.array([L.vo_f32_to_f16(float(v)) for v in np.asarray(x, np.float32).ravel()], np.uint16)


def matmul_q4_0(a, bq, m, n, k):
    a = _f32(a); out = np.empty((m, n), np.float32)
    lib().vo_matmul_q4_0(_p(a), _p(bq), _p(out), m, n, k)
    return out


def matmul_transposed(a, b, m, n, k):
    a, b = _f32(a), _f32(b); out = np.empty((m, n), np.float32)
    lib().vo_matmul_transposed(_p(a), _p(b), _p(out), m, n, k)
    return out


def matmul(a, b, m, n, k):
    a, b = _f32(a), _f32(b); out = np.empty((m, n), np.float32)
    lib().vo_matmul(_p(a), _p(b), _p(out), m, n, k)
    return out


def rmsnorm(x, w, eps):
    x, w = _f32(x), _f32(w); out = np.empty_like(x)
    lib().vo_rmsnorm(_p(x), _p(w), _p(out), x.shape[0], x.shape[1], eps)
    return out


def rope(q, k, head_dim, n_heads, n_kv_heads, seq_len, start_pos, rope_dim, theta, neox):
    q = _f32(q).copy(); k = None if k is None else _f32(k).copy()
    lib().vo_rope(_p(q), _p(k), head_dim, n_heads, n_kv_heads, seq_len, start_pos, rope_dim, theta, int(neox))
    return q, k


def rope_freqs(q, k, freqs, head_dim, n_heads, n_kv_heads, seq_len, start_pos, neox):
    q = _f32(q).copy(); k = None if k is None else _f32(k).copy(); freqs = _f32(freqs)
    lib().vo_rope_freqs(_p(q), _p(k), _p(freqs), head_dim, n_heads, n_kv_heads, seq_len, start_pos, int(neox))
    return q, k


def _ew1(fn, x):
    x = _f32(x); out = np.empty_like(x); fn(_p(x), _p(out), x.size); return out


def _ew2(fn, a, b):
    a, b = _f32(a), _f32(b); out = np.empty_like(a); fn(_p(a), _p(b), _p(out), a.size); return out


def silu(x): return _ew1(lib().vo_silu, x)
def gelu(x): return _ew1(lib().vo_gelu, x)
def silu_mul(g, u): return _ew2(lib().vo_silu_mul, g, u)
def gelu_mul(g, u): return _ew2(lib().vo_gelu_mul, g, u)
def add(a, b): return _ew2(lib().vo_add, a, b)
def mul(a, b): return _ew2(lib().vo_mul, a, b)


def softmax(x):
    x = _f32(x); out = np.empty_like(x)
    lib().vo_softmax(_p(x), _p(out), x.shape[0], x.shape[1]); return out


def embedding(ids, table, out_init=None):
    ids = np.ascontiguousarray(ids, np.int32); table = _f32(table)
    out = np.zeros((ids.size, table.shape[1]), np.float32) if out_init is None else _f32(out_init).copy()
    lib().vo_embedding(_p(ids), ids.size, _p(table), _p(out), table.shape[0], table.shape[1]); return out


def sdpa(q, k, v, kv_len, n_q, n_kv, d, scale, softcap=0.0, kv_head_stride=None):
    q, k, v = _f32(q), _f32(k), _f32(v); out = np.empty(n_q * d, np.float32)
    lib().vo_sdpa(_p(q), _p(k), _p(v), _p(out), kv_len, n_q, n_kv, d, scale, softcap,
                  kv_len * d if kv_head_stride is None else kv_head_stride)
    return out


def sdpa_prefill(q, k, v, seq_len, n_q, n_kv, d, scale, softcap=0.0):
    q, k, v = _f32(q), _f32(k), _f32(v); out = np.empty(seq_len * n_q * d, np.float32)
    lib().vo_sdpa_prefill(_p(q), _p(k), _p(v), _p(out), seq_len, n_q, n_kv, d, scale, softcap)
    return out


def argmax(x):
    x = _f32(x); return lib().vo_argmax(_p(x), x.size)


def sample(logits, temperature, top_k, top_p, r):
    x = _f32(logits); return lib().vo_sample(_p(x), x.size, temperature, top_k, top_p, r)


def reshape_paged_kv(src, pool, blk, off, n_kv, d, bs, is_v):
    src = _f32(src); blk = np.ascontiguousarray(blk, np.int32); off = np.ascontiguousarray(off, np.int32)
    fn = lib().vo_reshape_paged_kv_f16 if pool.dtype == np.uint16 else lib().vo_reshape_paged_kv_f32
    fn(_p(src), _p(pool), _p(blk), _p(off), blk.size, n_kv, d, bs, int(is_v))


def sdpa_paged(q, pool, table, kv_start, kv_len, bs, n_q, n_kv, d, scale, softcap=0.0):
    q = _f32(q); table = np.ascontiguousarray(table, np.int32); out = np.empty(n_q * d, np.float32)
    lib().vo_sdpa_paged(_p(q), _p(pool), int(pool.dtype == np.uint16), _p(table), _p(out), kv_start, kv_len,
                        bs, n_q, n_kv, d, scale, softcap)
    return out


class Pool:
    """runtime/gpu_block_pool.go bookkeeping + host data."""

    def __init__(self, n_layers, n_kv, d, bs, max_blocks, f16=True, handle=None):
        self.L = lib(); self.owned = handle is None
        self.h = handle or self.L.vo_pool_create(n_layers, n_kv, d, bs, max_blocks, int(f16))
        self.n_layers, self.n_kv, self.d, self.bs, self.max_blocks, self.f16 = n_layers, n_kv, d, bs, max_blocks, f16

    def __del__(self):
        if getattr(self, "owned", False) and self.h:
            self.L.vo_pool_destroy(self.h); self.h = None

    def create_seq(self, s): self.L.vo_pool_create_seq(self.h, s)
    def delete_seq(self, s): self.L.vo_pool_delete_seq(self.h, s)
    def truncate(self, s, n): self.L.vo_pool_truncate(self.h, s, n)
    def share(self, a, b, n): return self.L.vo_pool_share(self.h, a, b, n)
    def seq_len(self, s): return self.L.vo_pool_seq_len(self.h, s)
    def free_blocks(self, layer=0): return self.L.vo_pool_free_blocks(self.h, layer)

    def set_free_list(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        assert self.L.vo_pool_set_free_list(self.h, _p(ids), ids.size) == 0

    def store_kv(self, layer, s, start, k, v, n_tok):
        if k is None:                      # allocate the blocks of [start, start + n_tok) without writing them
            return self.L.vo_pool_store_kv(self.h, layer, s, start, None, None, n_tok)
        k, v = _f32(k), _f32(v)
        return self.L.vo_pool_store_kv(self.h, layer, s, start, _p(k), _p(v), n_tok)

    def table(self, layer, s):
        buf = np.zeros(self.max_blocks, np.int32)
        n = self.L.vo_pool_table(self.h, layer, s, _p(buf), self.max_blocks)
        return buf[:max(n, 0)].copy()

    def layer_data(self, layer):
        n = self.max_blocks * 2 * self.bs * self.n_kv * self.d
        ptr = self.L.vo_pool_layer_data(self.h, layer)
        ct = C.c_uint16 if self.f16 else C.c_float
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ct)), shape=(n,))

    def attention(self, layer, s, q, n_q, scale, softcap=0.0, window=0, kv_len=0):
        q = _f32(q); out = np.empty(n_q * self.d, np.float32)
        rc = self.L.vo_pool_attention(self.h, layer, s, _p(q), _p(out), n_q, scale, softcap, window, kv_len)
        assert rc == 0
        return out


class Model:
    def __init__(self, cfg: Config):
        self.L = lib(); self.cfg = cfg
        self.h = self.L.vo_model_create(C.byref(cfg))
        self.pool = Pool(cfg.n_layers, cfg.n_kv_heads, cfg.head_dim, 16, cfg.max_blocks, bool(cfg.kv_f16),
                         handle=self.L.vo_model_pool(self.h))

    def __del__(self):
        if getattr(self, "h", None):
            self.L.vo_model_destroy(self.h); self.h = None

    def set_layer(self, layer, slot, type_id, data):
        data = np.ascontiguousarray(data)
        assert self.L.vo_model_set_layer_tensor(self.h, layer, slot, type_id, _p(data)) == 0

    def set_global(self, which, type_id, data):
        data = np.ascontiguousarray(data)
        assert self.L.vo_model_set_global_tensor(self.h, which, type_id, _p(data)) == 0

    def forward(self, seq, tokens, start_pos, all_logits=False, want_hidden=False):
        tokens = np.ascontiguousarray(tokens, np.int32); T = tokens.size
        rows = T if (T == 1 or all_logits) else 1
        logits = np.empty((rows, self.cfg.vocab), np.float32)
        hidden = np.empty((self.cfg.n_layers + 1, T, self.cfg.hidden), np.float32) if want_hidden else None
        rc = self.L.vo_model_forward(self.h, seq, _p(tokens), T, start_pos, int(all_logits), _p(logits), _p(hidden))
        if rc != 0:
            raise RuntimeError(f"oracle forward failed rc={rc}")
        return (logits, hidden) if want_hidden else logits
