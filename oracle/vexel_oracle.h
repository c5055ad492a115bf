/*
 * vexel_oracle.h -- CPU restatement of the reference's decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the product (the CUDA library and the
 * host code above it) links, loads or calls this.  It exists so the tests and
 * the CPU-baseline leg of the benchmark can compare the CUDA path with the
 * reference's own arithmetic.
 *
 * Every function names the reference file:line whose loop order and rounding
 * it follows (paths are relative to the reference project root).  The
 * reference is Go and cannot be compiled where this is built, so parity is
 * pinned by transcribing the known-answer tests the reference holds for this
 * path (see tests/test_oracle_kats.py).
 *
 * Floating point: compiled with -ffp-contract=off.  The Go compiler does not
 * fuse a*b+c on amd64 (it may on arm64); this file takes the amd64 behaviour:
 * every multiply and add rounds separately to float32.
 */
#ifndef VEXEL_ORACLE_H
#define VEXEL_ORACLE_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF tensor type ids used here (pkg/gguf/gguf.go:40-75). */
enum { VO_F32 = 0, VO_F16 = 1, VO_Q4_0 = 2, VO_Q4_K = 12, VO_Q6_K = 14 };

/* ---- scalar conversions ------------------------------------------------ */
float    vo_f16_to_f32(uint16_t h);   /* pkg/gguf/dequant.go:231-261 */
uint16_t vo_f32_to_f16(float f);      /* IEEE round-to-nearest-even, what Metal's (half) cast does */

/* ---- GGUF block formats ------------------------------------------------ */
size_t vo_type_row_bytes(int type, int64_t k);                           /* pkg/gguf/gguf.go:77-131 */
void vo_dequant_q4_0(const uint8_t *data, int64_t n, float *out);         /* dequant.go:16-56   */
void vo_dequant_q4_k(const uint8_t *data, int64_t n, float *out);         /* dequant.go:342-396 */
void vo_dequant_q6_k(const uint8_t *data, int64_t n, float *out);         /* dequant.go:272-331 */
void vo_dequant(int type, const uint8_t *data, int64_t n, float *out);
void vo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn);  /* dequant.go:400-409 */

/* ---- backend/cpu/cpu.go kernels --------------------------------------- */
void vo_matmul(const float *a, const float *b, float *out, int m, int n, int k);             /* cpu.go:106-144 */
void vo_matmul_transposed(const float *a, const float *b, float *out, int m, int n, int k);   /* cpu.go:158-197 */
void vo_matmul_q4_0(const float *a, const uint8_t *bq, float *out, int m, int n, int k);      /* cpu.go:842-911 */
void vo_rmsnorm(const float *x, const float *w, float *out, int rows, int cols, float eps);   /* cpu.go:200-220 */
void vo_rope(float *q, float *k, int head_dim, int n_heads, int n_kv_heads, int seq_len,
             int start_pos, int rope_dim, float theta, int neox);                              /* cpu.go:226-303 */
void vo_rope_freqs(float *q, float *k, const float *freqs, int head_dim, int n_heads,
                   int n_kv_heads, int seq_len, int start_pos, int neox);                      /* cpu.go:308-375 */
void vo_silu(const float *x, float *out, int n);                                              /* cpu.go:378-387 */
void vo_silu_mul(const float *g, const float *u, float *out, int n);                          /* cpu.go:390-400 */
void vo_gelu(const float *x, float *out, int n);                                              /* cpu.go:440-454 */
void vo_gelu_mul(const float *g, const float *u, float *out, int n);                          /* cpu.go:457-473 */
void vo_softmax(const float *x, float *out, int rows, int cols);                              /* cpu.go:489-518 */
void vo_add(const float *a, const float *b, float *out, int n);                               /* cpu.go:521-529 */
void vo_mul(const float *a, const float *b, float *out, int n);                               /* cpu.go:532-540 */
void vo_scale(float *x, float s, int n);                                                      /* cpu.go:558-563 */
void vo_embedding(const int32_t *ids, int n_tok, const float *table, float *out,
                  int vocab, int dim);                                                        /* cpu.go:543-555 */
void vo_sdpa(const float *q, const float *k, const float *v, float *out, int kv_len,
             int n_q_heads, int n_kv_heads, int head_dim, float scale, float softcap,
             int kv_head_stride);                                       /* cpu.go:568-632, 705-767 */
void vo_sdpa_prefill(const float *q, const float *k, const float *v, float *out, int seq_len,
                     int n_q_heads, int n_kv_heads, int head_dim, float scale,
                     float softcap);                                    /* cpu.go:635-701, 770-838 */
int  vo_argmax(const float *x, int n);                                  /* pkg/sampler/sampler.go:79-90 */
void vo_final_softcap(float *logits, int n, float cap);                 /* runtime/model.go:340-349 */

/* ---- sampler (pkg/sampler/sampler.go:49-204), r = the uniform draw in [0,1) ---- */
int vo_sample(const float *logits, int n, float temperature, int top_k, float top_p, float r);

/* ---- paged KV kernels: the semantics of the Metal paged shaders ---------
 * pool layout per layer (backend/metal/metal_bridge_darwin.m:8539-8642):
 *   elem((blk*2 + isV) * bs*Hkv*D + off*Hkv*D + h*D + d)
 */
void vo_reshape_paged_kv_f32(const float *src, float *pool, const int32_t *blk, const int32_t *off,
                             int n_tok, int n_kv_heads, int head_dim, int block_size, int is_v);
void vo_reshape_paged_kv_f16(const float *src, uint16_t *pool, const int32_t *blk, const int32_t *off,
                             int n_tok, int n_kv_heads, int head_dim, int block_size, int is_v);
/* kv_start..kv_len-1 are attended; kv_start>0 only for sliding-window layers
 * (runtime/block.go:925-929).  pool_is_f16 selects the element type. */
void vo_sdpa_paged(const float *q, const void *pool, int pool_is_f16, const int32_t *table,
                   float *out, int kv_start, int kv_len, int block_size, int n_q_heads,
                   int n_kv_heads, int head_dim, float scale, float softcap);

/* ---- device block pool bookkeeping (runtime/gpu_block_pool.go) ---------- */
typedef struct vo_pool vo_pool;
vo_pool *vo_pool_create(int n_layers, int n_kv_heads, int head_dim, int block_size,
                        int max_blocks, int f16);                       /* :66-126 */
void vo_pool_destroy(vo_pool *p);
void vo_pool_create_seq(vo_pool *p, int64_t seq);                       /* :129-137 */
void vo_pool_delete_seq(vo_pool *p, int64_t seq);                       /* :140-160 */
void vo_pool_truncate(vo_pool *p, int64_t seq, int new_len);            /* :165-190 */
int  vo_pool_share(vo_pool *p, int64_t src, int64_t dst, int n_tokens); /* :572-607 */
int  vo_pool_store_kv(vo_pool *p, int layer, int64_t seq, int start_pos, const float *k,
                      const float *v, int n_tok);                       /* :223-323; 0 ok, -1 no seq, -2 out of blocks */
int  vo_pool_seq_len(vo_pool *p, int64_t seq);
int  vo_pool_table(vo_pool *p, int layer, int64_t seq, int32_t *out, int cap); /* returns n blocks */
int  vo_pool_free_blocks(vo_pool *p, int layer);
int  vo_pool_set_free_list(vo_pool *p, const int32_t *ids, int n);      /* test set-up: same hand-out order on both sides */
void *vo_pool_layer_data(vo_pool *p, int layer);
int  vo_pool_attention(vo_pool *p, int layer, int64_t seq, const float *q, float *out,
                       int n_q_heads, float scale, float softcap, int window,
                       int kv_len);                                     /* :337-389 */

/* ---- model (runtime/config.go, loader.go, block.go, decode.go) ---------- */
typedef struct {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;
    float rms_eps, rope_theta;
    int rope_neox;           /* config.go:413, false for llama/gemma2 */
    int geglu;               /* MLPGeGLU, config.go:437-452 */
    int post_norms;          /* config.go:449 */
    float embed_scale;       /* config.go:440 (0 = off) */
    float attn_softcap;      /* config.go:441-445 */
    float final_softcap;
    int sliding_window;      /* 0 = off */
    int window_alternating;  /* odd layers slide (block.go:464-476) */
    int max_blocks;          /* per layer */
    int kv_f16;              /* 1: f16 pool (model.go:310-314 default) */
} vo_config;

typedef struct vo_model vo_model;
enum {  /* per-layer tensor slots */
    VO_T_ATTN_NORM, VO_T_WQ, VO_T_WK, VO_T_WV, VO_T_WO, VO_T_POST_ATTN_NORM,
    VO_T_FFN_NORM, VO_T_W1, VO_T_W3, VO_T_W2, VO_T_POST_FFN_NORM, VO_T_PER_LAYER
};
enum { VO_G_EMBED = 0, VO_G_FINAL_NORM = 1, VO_G_OUTPUT = 2 };

vo_model *vo_model_create(const vo_config *cfg);
void vo_model_destroy(vo_model *m);
/* data is copied/dequantized as runtime/loader.go:81-212, 275-288 prescribes:
 * projections keep Q4_0 raw (fused matmul), K-quants become F32 (loader.go:214-271),
 * embedding always F32, a Q4_0 output head becomes F32. */
int vo_model_set_layer_tensor(vo_model *m, int layer, int slot, int type, const void *data);
int vo_model_set_global_tensor(vo_model *m, int which, int type, const void *data);
vo_pool *vo_model_pool(vo_model *m);
/* One forward pass of n_tok tokens of one sequence starting at start_pos
 * (runtime/decode.go:339-461 for n_tok==1, :961-1096 for prefill, :1446-1569 verify).
 * logits: n_tok==1 or all_logits -> [n_tok, vocab]; else last token only -> [vocab].
 * hidden (optional): [(n_layers+1), n_tok, hidden] residual stream after embedding and after each layer. */
int vo_model_forward(vo_model *m, int64_t seq, const int32_t *tokens, int n_tok, int start_pos,
                     int all_logits, float *logits, float *hidden);
void vo_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
