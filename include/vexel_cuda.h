/*
 * vexel_cuda.h -- C ABI of the B200 (sm_100a) CUDA backend for the Vexel inference engine.
 *
 * This is the boundary a cgo wrapper binds.  Every entry point is extern "C", takes plain
 * pointers / integers / floats, and returns an int status (VX_OK == 0).  Device buffers are
 * raw device addresses carried as uint64_t: the Go side passes DevicePtr.addr + DevicePtr.offset
 * (the reference keeps GPU offsets separate from the base, inference/tensor/device.go:36-80).
 *
 * Two layers:
 *   1. Interface-level kernels, 1:1 with the reference's backend interfaces
 *      (inference/backend/backend.go).  Each declaration cites the method it implements.
 *   2. The batched decode fast path: model + device block pool + one call per scheduler step,
 *      replacing the per-sequence loop of inference/runtime/decode.go:612-654.
 *
 * Threading: a vx_ctx serialises its entry points with a mutex and makes its device current on
 * every call (goroutines migrate between OS threads).  All work runs on one stream per context.
 * There is no CPU fallback: without a CUDA device vx_init fails with VX_E_CUDA.
 */
#ifndef VEXEL_CUDA_H
#define VEXEL_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vx_ctx vx_ctx;
typedef struct vx_model vx_model;
typedef uint64_t vx_dptr; /* device address (base + offset already applied) */

enum {
    VX_OK = 0,
    VX_E_BAD_ARG = 1,     /* programmer error: the Go wrapper panics (void interface methods) */
    VX_E_CUDA = 2,        /* CUDA runtime error, text in vx_last_error */
    VX_E_OOM = 3,         /* device allocation failed: Alloc returns a nil DevicePtr (backend.go:315-317) */
    VX_E_OOM_BLOCKS = 4,  /* block pool exhausted (runtime/gpu_block_pool.go:200-204) */
    VX_E_NO_SEQ = 5,      /* unknown sequence id (runtime/gpu_block_pool.go:229-232) */
    VX_E_TIMEOUT = 6,     /* a bounded device-side wait gave up */
    VX_E_UNSUPPORTED = 7
};

/* GGUF tensor type ids (inference/pkg/gguf/gguf.go:40-75) accepted for weights. */
enum { VX_T_F32 = 0, VX_T_F16 = 1, VX_T_Q4_0 = 2, VX_T_Q4_K = 12, VX_T_Q6_K = 14 };

/* ------------------------------------------------------------------ lifecycle
 * replaces inference/backend/cuda/backend.go:15-37 (NewBackend stub). */
int vx_init(int device, vx_ctx **out);
int vx_destroy(vx_ctx *ctx);
const char *vx_last_error(vx_ctx *ctx);          /* never NULL */
int vx_device_index(vx_ctx *ctx);                /* Backend.Device(), backend.go:311 */

/* ------------------------------------------------------------------ memory
 * Backend.Alloc/Free/ToDevice/ToHost/Sync (backend.go:317-331); AllocPermanent and ResetPool
 * (runtime/gpu_block_pool.go:69-81, runtime/decode.go:366; inference/backend/backend.go:8-10);
 * BufferCopier.CopyBuffer (backend.go:38-43).  vx_alloc buffers are recycled wholesale by
 * vx_reset_pool; vx_alloc_permanent buffers live until vx_free / vx_destroy. */
int vx_alloc(vx_ctx *ctx, size_t bytes, vx_dptr *out);
int vx_alloc_permanent(vx_ctx *ctx, size_t bytes, vx_dptr *out);
int vx_free(vx_ctx *ctx, vx_dptr p);
int vx_reset_pool(vx_ctx *ctx);
int vx_h2d(vx_ctx *ctx, vx_dptr dst, const void *src, size_t bytes);
int vx_d2h(vx_ctx *ctx, void *dst, vx_dptr src, size_t bytes);
int vx_d2d(vx_ctx *ctx, vx_dptr dst, vx_dptr src, size_t bytes);
int vx_memset(vx_ctx *ctx, vx_dptr dst, int byte, size_t bytes);
int vx_sync(vx_ctx *ctx);

/* ------------------------------------------------------------------ Backend kernels (backend.go:333-390)
 * All operands are float32 on the device unless stated. */
int vx_matmul_f32(vx_ctx *, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k);    /* MatMul :338 */
int vx_matmul_f32_t(vx_ctx *, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k);  /* MatMulTransposed :341 */
int vx_rmsnorm(vx_ctx *, vx_dptr x, vx_dptr w, vx_dptr out, int rows, int cols, float eps);              /* RMSNorm :345 */
int vx_rope(vx_ctx *, vx_dptr q, vx_dptr k /*0 = nil*/, int head_dim, int n_heads, int n_kv_heads,
            int seq_len, int start_pos, int rope_dim, float theta, int neox);                            /* RoPE :352 */
int vx_silu(vx_ctx *, vx_dptr x, vx_dptr out, int n);                                                    /* SiLU :356 */
int vx_silu_mul(vx_ctx *, vx_dptr gate, vx_dptr up, vx_dptr out, int n);                                 /* SiLUMul :360 */
int vx_softmax(vx_ctx *, vx_dptr x, vx_dptr out, int rows, int cols);                                    /* Softmax :364 */
int vx_add(vx_ctx *, vx_dptr a, vx_dptr b, vx_dptr out, int n);                                          /* Add :367 */
int vx_mul(vx_ctx *, vx_dptr a, vx_dptr b, vx_dptr out, int n);                                          /* Mul :370 */
int vx_embedding(vx_ctx *, vx_dptr ids_i32, int n_tokens, vx_dptr table, vx_dptr out, int vocab, int dim); /* Embedding :374 */
int vx_sdpa(vx_ctx *, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int kv_len, int n_q_heads,
            int n_kv_heads, int head_dim, float scale, int kv_head_stride);                              /* SDPA :382 */
int vx_sdpa_prefill(vx_ctx *, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int seq_len, int n_q_heads,
                    int n_kv_heads, int head_dim, float scale);                                          /* SDPAPrefill :389 */

/* Optional capability interfaces */
int vx_matmul_q4_0(vx_ctx *, vx_dptr a, vx_dptr b_raw, vx_dptr out, int m, int n, int k); /* QuantizedMatMul.MatMulQ4_0 backend.go:50 */
int vx_matmul_q4_k(vx_ctx *, vx_dptr a, vx_dptr b_raw, vx_dptr out, int m, int n, int k); /* MatMulQ4_K :55 */
int vx_matmul_q6_k(vx_ctx *, vx_dptr a, vx_dptr b_raw, vx_dptr out, int m, int n, int k); /* MatMulQ6_K :60 */
/* The three calls above repack the GGUF blocks into the kernels' layout.  For weights that live in a vx_alloc_permanent
 * buffer (as runtime/loader.go:507-708 uploads them) the repacked copy is kept and reused by later calls on the same
 * tensor; vx_h2d / vx_d2d / vx_memset into the raw bytes and vx_free drop it.  A kernel of this library must not be pointed
 * at such a tensor as its OUTPUT once it has served as a weight (the reference never does).  0 switches the cache off. */
int vx_set_repack_cache(vx_ctx *ctx, int enable);
int vx_argmax(vx_ctx *, vx_dptr x, int n, int *out_index);                /* ArgmaxOps.Argmax :202 (synchronous, first max wins) */
int vx_argmax_rows(vx_ctx *, vx_dptr x, int rows, int cols, vx_dptr out_i32); /* batched form, asynchronous */
int vx_gelu(vx_ctx *, vx_dptr x, vx_dptr out, int n);                     /* GELUOps.GELU :220 */
int vx_gelu_mul(vx_ctx *, vx_dptr gate, vx_dptr up, vx_dptr out, int n);  /* GELUOps.GELUMul :224 */
int vx_scale(vx_ctx *, vx_dptr buf, float scale, int n);                  /* ScaleOps.ScaleBuffer :262 */
int vx_sdpa_softcap(vx_ctx *, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int kv_len, int n_q_heads,
                    int n_kv_heads, int head_dim, float scale, float softcap, int kv_head_stride);       /* SoftCapAttentionOps.SDPASoftCap :234 */
int vx_sdpa_prefill_softcap(vx_ctx *, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int seq_len,
                            int n_q_heads, int n_kv_heads, int head_dim, float scale, float softcap);    /* SDPAPrefillSoftCap :238 */
int vx_rope_freqs(vx_ctx *, vx_dptr q, vx_dptr k, vx_dptr freqs, int head_dim, int n_heads,
                  int n_kv_heads, int seq_len, int start_pos, int neox);                                 /* ScaledRoPEOps :246 */
/* bit-exact dequantisation of GGUF blocks to float32 (inference/pkg/gguf/dequant.go:16-56, 272-331, 342-396) */
int vx_dequantize(vx_ctx *, int type, vx_dptr raw, vx_dptr out_f32, int64_t n_elements);

/* PagedKVOps (backend.go:415-466).  Pool layout per layer:
 * element((blk*2 + isV)*bs*Hkv*D + off*Hkv*D + h*D + d). */
int vx_reshape_paged_kv(vx_ctx *, vx_dptr src, vx_dptr pool, vx_dptr page_table_i32, vx_dptr block_offsets_i32,
                        int n_tokens, int n_kv_heads, int head_dim, int block_size, int is_value);       /* ReshapePagedKV :424 */
int vx_reshape_paged_kv_f16(vx_ctx *, vx_dptr src, vx_dptr pool, vx_dptr page_table_i32, vx_dptr block_offsets_i32,
                            int n_tokens, int n_kv_heads, int head_dim, int block_size, int is_value);   /* ReshapePagedKVF16 :457 */
int vx_sdpa_paged_decode(vx_ctx *, vx_dptr q, vx_dptr pool, vx_dptr block_table_i32, vx_dptr out,
                         int n_blocks, int block_size, int n_q_heads, int n_kv_heads, int head_dim,
                         float scale, int tokens_in_last_block);                                         /* SDPAPagedDecode :432 */
int vx_sdpa_paged_decode_f16(vx_ctx *, vx_dptr q, vx_dptr pool, vx_dptr block_table_i32, vx_dptr out,
                             int n_blocks, int block_size, int n_q_heads, int n_kv_heads, int head_dim,
                             float scale, int tokens_in_last_block);                                     /* SDPAPagedDecodeF16 :436 */
/* block_tables: host array of batch device addresses; seq_lens: host array (as the Go slices are) */
int vx_sdpa_paged_decode_batched(vx_ctx *, vx_dptr q, vx_dptr pool, const vx_dptr *block_tables, vx_dptr out,
                                 int batch, int max_blocks, int block_size, int n_q_heads, int n_kv_heads,
                                 int head_dim, float scale, const int *seq_lens, int pool_is_f16);       /* SDPAPagedDecodeBatched :447 */
int vx_sdpa_paged_decode_multiquery(vx_ctx *, vx_dptr q, vx_dptr pool, vx_dptr block_table_i32, vx_dptr out,
                                    vx_dptr kv_lens_i32, int n_blocks, int block_size, int n_q_heads,
                                    int n_kv_heads, int head_dim, float scale, int query_len,
                                    int pool_is_f16);                                                    /* SDPAPagedDecodeMultiquery :463 */
/* No counterpart in the reference.  vx_sdpa_paged_decode_f16 for callers that must not allocate while they attend (all
 * HBM already given to the KV pool, a latency-critical section, a non-reentrant allocator): the split-K scratch is a fixed
 * 4 MiB device array inside the library instead of the context's growable scratch, and the call makes no cudaMalloc /
 * cudaFree / host heap allocation.  Sizes beyond the array (see the definition; also n_blocks > 65536 or a block size above
 * 16384) are refused with VX_E_BAD_ARG.  The first call on a device resolves the array's address and may make the driver
 * load this library's kernels for that device, which is driver-side work that can allocate: make one warm-up call per
 * device before the section that must not allocate, and before any stream capture.  Calls that overlap on the GPU share
 * the array and race. */
int vx_sdpa_paged_decode_f16_noalloc(vx_ctx *, vx_dptr q, vx_dptr pool, vx_dptr block_table_i32, vx_dptr out,
                                     int n_blocks, int block_size, int n_q_heads, int n_kv_heads, int head_dim,
                                     float scale, int tokens_in_last_block);
/* the same paged kernel with the Gemma-2 variants the CPU branch applies
 * (runtime/block.go:925-953): softcap > 0 and/or kv_start (first attended position) per query */
int vx_sdpa_paged_decode_ex(vx_ctx *, vx_dptr q, vx_dptr pool, vx_dptr block_table_i32, vx_dptr out,
                            int kv_start, int kv_len, int block_size, int n_q_heads, int n_kv_heads,
                            int head_dim, float scale, float softcap, int pool_is_f16);

/* ------------------------------------------------------------------ batched decode fast path */
typedef struct {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab;   /* runtime/config.go:98-109 */
    float rms_eps, rope_theta;
    int rope_neox;            /* config.go:119 */
    int geglu;                /* MLPGeGLU, config.go:437-452 */
    int post_norms;           /* config.go:129 */
    float embed_scale;        /* config.go:133, 0 = off */
    float attn_softcap;       /* config.go:127 */
    float final_softcap;      /* config.go:128 (monotone: applied to returned logits only) */
    int sliding_window;       /* config.go:121, 0 = off */
    int window_alternating;   /* odd layers slide, runtime/block.go:464-476 */
    int max_blocks;           /* physical 16-token blocks per layer (runtime/model.go:305-327) */
    int max_seqs;             /* concurrent sequences tracked by the pool */
    int max_batch_tokens;     /* upper bound on packed query rows per step */
    int max_blocks_per_seq;   /* block-table width = ceil(context limit / 16) */
} vx_model_config;

/* per-layer tensor slots, named after inference/runtime/block.go:256-266 */
enum {
    VX_W_ATTN_NORM, VX_W_WQ, VX_W_WK, VX_W_WV, VX_W_WO, VX_W_POST_ATTN_NORM,
    VX_W_FFN_NORM, VX_W_W1, VX_W_W3, VX_W_W2, VX_W_POST_FFN_NORM, VX_W_PER_LAYER
};
enum { VX_G_EMBED = 0, VX_G_FINAL_NORM = 1, VX_G_OUTPUT = 2 };

/* replaces NewModelRuntime + CopyWeightsToDevice + CreateGPUBlockPool
 * (runtime/model.go:56-96, runtime/loader.go:507-708, runtime/model.go:305-327) */
int vx_model_create(vx_ctx *ctx, const vx_model_config *cfg, vx_model **out);
int vx_model_destroy(vx_model *m);
/* raw GGUF tensor bytes, row-major [n_out][k] in GGUF block format; data_on_device != 0 means `data`
 * is a device address.  layer < 0 selects the global slots (VX_G_*). */
int vx_model_set_tensor(vx_model *m, int layer, int slot, int ggml_type, const void *data,
                        size_t bytes, int data_on_device);
int vx_model_finalize(vx_model *m);    /* repack for the MMA kernels, fuse QKV and gate|up */
int vx_model_get_config(vx_model *m, vx_model_config *out);

/* GGUF files (pkg/gguf/gguf.go:246-501): header, metadata and tensor table parsed on the host, tensor data mapped.
 * vx_gguf_open always returns a handle (close it); on failure vx_gguf_error says why, in the reference's words. */
typedef struct vx_gguf vx_gguf;
int vx_gguf_open(const char *path, vx_gguf **out);                                 /* gguf.Open :246 */
int vx_gguf_close(vx_gguf *g);
const char *vx_gguf_error(vx_gguf *g);
int vx_gguf_tensor_count(vx_gguf *g);
int vx_gguf_tensor_info(vx_gguf *g, int index, char *name, int name_cap, int *ggml_type, int *n_dims,
                        uint64_t *ne4, uint64_t *file_offset, uint64_t *bytes);     /* TensorInfo :208-214; ne in GGUF order */
int vx_gguf_meta(vx_gguf *g, const char *key, char *out, int cap);                  /* File.Metadata[key] as text; VX_E_NO_SEQ if absent */
/* extractModelConfig (gguf.go:503-584) + ModelConfigFromGGUF (runtime/config.go:388-507): fills the architecture
 * fields of *cfg and leaves max_blocks / max_seqs / max_batch_tokens / max_blocks_per_seq to the caller */
int vx_gguf_model_config(vx_gguf *g, vx_model_config *cfg);
/* LoadWeightsGGUF + CopyWeightsToDevice (runtime/loader.go:28-212, 507-708) into a model created from that config,
 * followed by vx_model_finalize */
int vx_model_load_gguf(vx_model *m, vx_gguf *g);

/* GPUBlockPool sequence bookkeeping, device-resident (runtime/gpu_block_pool.go:129-190, 572-635) */
int vx_seq_create(vx_model *m, int64_t seq_id);
int vx_seq_delete(vx_model *m, int64_t seq_id);
int vx_seq_truncate(vx_model *m, int64_t seq_id, int new_len);
int vx_seq_share(vx_model *m, int64_t src_seq, int64_t dst_seq, int n_tokens);
int vx_seq_len(vx_model *m, int64_t seq_id, int *out_len);
int vx_seq_block_table(vx_model *m, int64_t seq_id, int32_t *out, int cap, int *out_n); /* device -> host copy */
int vx_pool_stats(vx_model *m, int *total_blocks, int *free_blocks, int *shared_blocks);  /* BlockStats :610-625 */
int vx_pool_layer_ptr(vx_model *m, int layer, vx_dptr *out, size_t *bytes);
/* GPUBlockPool.freeList (runtime/gpu_block_pool.go:36, 200-219) as the stack it is, bottom first: the next block handed out
 * is the last entry.  *n_out = number of free blocks per layer. */
int vx_pool_free_list(vx_model *m, int32_t *out, int cap, int *n_out);
/* test/bench helper: give a sequence `len` tokens of KV filled with deterministic f16 noise (no forward pass) */
int vx_seq_fill_synthetic(vx_model *m, int64_t seq_id, int len, uint32_t seed);

/* Sampler.Config plus the uniform draw of one Sample call (pkg/sampler/sampler.go:9-14, 49-76, 206-218).
 * temperature 0 = greedy; top_k 0 = off; top_p 0 or >= 1 = off; u in [0,1) is what rng.Float32() returned. */
typedef struct { float temperature; int32_t top_k; float top_p; float u; } vx_sample_params;
/* Sampler.Sample for `rows` contiguous logits rows of n floats on the device (the rows are overwritten by
 * their probabilities); synchronous like ArgmaxOps.Argmax.  out_tokens is a host array. */
int vx_sample_rows(vx_ctx *, vx_dptr logits, int rows, int n, const vx_sample_params *params, int32_t *out_tokens);

/* One scheduler step over a ragged batch: replaces Scheduler.runDecodeStep's per-sequence calls
 * (scheduler/scheduler.go:290-303 -> runtime/decode.go:612-654).  Row i of the batch is sequence
 * seq_ids[i] fed q_lens[i] tokens (NULL = 1 each; >1 = speculative verify, decode.go:1446-1569)
 * starting at positions[i], which must equal the sequence's current length.  tokens holds
 * sum(q_lens) ids.  out_tokens receives the greedy (first-max) token of every packed row.
 * logits (optional, host) receives [sum(q_lens), vocab] float32. */
int vx_decode_step(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens,
                   const int32_t *positions, const int32_t *q_lens, int32_t *out_tokens,
                   float *logits);
/* vx_decode_step with options, for the two callers the plain call cannot serve.
 *  - Speculative verify with hidden states (VerifySpeculativeWithPagedKVAndHidden, runtime/decode.go:1446-1569): pass
 *    `hidden` (host, [output rows, hidden] float32) to receive the post-final-norm hidden state of every output row
 *    (decode.go:1543-1557), next to the logits.
 *  - A scheduler step that mixes decoding sequences with prompt chunks (Scheduler.runDecodeStep + runBatchedPrefill,
 *    scheduler/scheduler.go:245-303, 486-550, as ONE packed step): VX_STEP_PROMPT_ROWS makes multi-row entries prompt chunks
 *    (PrefillWithPagedKV semantics, decode.go:961-1096: an entry that starts at position 0 attends over its fresh float32 K/V;
 *    later chunks read the pages), VX_STEP_LAST_ROWS limits the outputs (tokens, logits, hidden, sampling records) to the last
 *    row of every entry, n_seqs rows in batch order.
 * params (optional): one sampling record per output row, as in vx_decode_step_sampled. */
#define VX_STEP_LAST_ROWS 1
#define VX_STEP_PROMPT_ROWS 2
int vx_decode_step_ex(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                      const int32_t *q_lens, int flags, const vx_sample_params *params, int32_t *out_tokens, float *logits,
                      float *hidden);
/* vx_prefill whose returned token is sampled (one record, for the last prompt position) */
int vx_prefill_sampled(vx_model *m, int64_t seq_id, const int32_t *tokens, int n_tokens, int start_pos,
                       const vx_sample_params *params, int32_t *out_token, float *logits);
/* vx_decode_step with on-device sampling in place of Scheduler.sampleToken's host path (scheduler/scheduler.go:783-820):
 * params holds one record per packed row. */
int vx_decode_step_sampled(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                           const int32_t *q_lens, const vx_sample_params *params, int32_t *out_tokens, float *logits);

/* Greedy generation of n_steps tokens for a fixed batch with the token feedback kept on the device (no host
 * round trip between steps).  tokens/positions describe the first step as in vx_decode_step (one token per
 * sequence).  out_tokens (optional, host) receives [n_steps, n_seqs]; device_ms (optional) the CUDA-event time of
 * the steps on the context's stream. */
int vx_decode_run(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                  int n_steps, int32_t *out_tokens, float *device_ms);
/* Prompt processing for one sequence (runtime/decode.go:961-1096): start_pos == 0 attends causally
 * over the fresh float32 K/V (SDPAPrefill), start_pos > 0 goes through the paged multi-query
 * kernel.  out_token / logits refer to the last prompt token. */
int vx_prefill(vx_model *m, int64_t seq_id, const int32_t *tokens, int n_tokens, int start_pos,
               int32_t *out_token, float *logits);

/* parity instrumentation: capture the residual stream after the embedding and after each layer of
 * the next forward ([n_layers+1, rows, hidden] float32), the idea of inference/debug's capture hooks. */
int vx_model_set_capture(vx_model *m, int enable);
int vx_model_get_capture(vx_model *m, float *host_out, size_t n_floats);
/* slot mapping / positions / cu_seqlens produced by the packing kernel for the last step */
int vx_model_get_packing(vx_model *m, int32_t *cu_seqlens, int32_t *slot_mapping, int32_t *row_kv_len,
                         int n_seqs, int n_rows);
/* counters: kernels launched and steps run since creation */
int vx_model_counters(vx_model *m, uint64_t *kernel_launches, uint64_t *steps);
/* steps replayed from a CUDA graph so far, and how many times an executable graph was taken over by in-place update
 * because only the attention grids had changed */
int vx_model_graph_stats(vx_model *m, uint64_t *replays, uint64_t *takeovers);
/* timing of the dominant kernel class inside vx_decode_step (CUDA events on the context's stream):
 * which: 0 = paged attention, 1 = quantised projections.  Returns accumulated ms and launch count. */
int vx_model_kernel_time(vx_model *m, int which, int enable, float *ms, uint64_t *launches);
/* deterministic synthetic Q4_0 weights generated on the device: ~N(0, sigma) quantised with
 * d = signed-absmax / -8, q = clamp(round(x/d) + 8, 0, 15); writes GGUF Q4_0 blocks */
int vx_synth_q4_0(vx_ctx *ctx, vx_dptr dst_raw, int64_t n_elements, uint64_t seed, float sigma);
/* bench helper: valid Q4_K (type 12) or Q6_K (type 14) blocks with hashed payload and super-scales chosen for a
 * dequantised standard deviation near sigma; for timing runs on K-quant model shapes */
int vx_synth_kquant(vx_ctx *ctx, vx_dptr dst_raw, int ggml_type, int64_t n_elements, uint64_t seed, float sigma);
/* bench helper: permute the pool's free list so that consecutive logical blocks land on scattered
 * physical blocks; only valid while no sequence holds blocks */
int vx_pool_shuffle_free_list(vx_model *m, uint32_t seed);
/* GGUF bytes of all weights read once per step (projections, output head, norm vectors) */
int vx_model_weight_bytes(vx_model *m, uint64_t *bytes);
/* activation terms fed to the tensor cores by the projections: 2 = fp16 hi+lo split (float32-faithful,
 * default), 1 = single fp16 (half the MMA work, ~2e-4 relative rounding per projection) */
int vx_set_gemm_terms(int terms);
/* steps of a recurring shape are replayed from CUDA graphs (default on; 0 = launch every kernel individually) */
int vx_set_graphs(int enable);
/* failure-path self-test: a kernel waits, with a limit of limit_us microseconds, on a barrier that is never signalled; it
 * must return (reached_end = 1) and the next vx_sync must report VX_E_TIMEOUT while the context stays usable.  This is
 * how every device-side wait of the library behaves when its peer never shows up; no counterpart in the reference. */
int vx_selftest_bounded_wait(vx_ctx *ctx, int limit_us, int *reached_end);
/* batches with at least this many rows run the projections on the tcgen05 kernel (default 17;
 * 0 = always the mma.sync kernel) */
int vx_set_tc_min_rows(int rows);
/* Q4_0, Q4_K and Q6_K projections of 17..64 batch rows run on the persistent tcgen05 kernel (one CTA per SM walking weight
 * tiles, its pipeline kept full across tiles; Q4_K adds a small kernel for its minima).  mode 0 = one CTA per tile; 1 =
 * persistent with split-K slices aligned to tiles; 2 (default) = persistent, and where it is cheaper the stages of all tiles
 * are cut into one equal run per CTA (a tile's partial sums then come from the CTAs that share it); 3 = that cut wherever it
 * applies, 4 = as 2 but the K-quant formats on the one-CTA-per-tile kernel (both for timing comparisons).  No counterpart in
 * the reference. */
int vx_set_persistent_projections(int mode);
/* Q4_0 projections of 1..4 batch rows (Q4_K: 1..3) run on the weight-streaming mma.sync kernel (the single-sequence decode of
 * runtime/block.go:947-1060: one quantised mat-vec per projection); 0 = the staged mma.sync kernel as for 5..16 rows.
 * Default on. */
int vx_set_thin_batch_projections(int enable);
/* timing experiments only: bit 0 skips every projection launch of a step, bit 1 the row kernels, bit 2 the attention
 * kernels (the step's results are then meaningless; what remains is timed to attribute a step's time to kernel classes).
 * 0 restores the real step. */
int vx_debug_skip(int mask);
/* projection kernels are launched as programmatic dependents of the kernel before them (their set-up and first weight
 * tiles overlap its tail); 0 = plain stream order.  Default on.  No counterpart in the reference. */
int vx_set_dependent_launch(int enable);

/* ------------------------------------------------------------------ tensor parallelism (one process per GPU, NCCL)
 * No counterpart in the reference, which keeps whole Wq..W2 per block on one device (runtime/block.go:256-266).  A model too
 * large for (or too slow on) one GPU is split Megatron-style: Wq/Wk/Wv and W1/W3 by output rows, Wo and W2 by input columns
 * (their outputs are summed over the ranks with ncclAllReduce on the compute stream, once after each), the output head by
 * vocabulary rows (local first-maximum, one all-gather of (value, index) pairs).  Every rank runs the same step on the same
 * token ids; the KV pool of a rank holds its own KV heads only.
 *   rank 0: vx_tp_unique_id(buf, 128) and hand buf to the other ranks; every rank: vx_tp_init(ctx, buf, rank, world);
 *   vx_model_create with the LOCAL counts (n_heads / world, n_kv_heads / world, ffn / world, vocab / world),
 *   vx_model_enable_tp(model, vocab_full), then vx_model_set_tensor with the rank's slices (the embedding and the norms whole).
 * Steps are greedy (vx_decode_step, vx_prefill, vx_decode_run); logits, if requested, are the rank's vocabulary slice. */
int vx_tp_unique_id(void *out, int cap);
int vx_tp_init(vx_ctx *ctx, const void *unique_id, int rank, int world);
int vx_tp_shutdown(vx_ctx *ctx);
int vx_model_enable_tp(vx_model *m, int vocab_full);

/* ------------------------------------------------------------------ continuous-batching scheduler
 * The host loop of inference/scheduler (Scheduler.step / runDecodeStep, scheduler/scheduler.go:168-483; Sequence state
 * machine, scheduler/sequence.go:15-80) over vx_decode_step_ex, for embedders without the Go scheduler.  Every iteration
 * is ONE packed step: the decoding sequences plus the next chunk of each prompt being read, up to the model's
 * max_batch_tokens.  The batch is formed in arrival order; a request is admitted when the pool can hold its prompt plus its
 * token limit, waits otherwise (taking no batch slot), and is refused if it could never fit; requests without a limit
 * reserve their prompt and may be preempted when the pool runs dry. */
typedef struct vx_sched vx_sched;
typedef struct {
    int max_batch_size;   /* Config.MaxBatchSize, scheduler.go:23 */
    int max_sequences;    /* Config.MaxSequences :24 (enforced here; 0 = unlimited) */
    int max_tokens;       /* Config.MaxTokens :25 (0 = unlimited) */
    int eos_token;        /* stop token id, < 0 = none */
    float temperature;    /* Config.SamplerConfig (sampler.Config :9-14): 0 = greedy */
    int top_k;
    float top_p;
    uint64_t seed;        /* seeds the scheduler's own uniform generator (the reference seeds math/rand, whose stream is not reproduced) */
} vx_sched_config;
typedef struct {          /* SchedulerMetrics, scheduler.go:30-38 */
    int active_sequences, completed_sequences, total_tokens, prefill_tokens, decode_tokens;
    double prefill_seconds, decode_seconds;
} vx_sched_metrics;
int vx_sched_create(vx_model *m, const vx_sched_config *cfg, vx_sched **out);
int vx_sched_destroy(vx_sched *s);
int vx_sched_add_sequence(vx_sched *s, int64_t id, const int32_t *prompt, int n_prompt, int max_tokens);   /* AddSequence :645-676 */
int vx_sched_remove_sequence(vx_sched *s, int64_t id);                                                     /* RemoveSequence :690-698 */
int vx_sched_step(vx_sched *s, int *n_active_out);                                                         /* step :168-203 */
/* TokenChan drain (sequence.go:70-80).  *finished: 0 = still running, 1 = ended and drained, 2 = ended because the request
 * was refused: its prompt plus token limit can never fit the block pool or one block table (where the reference stops its
 * whole loop with an allocation error, scheduler.go:134-136).  Requests whose end has been reported are forgotten once a few
 * hundred of them have piled up (VX_E_NO_SEQ from then on), or when their id is added again. */
int vx_sched_poll(vx_sched *s, int64_t id, int32_t *out, int cap, int *n_out, int *finished);
int vx_sched_get_metrics(vx_sched *s, vx_sched_metrics *out);                                                /* Metrics :475-481 */
/* how many times a sequence was preempted to free blocks (its tokens are read again later), and how many requests were
 * refused; no counterpart in the reference, whose loop ends on the first allocation failure */
int vx_sched_get_pressure(vx_sched *s, uint64_t *preemptions, uint64_t *refused);
int vx_model_max_blocks(vx_model *m);   /* physical blocks per layer of the model's pool */

#ifdef __cplusplus
}
#endif
#endif
