// The batched decode fast path: model weights, the device-resident block pool, and one call per
// scheduler step.  Replaces the per-sequence loop of inference/runtime/decode.go:612-654 and the host
// bookkeeping of inference/runtime/gpu_block_pool.go with device kernels:
//   pack_kernel        cu_seqlens / slot mapping / block tables / split-K work lists by prefix scans
//   add_norm_split     residual add (+ Gemma post-norm) + RMSNorm + fp16 hi/lo split for the projections
//   rope_append        RoPE on q,k and the f32->f16 append of k,v into the paged pool
//   vxp_attention      paged FlashDecoding (vx_paged.cu)       vxq_gemm  dequant-fused projections (vx_quant.cu)
// Layer order and arithmetic follow inference/runtime/block.go:763-1081.
#include <math.h>
#include <string.h>

#include <cooperative_groups.h>

#include <algorithm>
#include <map>
#include <tuple>

#include "vx_paged.cuh"

namespace {

constexpr int BS = 16;   // tokens per KV block (runtime/decode.go:351)
constexpr int MAX_PARTS = 8;
constexpr int MAX_WORK = 32768;

struct ColW { VxWeight w; int col; };      // a projection writing output columns [col, col + w.n)
struct LayerW {
    std::vector<ColW> wqkv;                // one fused Wq|Wk|Wv matrix when the three share a block format, else one per format run
    VxWeight wo, w13, w2;
    float *attn_norm = nullptr, *ffn_norm = nullptr, *post_attn_norm = nullptr, *post_ffn_norm = nullptr;
};
struct RawTensor { int type = -1; void *dev = nullptr; size_t bytes = 0; };

}  // namespace

struct vx_model {
    vx_ctx *c = nullptr;
    vx_model_config cfg{};
    bool finalized = false;
    std::vector<RawTensor> raw;           // [layer][VX_W_PER_LAYER] + 3 globals, until finalize
    std::vector<LayerW> layers;
    std::vector<void *> owned;            // device allocations freed at destroy
    RawTensor embed;                      // kept in GGUF form; rows are dequantised on lookup
    float *final_norm = nullptr;
    VxWeight w_out;
    size_t weight_bytes = 0;
    // ---- pool
    __half *pool = nullptr; size_t layer_stride = 0;      // elements per layer
    int32_t *d_tables = nullptr; const int32_t **d_table_ptrs = nullptr;
    int32_t *d_seq_len = nullptr, *d_n_blocks = nullptr, *d_free_list = nullptr, *d_free_top = nullptr, *d_refcnt = nullptr;
    int32_t *d_status = nullptr;
    std::unordered_map<int64_t, int> seq_slot;
    std::vector<int> free_slots, h_seq_len, h_n_blocks;
    int h_free = 0;
    // ---- per-step buffers
    int32_t *d_step_in = nullptr, *h_step_in = nullptr;   // pinned staging + device copy
    int32_t *d_cu = nullptr, *d_row_slot = nullptr, *d_row_pos = nullptr, *d_slot_map = nullptr, *d_row_kv_len = nullptr,
            *d_row_kv_start = nullptr, *d_row_route = nullptr, *d_last_row = nullptr;
    unsigned int *d_row_bound = nullptr;         // per packed row: upper bound of the attention output's magnitude (float bits)
    float *d_hidden = nullptr;                   // post-final-norm hidden states of the output rows of the last step
    bool fast_attn_shape = false;                // the paged attention kernels that walk work lists cover this head shape
    // tensor parallelism: this model is one rank's slice (local heads / FFN columns / vocabulary rows in cfg); the embedding
    // table covers the whole vocabulary
    bool tp = false; int vocab_full = 0; float *ar_buf = nullptr; void *tp_scratch = nullptr;
    int4 *d_work[2] = {nullptr, nullptr}; int32_t *d_rws[2] = {nullptr, nullptr}; int32_t *d_n_work[2] = {nullptr, nullptr};
    float *d_partials = nullptr;
    float *d_cos = nullptr, *d_sin = nullptr, *d_freq = nullptr;
    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *parts = nullptr, *logits = nullptr;
    size_t parts_cap = 0;
    VxSplit sp_h{}, sp_q{}, sp_f{};
    int32_t *d_out_tok = nullptr, *h_out_tok = nullptr;
    void *d_sample = nullptr;                    // per-row sampling parameters of the current step
    float *capture = nullptr; bool capture_on = false; int capture_rows = 0;
    int last_rows = 0, last_seqs = 0;
    uint64_t steps = 0;
    // CUDA graphs of whole steps, keyed by everything that shapes the launches (see enqueue_step)
    struct GraphKey {
        int n_seqs, rows, logit_rows, chunk0, chunk1, nw0, nw1, out_flags;
        bool operator<(const GraphKey &o) const {
            return std::tie(n_seqs, rows, logit_rows, chunk0, chunk1, nw0, nw1, out_flags) <
                   std::tie(o.n_seqs, o.rows, o.logit_rows, o.chunk0, o.chunk1, o.nw0, o.nw1, o.out_flags);
        }
    };
    struct GraphEntry { cudaGraphExec_t exec = nullptr; int seen = 0; uint64_t launches = 0; };
    std::map<GraphKey, GraphEntry> graphs;
    uint64_t graph_replays = 0, graph_updates = 0;
    int32_t *d_run_out = nullptr; size_t run_out_cap = 0;
    // kernel timing
    bool time_on[2] = {false, false}; float time_ms[2] = {0, 0}; uint64_t time_n[2] = {0, 0};
    std::vector<cudaEvent_t> ev_pool; std::vector<std::pair<int, int>> ev_used;   // (which, index of start event)
    size_t ev_next = 0;
};

namespace {

int model_alloc(vx_model *m, size_t bytes, void **out) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 16);
    if (e != cudaSuccess) { cudaGetLastError(); return vx_fail(m->c, VX_E_OOM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e)); }
    m->owned.push_back(p);
    *out = p;
    return VX_OK;
}
template <typename T> int model_alloc_t(vx_model *m, size_t n, T **out) { return model_alloc(m, n * sizeof(T), (void **)out); }

void slot_dims(const vx_model_config &c, int slot, int *n, int *k) {
    int qd = c.n_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
    switch (slot) {
    case VX_W_WQ: *n = qd; *k = c.hidden; break;
    case VX_W_WK: case VX_W_WV: *n = kvd; *k = c.hidden; break;
    case VX_W_WO: *n = c.hidden; *k = qd; break;
    case VX_W_W1: case VX_W_W3: *n = c.ffn; *k = c.hidden; break;
    case VX_W_W2: *n = c.hidden; *k = c.ffn; break;
    default: *n = 1; *k = c.hidden; break;
    }
}
size_t type_row_bytes(int type, int k) {
    switch (type) {
    case VX_T_F32: return (size_t)k * 4;
    case VX_T_F16: return (size_t)k * 2;
    case VX_T_Q4_0: return (size_t)(k / 32) * 18;
    case VX_T_Q4_K: return (size_t)(k / 256) * 144;
    case VX_T_Q6_K: return (size_t)(k / 256) * 210;
    default: return 0;
    }
}

// ------------------------------------------------------------------ sequence bookkeeping kernels
// runtime/gpu_block_pool.go:210-219 (releaseBlock) applied to table entries [keep, n_blocks), in table order
__global__ void seq_release_kernel(int32_t *tables, int width, int32_t *n_blocks, int32_t *seq_len, int32_t *free_list,
                                   int32_t *free_top, int32_t *refcnt, int slot, int keep, int new_len) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int nb = n_blocks[slot], top = *free_top;
    for (int i = keep; i < nb; i++) {
        int b = tables[(size_t)slot * width + i];
        int rc = refcnt[b];
        if (rc <= 1) { refcnt[b] = 0; free_list[top++] = b; }
        else refcnt[b] = rc - 1;
    }
    *free_top = top;
    if (keep < nb) n_blocks[slot] = keep;
    seq_len[slot] = new_len;
}
// runtime/gpu_block_pool.go:572-607
__global__ void seq_share_kernel(int32_t *tables, int width, int32_t *n_blocks, int32_t *seq_len, int32_t *refcnt, int src, int dst,
                                 int nb, int n_tokens) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int dn = n_blocks[dst];
    for (int i = 0; i < nb; i++) {
        int b = tables[(size_t)src * width + i];
        tables[(size_t)dst * width + dn + i] = b;
        refcnt[b]++;
    }
    n_blocks[dst] = dn + nb;
    if (n_tokens > seq_len[dst]) seq_len[dst] = n_tokens;
}
// grows one sequence to new_len tokens (allocBlock order of runtime/gpu_block_pool.go:200-208: pop from the end)
__global__ void seq_grow_kernel(int32_t *tables, int width, int32_t *n_blocks, int32_t *seq_len, int32_t *free_list,
                                int32_t *free_top, int32_t *refcnt, int slot, int new_len, int32_t *status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int need = (new_len + BS - 1) / BS, nb = n_blocks[slot], top = *free_top;
    if (need - nb > top || need > width) { *status = VX_E_OOM_BLOCKS; return; }
    for (; nb < need; nb++) { int b = free_list[--top]; refcnt[b] = 1; tables[(size_t)slot * width + nb] = b; }
    n_blocks[slot] = nb; *free_top = top;
    if (new_len > seq_len[slot]) seq_len[slot] = new_len;
}
__global__ void init_free_list_kernel(int32_t *free_list, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) free_list[i] = i;   // ascending, so the first pop is n-1 (runtime/gpu_block_pool.go:114-116)
}
__global__ void init_table_ptrs_kernel(const int32_t **ptrs, const int32_t *tables, int width, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) ptrs[i] = tables + (size_t)i * width;
}
__device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16; return x;
}
// fills the KV of positions [0,len) of one sequence in every layer with fp16 noise in [-0.25, 0.25)
__global__ void fill_noise_kernel(__half *pool, size_t layer_stride, int n_layers, const int32_t *table, int len, int hs, uint32_t seed) {
    size_t per_layer = (size_t)len * hs * 2;   // K and V
    size_t total = per_layer * n_layers;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int layer = (int)(idx / per_layer); size_t r = idx % per_layer;
        int is_v = (int)(r / ((size_t)len * hs)); size_t r2 = r % ((size_t)len * hs);
        int pos = (int)(r2 / hs), e = (int)(r2 % hs);
        size_t part = (size_t)BS * hs;
        size_t dst = (size_t)layer * layer_stride + (size_t)table[pos / BS] * 2 * part + (is_v ? part : 0) + (size_t)(pos % BS) * hs + e;
        uint32_t h = hash32((uint32_t)idx * 2654435761u + seed);
        pool[dst] = __float2half_rn(((int)(h & 0xFFFF) - 32768) * (0.25f / 32768.f));
    }
}
// random permutation of the free list by sorting on hashed keys (single block, bitonic-free: rank by counting)
__global__ void shuffle_free_list_kernel(int32_t *free_list, int32_t *tmp, int n, uint32_t seed) {
    // rank of element i = number of elements with a smaller (hash, index) key
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t ki = hash32((uint32_t)i ^ seed);
        int rank = 0;
        for (int j = 0; j < n; j++) { uint32_t kj = hash32((uint32_t)j ^ seed); rank += (kj < ki) || (kj == ki && j < i); }
        tmp[rank] = free_list[i];
    }
}

// ------------------------------------------------------------------ the packing kernel (one CTA)
// step_in = [n_seqs slots][n_seqs q_lens][n_seqs positions][n_seqs routes][n_rows tokens]
// route of a batch entry: 0 = its rows go through the split-K work lists, otherwise another attention kernel serves them
struct PackArgs {
    const int32_t *step_in; int n_seqs, n_rows;
    int32_t *row_route, *last_row;
    int32_t *tables; int width; int32_t *seq_len, *n_blocks, *free_list, *free_top, *refcnt, *status;
    int32_t *cu, *row_slot, *row_pos, *slot_map, *row_kv_len, *row_kv_start;
    int window;                          // 0 = no sliding layers
    int4 *work0, *work1; int32_t *rws0, *rws1, *n_work0, *n_work1; int chunk0, chunk1, max_work;
};
__global__ void __launch_bounds__(1024) pack_kernel(PackArgs a) {
    __shared__ int tmp[33];
    __shared__ int s_err, s_ovf;
    const int32_t *slots = a.step_in, *qlens = a.step_in + a.n_seqs, *positions = a.step_in + 2 * a.n_seqs, *routes = a.step_in + 3 * a.n_seqs;
    if (threadIdx.x == 0) { s_err = 0; s_ovf = 0; }
    __syncthreads();
    // pass A: validate, prefix sums of q_len (rows) and of newly needed blocks; nothing is modified yet
    int row_base = 0, need_base = 0;
    for (int i0 = 0; i0 < a.n_seqs; i0 += blockDim.x) {
        int i = i0 + threadIdx.x, ql = 0, need = 0;
        if (i < a.n_seqs) {
            int s = slots[i]; ql = qlens[i];
            int start = a.seq_len[s];
            if (positions[i] != start || ql <= 0) atomicExch(&s_err, VX_E_BAD_ARG);
            int nb_new = (start + ql + BS - 1) / BS;
            if (nb_new > a.width) atomicExch(&s_err, VX_E_OOM_BLOCKS);
            need = max(0, nb_new - a.n_blocks[s]);
        }
        int tq, tn;
        int oq = vx_block_excl_scan(ql, tmp, &tq);
        int on = vx_block_excl_scan(need, tmp, &tn);
        if (i < a.n_seqs) { a.cu[i] = row_base + oq; a.row_kv_start[i] = need_base + on; /* scratch: block offset */ }
        row_base += tq; need_base += tn;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        a.cu[a.n_seqs] = row_base;
        if (row_base != a.n_rows) s_err = VX_E_BAD_ARG;
        if (need_base > *a.free_top) s_err = VX_E_OOM_BLOCKS;
    }
    __syncthreads();
    if (s_err) {
        // a refused step must not touch anybody's KV: the kernels that follow see no work items and no pool slot
        for (int t = threadIdx.x; t <= a.n_rows; t += blockDim.x) {
            a.rws0[t] = 0; a.rws1[t] = 0;
            if (t < a.n_rows) { a.slot_map[t] = -1; a.row_kv_len[t] = 0; a.row_kv_start[t] = 0; a.row_route[t] = 0; a.row_pos[t] = 0; a.row_slot[t] = slots[0]; }
        }
        for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x) a.last_row[i] = 0;
        if (threadIdx.x == 0) { *a.status = s_err; *a.n_work0 = 0; *a.n_work1 = 0; }
        return;
    }
    // pass B: pop blocks in batch order (sequence i takes the pops numbered [off_i, off_i + need_i) from the end of the stack)
    const int top = *a.free_top;
    __syncthreads();
    for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x) {
        int s = slots[i], ql = qlens[i], start = a.seq_len[s];
        int nb = a.n_blocks[s], nb_new = (start + ql + BS - 1) / BS, off = a.row_kv_start[i];
        for (int j = 0; nb + j < nb_new; j++) {
            int b = a.free_list[top - 1 - (off + j)];
            a.refcnt[b] = 1;
            a.tables[(size_t)s * a.width + nb + j] = b;
        }
        if (nb_new > nb) a.n_blocks[s] = nb_new;
        a.seq_len[s] = start + ql;
    }
    __syncthreads();
    if (threadIdx.x == 0) *a.free_top = top - need_base;
    // per-row arrays
    for (int t = threadIdx.x; t < a.n_rows; t += blockDim.x) {
        int lo = 0, hi = a.n_seqs;                       // last i with cu[i] <= t
        while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (a.cu[mid] <= t) lo = mid; else hi = mid; }
        int s = slots[lo], pos = positions[lo] + (t - a.cu[lo]);
        a.row_slot[t] = s; a.row_pos[t] = pos; a.row_route[t] = routes[lo];
        a.slot_map[t] = a.tables[(size_t)s * a.width + pos / BS] * BS + pos % BS;
        a.row_kv_len[t] = pos + 1;
    }
    for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x) a.last_row[i] = a.cu[i] + qlens[i] - 1;
    __syncthreads();
    for (int t = threadIdx.x; t < a.n_rows; t += blockDim.x)
        a.row_kv_start[t] = a.window > 0 ? max(0, a.row_pos[t] + 1 - a.window) : 0;   // runtime/block.go:925-929
    __syncthreads();
    int n0 = vx_build_work(a.n_rows, nullptr, a.row_kv_len, a.row_route, BS, a.chunk0, a.work0, a.rws0, a.max_work, &s_ovf, tmp);
    if (threadIdx.x == 0) *a.n_work0 = n0;
    if (a.window > 0) {
        int n1 = vx_build_work(a.n_rows, a.row_kv_start, a.row_kv_len, a.row_route, BS, a.chunk1, a.work1, a.rws1, a.max_work, &s_ovf, tmp);
        if (threadIdx.x == 0) *a.n_work1 = n1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_ovf) *a.status = VX_E_BAD_ARG;
}

// cos/sin of angle = float32(pos) * freq[j], evaluated in float64 and rounded once (backend/cpu/cpu.go:256-260)
__global__ void rope_table_kernel(const int32_t *row_pos, const float *freq, float *cs, float *sn, int n_rows, int half) {
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_rows * half) return;
    int t = idx / half, j = idx % half;
    float angle = __fmul_rn((float)row_pos[t], freq[j]);
    cs[idx] = (float)cos((double)angle); sn[idx] = (float)sin((double)angle);
}

// ------------------------------------------------------------------ embedding (GGUF rows dequantised on lookup)
__global__ void embed_kernel(const int32_t *tokens, const void *table, int type, float *x, int hidden, int vocab, float scale) {
    int t = blockIdx.x, id = tokens[t];
    float *o = x + (size_t)t * hidden;
    if (id < 0 || id >= vocab) { for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = 0.f; return; }
    if (type == VX_T_Q4_0) {
        const uint8_t *row = (const uint8_t *)table + (size_t)id * (hidden / 32) * 18;
        for (int j = threadIdx.x; j < hidden / 2; j += blockDim.x) {     // one packed byte per iteration
            int b = j >> 4, i = j & 15;
            const uint8_t *blk = row + b * 18;
            float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
            uint8_t bv = blk[2 + i];
            float lo = __fmul_rn(d, (float)((int)(bv & 0xF) - 8)), hi = __fmul_rn(d, (float)((int)(bv >> 4) - 8));
            if (scale != 0.f) { lo = __fmul_rn(lo, scale); hi = __fmul_rn(hi, scale); }
            o[b * 32 + i] = lo; o[b * 32 + i + 16] = hi;
        }
    } else {
        const float *row = (const float *)table + (size_t)id * hidden;
        for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = scale != 0.f ? __fmul_rn(row[j], scale) : row[j];
    }
}

// ------------------------------------------------------------------ residual add + RMSNorm + split
// x[row] += (post_w ? rmsnorm(sum parts)*post_w : sum parts);  y = rmsnorm(x)*w;  y -> fp16 hi/lo (+ per-block sums).
// n_parts == 0 skips the add; w == nullptr skips the norm/split.  One CTA of 1024 threads per row, row in registers.
// row_idx (optional, only with n_parts == 0): CTA r reads row row_idx[r] of x and writes split row r (the final norm of
// the last row of every sequence).  normed_out (optional): the normalised row as float32 [r][hidden], which is the
// post-final-norm hidden state VerifySpeculativeWithPagedKVAndHidden returns (runtime/decode.go:1543-1557).
template <int NC>
__global__ void __launch_bounds__(VX_ROW_THREADS)
add_norm_split_kernel(float *x, const float *parts, int n_parts, size_t part_stride, int part_ld, const float *post_w, const float *w,
                      float eps, int hidden, VxSplit s, float *capture, const int32_t *row_idx, float *normed_out) {
    __shared__ float red[32];
    vx_pdl_wait();             // (chained launch: the kernel before this one has completed)
    vx_pdl_trigger();          // the projection that follows may become resident and fetch its first weights now
    const int r = blockIdx.x;
    float *xr = x + (size_t)(row_idx ? row_idx[r] : r) * hidden;
    float4 v[NC];
    const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
        v[c] = k0 < hidden ? *reinterpret_cast<const float4 *>(xr + k0) : z4;
    }
    if (n_parts > 0) {
        float4 a[NC];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < NC; c++) {
            int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
            a[c] = z4;
            if (k0 < hidden)
                for (int p = 0; p < n_parts; p++) {
                    float4 t = *reinterpret_cast<const float4 *>(parts + p * part_stride + (size_t)r * part_ld + k0);
                    a[c].x += t.x; a[c].y += t.y; a[c].z += t.z; a[c].w += t.w;
                }
            ss = fmaf(a[c].x, a[c].x, fmaf(a[c].y, a[c].y, fmaf(a[c].z, a[c].z, fmaf(a[c].w, a[c].w, ss))));
        }
        if (post_w) {   // Gemma 2 post-norm, runtime/block.go:985-987 / 1067-1070
            ss = block_sum(ss, red);
            float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps));
#pragma unroll
            for (int c = 0; c < NC; c++) {
                int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
                if (k0 < hidden) {
                    float4 pw = *reinterpret_cast<const float4 *>(post_w + k0);
                    a[c].x = __fmul_rn(__fdiv_rn(a[c].x, rms), pw.x); a[c].y = __fmul_rn(__fdiv_rn(a[c].y, rms), pw.y);
                    a[c].z = __fmul_rn(__fdiv_rn(a[c].z, rms), pw.z); a[c].w = __fmul_rn(__fdiv_rn(a[c].w, rms), pw.w);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < NC; c++) {
            int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
            v[c].x = __fadd_rn(v[c].x, a[c].x); v[c].y = __fadd_rn(v[c].y, a[c].y);
            v[c].z = __fadd_rn(v[c].z, a[c].z); v[c].w = __fadd_rn(v[c].w, a[c].w);
            if (k0 < hidden) *reinterpret_cast<float4 *>(xr + k0) = v[c];
        }
    }
    if (capture) {
#pragma unroll
        for (int c = 0; c < NC; c++) {
            int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
            if (k0 < hidden) *reinterpret_cast<float4 *>(capture + (size_t)r * hidden + k0) = v[c];
        }
    }
    if (!w) return;
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NC; c++) ss = fmaf(v[c].x, v[c].x, fmaf(v[c].y, v[c].y, fmaf(v[c].z, v[c].z, fmaf(v[c].w, v[c].w, ss))));
    ss = block_sum(ss, red);
    const float rms = __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps));   // backend/cpu/cpu.go:213-218
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
        if (k0 < hidden) {
            float4 ww = *reinterpret_cast<const float4 *>(w + k0);
            v[c].x = __fmul_rn(__fdiv_rn(v[c].x, rms), ww.x); v[c].y = __fmul_rn(__fdiv_rn(v[c].y, rms), ww.y);
            v[c].z = __fmul_rn(__fdiv_rn(v[c].z, rms), ww.z); v[c].w = __fmul_rn(__fdiv_rn(v[c].w, rms), ww.w);
            if (normed_out) *reinterpret_cast<float4 *>(normed_out + (size_t)r * hidden + k0) = v[c];
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[c].x), fabsf(v[c].y)), fmaxf(fabsf(v[c].z), fabsf(v[c].w))));
    }
    amax = block_max(amax, red);
    float sc, inv;
    vx_row_scale(amax, sc, inv);
    if (threadIdx.x == 0) s.scale[r] = sc;
    __half *hi = s.hi + (size_t)r * s.k_pad, *lo = s.lo + (size_t)r * s.k_pad;
    float *bs = s.bsum + (size_t)r * (s.k_pad / 32);
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
        if (k0 < s.k_pad) {
            const float t[4] = {v[c].x * inv, v[c].y * inv, v[c].z * inv, v[c].w * inv};
            vx_split_store4(t, hi, lo, bs, k0);
        }
    }
}

// ------------------------------------------------------------------ RoPE + KV append
// qkv row = [q (Hq*D) | k (Hkv*D) | v (Hkv*D)] float32.  q and k are rotated in place (backend/cpu/cpu.go:226-303);
// k and v are rounded to fp16 (round-to-nearest-even, as reshape_paged_kv_f16) and written to the row's pool slot.
constexpr int ROPE_HEADS = 4;   // heads per CTA
// src holds n_parts split-K partial results [n_parts][rows][ld] of the fused QKV projection; their sum is the row.
// grid: (rows, ceil((Hq + 2*Hkv) / ROPE_HEADS)); the heads of a row are q heads, then k heads, then v heads.
__global__ void __launch_bounds__(128)
rope_append_kernel(const float *src, int n_parts, size_t part_stride, float *qkv, int ld,   // src may alias qkv (n_parts == 1)
                   const float *__restrict__ cs, const float *__restrict__ sn, const int32_t *__restrict__ slot_map,
                   __half *__restrict__ pool_layer, int n_heads, int n_kv_heads, int D, int neox, unsigned int *row_bound) {
    vx_pdl_wait();
    vx_pdl_trigger();
    const int t = blockIdx.x, half = D / 2;
    if (row_bound && blockIdx.y == 0 && threadIdx.x == 0) row_bound[t] = 0u;   // the attention kernels behind this one raise it
    const int h0 = blockIdx.y * ROPE_HEADS, h1 = min(h0 + ROPE_HEADS, n_heads + 2 * n_kv_heads);
    const float *srow = src + (size_t)t * ld;
    float *drow = qkv + (size_t)t * ld;
    const float *c = cs + (size_t)t * half, *s = sn + (size_t)t * half;
    const int slot = slot_map[t];
    if (slot < 0) return;                      // the packing kernel refused the step: nothing may reach the pool
    const size_t hs = (size_t)n_kv_heads * D, part = (size_t)BS * hs;
    __half *kdst = pool_layer + (size_t)(slot / BS) * 2 * part + (size_t)(slot % BS) * hs;
    __half *vdst = kdst + part;
    const int n_pairs = (h1 - h0) * half;
    for (int idx = threadIdx.x; idx < n_pairs; idx += blockDim.x) {
        const int hd = h0 + idx / half, j = idx % half;
        if (hd < n_heads + n_kv_heads) {       // q or k head: rotate the pair (i0, i1)
            const int i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
            const size_t o0 = (size_t)hd * D + i0, o1 = (size_t)hd * D + i1;
            float a = 0.f, b = 0.f;
            for (int p = 0; p < n_parts; p++) { a += srow[p * part_stride + o0]; b += srow[p * part_stride + o1]; }
            const float r0 = __fsub_rn(__fmul_rn(a, c[j]), __fmul_rn(b, s[j]));
            const float r1 = __fadd_rn(__fmul_rn(a, s[j]), __fmul_rn(b, c[j]));
            drow[o0] = r0; drow[o1] = r1;
            if (hd >= n_heads) {
                const int kh = hd - n_heads;
                kdst[(size_t)kh * D + i0] = __float2half_rn(r0);
                kdst[(size_t)kh * D + i1] = __float2half_rn(r1);
            }
        } else {                                // v head: two consecutive elements
            const int vh = hd - n_heads - n_kv_heads;
            const size_t o = (size_t)hd * D + 2 * j;
            float a = 0.f, b = 0.f;
            for (int p = 0; p < n_parts; p++) { a += srow[p * part_stride + o]; b += srow[p * part_stride + o + 1]; }
            drow[o] = a; drow[o + 1] = b;
            vdst[(size_t)vh * D + 2 * j] = __float2half_rn(a);
            vdst[(size_t)vh * D + 2 * j + 1] = __float2half_rn(b);
        }
    }
}

// ------------------------------------------------------------------ gated activation (SwiGLU / GeGLU) + split
__device__ __forceinline__ float gate_act(float g, float u, int geglu) {
    float a;
    if (geglu) {   // backend/cpu/cpu.go:457-473
        const float s2pi = 0.7978845608f, coeff = 0.044715f;
        float x3 = __fmul_rn(__fmul_rn(g, g), g);
        float ta = __fmul_rn(s2pi, __fadd_rn(g, __fmul_rn(coeff, x3)));
        float th = (float)tanh((double)ta);
        a = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, th));
    } else {       // backend/cpu/cpu.go:390-400
        float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-g))));
        a = __fmul_rn(g, sg);
    }
    return __fmul_rn(a, u);
}
// h13 row = [gate (F) | up (F)]; act = activation(gate)*up is split for the W2 projection without touching memory in between
// One thread-block cluster per row: CL CTAs of 1024 threads share the row's columns (thread t of CTA q owns columns
// ((c * CL + q) * 1024 + t) * 4 .. +3 of chunk c) and exchange their partial maxima through distributed shared memory, so a
// thin batch spreads the float64 activation math over CL SMs instead of one.
template <int NC>
__global__ void __launch_bounds__(VX_ROW_THREADS)
act_split_kernel(const float *__restrict__ h13, int n_parts, size_t part_stride, int ffn, int geglu, VxSplit s) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = (int)cluster.num_blocks(), q = (int)cluster.block_rank();
    __shared__ float red[32];
    __shared__ float cl_amax;
    vx_pdl_wait();             // (chained launch: the kernel before this one has completed)
    vx_pdl_trigger();          // the projection that follows may become resident and fetch its first weights now
    const int r = blockIdx.x / CL;
    const float *gr = h13 + (size_t)r * 2 * ffn, *ur = gr + ffn;
    float4 v[NC];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = ((c * CL + q) * VX_ROW_THREADS + threadIdx.x) * 4;
        v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k0 < ffn) {
            float4 g = *reinterpret_cast<const float4 *>(gr + k0), u = *reinterpret_cast<const float4 *>(ur + k0);
            for (int p = 1; p < n_parts; p++) {     // split-K partials of the fused gate|up projection
                const float4 g2 = *reinterpret_cast<const float4 *>(gr + p * part_stride + k0), u2 = *reinterpret_cast<const float4 *>(ur + p * part_stride + k0);
                g.x += g2.x; g.y += g2.y; g.z += g2.z; g.w += g2.w; u.x += u2.x; u.y += u2.y; u.z += u2.z; u.w += u2.w;
            }
            v[c] = make_float4(gate_act(g.x, u.x, geglu), gate_act(g.y, u.y, geglu), gate_act(g.z, u.z, geglu), gate_act(g.w, u.w, geglu));
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[c].x), fabsf(v[c].y)), fmaxf(fabsf(v[c].z), fabsf(v[c].w))));
    }
    amax = block_max(amax, red);
    if (CL > 1) {
        if (threadIdx.x == 0) cl_amax = amax;
        cluster.sync();
        for (int o = 0; o < CL; o++) amax = fmaxf(amax, *cluster.map_shared_rank(&cl_amax, o));
        cluster.sync();                            // nobody leaves while a peer may still read its maximum
    }
    float sc, inv;
    vx_row_scale(amax, sc, inv);
    if (threadIdx.x == 0 && q == 0) s.scale[r] = sc;
    __half *hi = s.hi + (size_t)r * s.k_pad, *lo = s.lo + (size_t)r * s.k_pad;
    float *bs = s.bsum + (size_t)r * (s.k_pad / 32);
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = ((c * CL + q) * VX_ROW_THREADS + threadIdx.x) * 4;
        if (k0 < s.k_pad) {
            const float t[4] = {v[c].x * inv, v[c].y * inv, v[c].z * inv, v[c].w * inv};
            vx_split_store4(t, hi, lo, bs, k0);
        }
    }
}

__global__ void final_softcap_kernel(float *logits, long n, float cap) {   // runtime/model.go:340-349
    long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (i < n) logits[i] = (float)((double)cap * tanh((double)logits[i] * (1.0 / (double)cap)));
}

}  // namespace

// launchers living in other translation units
int vxe_argmax_rows(vx_ctx *c, const float *x, int rows, int cols, int32_t *out);
int vxs_sample_rows(vx_ctx *c, float *logits, long ld, int rows, int n, const void *d_params, float final_softcap, int32_t *d_out);
int vxe_sdpa_strided(vx_ctx *c, const float *q, int q_ld, const float *k, const float *v, float *out, int out_ld, int rows, int kv_len,
                     int causal, int hq, int hkv, int d, long pos_stride, long head_stride, float scale, float softcap);

namespace {

// ---- timing helpers
void time_begin(vx_model *m, int which) {
    if (!m->time_on[which]) return;
    if (m->ev_next + 2 > m->ev_pool.size()) {
        for (int i = 0; i < 64; i++) { cudaEvent_t e; cudaEventCreate(&e); m->ev_pool.push_back(e); }
    }
    m->ev_used.push_back({which, (int)m->ev_next});
    cudaEventRecord(m->ev_pool[m->ev_next], m->c->stream);
}
void time_end(vx_model *m, int which) {
    if (!m->time_on[which]) return;
    cudaEventRecord(m->ev_pool[m->ev_next + 1], m->c->stream);
    m->ev_next += 2;
}
void time_collect(vx_model *m) {   // call after the stream has been synchronised
    for (auto &u : m->ev_used) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, m->ev_pool[u.second], m->ev_pool[u.second + 1]) == cudaSuccess) { m->time_ms[u.first] += ms; m->time_n[u.first]++; }
    }
    m->ev_used.clear(); m->ev_next = 0;
}

static int g_dbg_skip = 0;      // timing experiments only (wrong results): 1 no projections, 2 no row kernels, 4 no attention
int gemm(vx_model *m, const VxWeight &w, const VxSplit &x, int rows, float *out, int ld_out, int *n_parts) {
    if (g_dbg_skip & 1) { *n_parts = 1; return VX_OK; }
    time_begin(m, 1);
    int rc = vxq_gemm(m->c, w, x, rows, out, ld_out, n_parts, m->parts, m->parts_cap);
    time_end(m, 1);
    return rc;
}
// projection whose consumer wants a plain [rows][n] result
int gemm_full(vx_model *m, const VxWeight &w, const VxSplit &x, int rows, float *out, int ld_out) {
    int np = 1;
    VX_TRY(gemm(m, w, x, rows, out, ld_out, &np));
    if (np > 1) VX_TRY(vxq_reduce_parts(m->c, m->parts, np, rows, w.n, out, ld_out));
    return VX_OK;
}

int add_norm_split_rows(vx_model *m, float *x, int rows, const float *parts, int n_parts, size_t part_stride, int part_ld,
                        const float *post_w, const float *w, const VxSplit &s, float *capture, const int32_t *row_idx = nullptr,
                        float *normed_out = nullptr) {
    if (g_dbg_skip & 2) return VX_OK;
    const int H = m->cfg.hidden;
    if (H > 8192) return vx_fail(m->c, VX_E_UNSUPPORTED, "hidden size %d > 8192", H);
    cudaError_t le;
    if (H > 4096) le = vx_launch_chain(add_norm_split_kernel<2>, dim3(rows), dim3(VX_ROW_THREADS), 0, m->c->stream, x, parts, n_parts, part_stride, part_ld, post_w, w, m->cfg.rms_eps, H, s, capture, row_idx, normed_out);
    else le = vx_launch_chain(add_norm_split_kernel<1>, dim3(rows), dim3(VX_ROW_THREADS), 0, m->c->stream, x, parts, n_parts, part_stride, part_ld, post_w, w, m->cfg.rms_eps, H, s, capture, row_idx, normed_out);
    if (le != cudaSuccess) return vx_cuda_fail(m->c, le, "add + norm launch");
    VX_LAUNCH_CHECK(m->c);
    return VX_OK;
}
int add_norm_split(vx_model *m, int rows, const float *parts, int n_parts, size_t part_stride, int part_ld, const float *post_w,
                   const float *w, const VxSplit &s, float *capture) {
    return add_norm_split_rows(m, m->x, rows, parts, n_parts, part_stride, part_ld, post_w, w, s, capture);
}
int act_split(vx_model *m, int rows, int n_parts) {
    if (g_dbg_skip & 2) return VX_OK;
    const int F = m->cfg.ffn;
    const size_t pstride = (size_t)rows * 2 * F;
    // cluster size: a thin batch spreads each row over up to four SMs; from ~a third of the SMs in rows on, one CTA per row
    // is faster (measured at 64 rows: 9 us alone against 12 us in clusters of four)
    int cl = 1;
    while (cl < 4 && rows * cl * 2 <= m->c->sm_count / 2 && m->sp_f.k_pad > cl * VX_ROW_THREADS * 4) cl *= 2;
    int nc = ceil_div(m->sp_f.k_pad, cl * VX_ROW_THREADS * 4);
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(rows * cl); lc.blockDim = dim3(VX_ROW_THREADS); lc.dynamicSmemBytes = 0; lc.stream = m->c->stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = cl; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = g_vx_pdl >= 2 ? 2 : 1;
    const float *parts_c = m->parts;
    switch (nc) {
#define VX_ACT_CASE(N) case N: VX_CUDA(m->c, cudaLaunchKernelEx(&lc, act_split_kernel<N>, parts_c, n_parts, pstride, F, m->cfg.geglu, m->sp_f)); break;
        VX_ACT_CASE(1) VX_ACT_CASE(2) VX_ACT_CASE(3) VX_ACT_CASE(4) VX_ACT_CASE(5) VX_ACT_CASE(6) VX_ACT_CASE(7) VX_ACT_CASE(8)
#undef VX_ACT_CASE
    default: return vx_fail(m->c, VX_E_UNSUPPORTED, "ffn size %d is not supported (max 32768)", F);
    }
    VX_LAUNCH_CHECK(m->c);
    return VX_OK;
}

bool layer_slides(const vx_model_config &c, int layer) {   // runtime/block.go:464-476
    if (c.sliding_window <= 0) return false;
    return c.window_alternating ? (layer % 2 == 1) : true;
}

// Rows of one batch entry that do not go through the split-K work lists.
//   route 1: causal attention over the fresh float32 K/V of this call (a prompt that starts at position 0, block.go:891-895)
//   route 2: the multi-row tensor-core kernel over the pages (a long chunk of one sequence, decode.go:1033-1060)
struct RowRange { int row0, n, route; };
enum { OUT_LAST_ROWS = 1, OUT_HIDDEN = 2 };     // output flags of a step (also part of the graph key)

// The transformer stack over `rows` packed query rows whose packing arrays are already on the device.
// special: the row ranges served by the prefill kernels; every other row (plain_rows of them) takes paged decode attention.
// Outputs (logits, tokens, optionally post-norm hidden states) are produced for logit_rows rows: the trailing rows, or with
// OUT_LAST_ROWS the last row of each of the logit_rows (= n_seqs) batch entries.
int forward(vx_model *m, int rows, const std::vector<RowRange> &special, int plain_rows, int n_work_host[2], const int chunk_pages[2],
            int logit_rows, int out_flags) {
    vx_ctx *c = m->c; const vx_model_config &cf = m->cfg;
    const int H = cf.hidden, Hq = cf.n_heads, Hkv = cf.n_kv_heads, D = cf.head_dim, F = cf.ffn;
    const int qd = Hq * D, kvd = Hkv * D, nqkv = qd + 2 * kvd;
    const float scale = (float)(1.0 / sqrt((double)D));   // block.go:862
    const int32_t *tokens = m->d_step_in + 4 * m->last_seqs;
    embed_kernel<<<rows, 256, 0, c->stream>>>(tokens, m->embed.dev, m->embed.type, m->x, H, m->tp ? m->vocab_full : cf.vocab, cf.embed_scale);
    VX_LAUNCH_CHECK(c);
    {
        int n = rows * (D / 2);
        rope_table_kernel<<<ceil_div(n, 256), 256, 0, c->stream>>>(m->d_row_pos, m->d_freq, m->d_cos, m->d_sin, rows, D / 2);
        VX_LAUNCH_CHECK(c);
    }
    const size_t cap_stride = (size_t)rows * H;
    int np_prev = 0;                 // partial count of the previous W2 projection, consumed by the next add
    const float *post_prev = nullptr, *prev_out = m->parts;
    for (int l = 0; l < cf.n_layers; l++) {
        const LayerW &L = m->layers[l];
        // x += W2 output of the previous layer; normOut = RMSNorm(x) (block.go:836)
        VX_TRY(add_norm_split(m, rows, prev_out, np_prev, (size_t)rows * H, H, post_prev, L.attn_norm, m->sp_h,
                              m->capture_on ? m->capture + (size_t)l * cap_stride : nullptr));
        int np_qkv = 1;
        const float *qkv_src = m->parts;
        if (L.wqkv.size() == 1) {
            VX_TRY(gemm(m, L.wqkv[0].w, m->sp_h, rows, m->parts, nqkv, &np_qkv));      // block.go:841-854
        } else {   // mixed block formats: one projection per format run, written side by side; RoPE then runs in place
            for (const ColW &cw : L.wqkv) VX_TRY(gemm_full(m, cw.w, m->sp_h, rows, m->qkv + cw.col, nqkv));
            qkv_src = m->qkv;
        }
        if (!(g_dbg_skip & 2)) {
            dim3 rg(rows, ceil_div(Hq + 2 * Hkv, ROPE_HEADS));
            cudaError_t le = vx_launch_chain(rope_append_kernel, rg, dim3(128), 0, c->stream, qkv_src, np_qkv, (size_t)rows * nqkv, m->qkv, nqkv,
                                             (const float *)m->d_cos, (const float *)m->d_sin, (const int32_t *)m->d_slot_map,
                                             m->pool + (size_t)l * m->layer_stride, Hq, Hkv, D, (int)cf.rope_neox,
                                             (special.empty() && !(g_dbg_skip & 8)) ? m->d_row_bound : nullptr);   // block.go:858-868
            if (le != cudaSuccess) return vx_cuda_fail(c, le, "RoPE + append launch");
            VX_LAUNCH_CHECK(c);
        }
        time_begin(m, 0);
        bool split_done = false;
        {
            const int wl = layer_slides(cf, l) ? 1 : 0;
            VxAttnArgs a{};
            a.q = m->qkv; a.q_row_stride = nqkv; a.pool = m->pool + (size_t)l * m->layer_stride; a.pool_is_f16 = 1;
            a.tables = m->d_table_ptrs; a.row_slot = m->d_row_slot;
            a.row_kv_start = wl ? m->d_row_kv_start : nullptr; a.row_kv_len = m->d_row_kv_len;
            a.work = m->d_work[wl]; a.n_work_dev = m->d_n_work[wl]; a.n_work = n_work_host[wl]; a.row_work_start = m->d_rws[wl];
            a.partials = m->d_partials; a.out = m->attn; a.out_row_stride = qd;
            a.rows = rows; a.n_q_heads = Hq; a.n_kv_heads = Hkv; a.head_dim = D; a.block_size = BS;
            a.scale = scale; a.softcap = cf.attn_softcap;
            // every row walks the work list: the kernels report a bound of each row's output and the merge spreads a row over
            // several CTAs (rows served by the prompt kernels below have no such bound)
            a.row_bound = (special.empty() && !(g_dbg_skip & (2 | 8))) ? m->d_row_bound : nullptr;
            for (const RowRange &r : special) {
                if (r.route == 1) {
                    const float *q = m->qkv + (size_t)r.row0 * nqkv;
                    float *o = m->attn + (size_t)r.row0 * qd;
                    int rc = vxp_prefill_f32(c, q, nqkv, q + qd, q + qd + kvd, nqkv, o, qd, r.n, Hq, Hkv, D, scale, cf.attn_softcap);
                    if (rc == VX_E_UNSUPPORTED)
                        rc = vxe_sdpa_strided(c, q, nqkv, q + qd, q + qd + kvd, o, qd, r.n, 0, 1, Hq, Hkv, D, nqkv, D, scale, cf.attn_softcap);
                    VX_TRY(rc);
                } else {
                    // a long chunk of one sequence walks the cache once per 64 rows instead of once per row
                    VX_TRY(vxp_prefill_rows(c, a, r.row0, r.n));
                }
            }
            // at most this many split-K chunks per row: the table width bounds a row's pages
            const int n_max = ceil_div(cf.max_blocks_per_seq, max(chunk_pages[wl], 1)) + 1;
            // rows served above have no work items; the merge reads their finished output rows back
            if (plain_rows > 0 && !(g_dbg_skip & 4)) VX_TRY(vxp_attention_split(c, a, &m->sp_q, n_max, &split_done));  // block.go:872 / 881-890
            if (g_dbg_skip & 4) split_done = true;
        }
        time_end(m, 0);
        if (!split_done) VX_TRY(vxq_split_rows(c, m->attn, rows, qd, qd, m->sp_q));
        int np_o = 1;
        VX_TRY(gemm(m, L.wo, m->sp_q, rows, m->parts, H, &np_o));                       // block.go:983
        const float *wo_out = m->parts;
        if (m->tp) {   // this rank holds a column slice of Wo: its output is a partial sum over the ranks
            VX_TRY(vxq_reduce_parts(c, m->parts, np_o, rows, H, m->ar_buf, H));
            VX_TRY(vxtp_allreduce_sum(c, m->ar_buf, (size_t)rows * H));
            wo_out = m->ar_buf; np_o = 1;
        }
        // x += Wo output (post-attn norm first for Gemma 2); normOut = RMSNorm(x, ffn_norm) (block.go:985-997)
        VX_TRY(add_norm_split(m, rows, wo_out, np_o, (size_t)rows * H, H, cf.post_norms ? L.post_attn_norm : nullptr, L.ffn_norm,
                              m->sp_h, nullptr));
        int np_13 = 1;
        VX_TRY(gemm(m, L.w13, m->sp_h, rows, m->parts, 2 * F, &np_13));                 // block.go:1045-1049
        VX_TRY(act_split(m, rows, np_13));                                              // block.go:1051-1057
        VX_TRY(gemm(m, L.w2, m->sp_f, rows, m->parts, H, &np_prev));                    // block.go:1060
        if (m->tp) {   // W2 is split along its input columns as well
            VX_TRY(vxq_reduce_parts(c, m->parts, np_prev, rows, H, m->ar_buf, H));
            VX_TRY(vxtp_allreduce_sum(c, m->ar_buf, (size_t)rows * H));
            prev_out = m->ar_buf; np_prev = 1;
        } else prev_out = m->parts;
        post_prev = cf.post_norms ? L.post_ffn_norm : nullptr;
    }
    // last residual add, then the final norm on the rows that need logits (decode.go:442, 1057-1086)
    const bool last_rows = (out_flags & OUT_LAST_ROWS) != 0;
    const int r0 = last_rows ? 0 : rows - logit_rows;
    VX_TRY(add_norm_split(m, rows, prev_out, np_prev, (size_t)rows * H, H, post_prev, nullptr, m->sp_h,
                          m->capture_on ? m->capture + (size_t)cf.n_layers * cap_stride : nullptr));
    // norm + split only the logit rows (the trailing ones, or the last row of every entry), written to split rows [0, logit_rows)
    VX_TRY(add_norm_split_rows(m, m->x + (size_t)r0 * H, logit_rows, nullptr, 0, 0, 0, nullptr, m->final_norm, m->sp_h, nullptr,
                               last_rows ? m->d_last_row : nullptr, (out_flags & OUT_HIDDEN) ? m->d_hidden : nullptr));
    VX_TRY(gemm_full(m, m->w_out, m->sp_h, logit_rows, m->logits, cf.vocab));           // model.go:352-422
    VX_TRY(vxe_argmax_rows(c, m->logits, logit_rows, cf.vocab, m->d_out_tok));          // sampler.go:79-90
    if (m->tp)     // the head is split by vocabulary rows: the local maxima meet in one small all-gather
        VX_TRY(vxtp_global_argmax(c, m->logits, cf.vocab, m->d_out_tok, logit_rows, cf.vocab, m->tp_scratch, m->d_out_tok));
    return VX_OK;
}

int check_status(vx_model *m) {
    int32_t st = 0;
    VX_CUDA(m->c, cudaMemcpyAsync(m->h_out_tok + m->cfg.max_batch_tokens, m->d_status, 4, cudaMemcpyDeviceToHost, m->c->stream));
    VX_CUDA(m->c, cudaStreamSynchronize(m->c->stream));
    st = m->h_out_tok[m->cfg.max_batch_tokens];
    VX_TRY(vx_check_device_error(m->c));
    if (st != 0) {
        cudaMemsetAsync(m->d_status, 0, 4, m->c->stream);
        return vx_fail(m->c, st, "device bookkeeping reported status %d (%s)", st,
                       st == VX_E_OOM_BLOCKS ? "block pool exhausted" : "inconsistent step arguments");
    }
    return VX_OK;
}

int refresh_free(vx_model *m) {
    VX_CUDA(m->c, cudaMemcpyAsync(m->h_out_tok + m->cfg.max_batch_tokens + 1, m->d_free_top, 4, cudaMemcpyDeviceToHost, m->c->stream));
    VX_CUDA(m->c, cudaStreamSynchronize(m->c->stream));
    m->h_free = m->h_out_tok[m->cfg.max_batch_tokens + 1];
    return VX_OK;
}

// chooses the split-K chunk (in pages) for a step and returns the exact work-item count
int plan_chunks(vx_model *m, const std::vector<int> &kv_start, const std::vector<int> &kv_len, int *chunk_out) {
    long pages = 0;
    for (size_t i = 0; i < kv_len.size(); i++) pages += (kv_len[i] - 1) / BS - kv_start[i] / BS + 1;
    long target = 6L * m->c->sm_count;
    // grouped-query shapes have few KV heads, hence few CTAs per chunk: longer chunks amortise a CTA's start-up
    // (block-table and query loads) and merge over more pages.  Multi-head shapes: 32 pages measured best at 64 sequences
    // (step 9.87 ms against 9.98 at 16 and at 48, 9.99 at 64, 10.30 at 8: fewer partial sums to write and merge against a
    // longer tail of the last wave)
    long max_chunk = m->cfg.n_heads > m->cfg.n_kv_heads ? 64 : 32;
    if (g_dbg_skip >> 8) max_chunk = g_dbg_skip >> 8;       // timing experiments: another cap
    int chunk = (int)std::min<long>(max_chunk, std::max<long>(4, (pages * m->cfg.n_kv_heads + target - 1) / target));
    for (;;) {
        long n = 0;
        for (size_t i = 0; i < kv_len.size(); i++) { int np = (kv_len[i] - 1) / BS - kv_start[i] / BS + 1; n += (np + chunk - 1) / chunk; }
        if (n <= MAX_WORK) { *chunk_out = chunk; return (int)n; }
        chunk *= 2;
    }
}

// advances a resident batch by one position: every sequence is fed the token the previous step produced
__global__ void advance_step_kernel(int32_t *step_in, int n_seqs, const int32_t *prev_tokens) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_seqs) return;
    step_in[2 * n_seqs + i] += 1;
    step_in[4 * n_seqs + i] = prev_tokens[i];
}

// Host half of a step: validation and admission control against the host mirror, attention routes, split-K planning, then
// the mirror update.  No device state is touched; on failure nothing has changed.
struct StepPlan { int n_seqs = 0, rows = 0, chunk[2] = {4, 4}, n_work[2] = {0, 0}, plain_rows = 0; std::vector<RowRange> special; std::vector<int> routes; };
constexpr int PF_MIN_ROWS = 32;      // from this many rows of one sequence on, the multi-row kernel beats per-row decode attention
int plan_step(vx_model *m, int n_seqs, const int *slots, const int32_t *positions, const int32_t *q_lens, bool prompt_rows, StepPlan *p) {
    vx_ctx *c = m->c; const vx_model_config &cf = m->cfg;
    int rows = 0;
    for (int i = 0; i < n_seqs; i++) rows += q_lens ? q_lens[i] : 1;
    if (rows <= 0 || rows > cf.max_batch_tokens) return vx_fail(c, VX_E_BAD_ARG, "step has %d rows (limit %d)", rows, cf.max_batch_tokens);
    long need = 0;
    std::vector<int> kv_len, kv_start0, kv_start1;
    std::vector<char> seen(cf.max_seqs, 0);
    kv_len.reserve(rows);
    p->special.clear(); p->routes.assign(n_seqs, 0);
    const bool pf_rows_ok = cf.head_dim == 64 || cf.head_dim == 128;
    int row0 = 0, n_special_rows = 0;
    for (int i = 0; i < n_seqs; i++) {
        int s = slots[i], ql = q_lens ? q_lens[i] : 1;
        if (ql <= 0) return vx_fail(c, VX_E_BAD_ARG, "q_len[%d] = %d", i, ql);
        if (seen[s]) return vx_fail(c, VX_E_BAD_ARG, "sequence appears twice in one step");
        seen[s] = 1;
        if (positions[i] != m->h_seq_len[s])
            return vx_fail(c, VX_E_BAD_ARG, "position %d of batch entry %d != sequence length %d", positions[i], i, m->h_seq_len[s]);
        int nb_new = (positions[i] + ql + BS - 1) / BS;
        if (nb_new > cf.max_blocks_per_seq) return vx_fail(c, VX_E_OOM_BLOCKS, "sequence would need %d blocks (table width %d)", nb_new, cf.max_blocks_per_seq);
        need += std::max(0, nb_new - m->h_n_blocks[s]);
        if (prompt_rows && positions[i] == 0) p->routes[i] = 1;
        else if (ql >= PF_MIN_ROWS && pf_rows_ok) p->routes[i] = 2;
        if (p->routes[i]) n_special_rows += ql;
        row0 += ql;
    }
    if (need > m->h_free) return vx_fail(c, VX_E_OOM_BLOCKS, "no free blocks: need %ld, have %d (max=%d)", need, m->h_free, cf.max_blocks);
    // a head shape outside the work-list kernels falls back to a kernel that serves every row: no mixing with the prefill routes
    if (!m->fast_attn_shape && n_special_rows != rows) { p->routes.assign(n_seqs, 0); n_special_rows = 0; }
    row0 = 0;
    for (int i = 0; i < n_seqs; i++) {
        int ql = q_lens ? q_lens[i] : 1;
        if (p->routes[i]) p->special.push_back(RowRange{row0, ql, p->routes[i]});
        else for (int j = 0; j < ql; j++) kv_len.push_back(positions[i] + j + 1);
        row0 += ql;
    }
    p->plain_rows = rows - n_special_rows;
    kv_start0.assign(kv_len.size(), 0); kv_start1.assign(kv_len.size(), 0);
    if (cf.sliding_window > 0) for (size_t t = 0; t < kv_len.size(); t++) kv_start1[t] = std::max(0, kv_len[t] - cf.sliding_window);
    p->n_seqs = n_seqs; p->rows = rows; p->chunk[0] = p->chunk[1] = 4; p->n_work[0] = p->n_work[1] = 0;
    if (p->plain_rows > 0) {
        p->n_work[0] = plan_chunks(m, kv_start0, kv_len, &p->chunk[0]);
        if (cf.sliding_window > 0) p->n_work[1] = plan_chunks(m, kv_start1, kv_len, &p->chunk[1]);
    }
    for (int i = 0; i < n_seqs; i++) {
        int s = slots[i], ql = q_lens ? q_lens[i] : 1;
        int nb_new = (positions[i] + ql + BS - 1) / BS;
        if (nb_new > m->h_n_blocks[s]) { m->h_free -= nb_new - m->h_n_blocks[s]; m->h_n_blocks[s] = nb_new; }
        m->h_seq_len[s] = positions[i] + ql;
    }
    return VX_OK;
}

// After a step failed between the planning and its synchronisation the host mirror may be ahead of or behind the device
// (the packing kernel refuses a step as a whole, a launch error can strike after it ran): read the device state back.
void resync_mirror(vx_model *m) {
    vx_ctx *c = m->c;
    cudaStreamSynchronize(c->stream);
    std::vector<int32_t> len(m->cfg.max_seqs), nb(m->cfg.max_seqs);
    int32_t top = m->h_free;
    bool ok = cudaMemcpy(len.data(), m->d_seq_len, 4 * len.size(), cudaMemcpyDeviceToHost) == cudaSuccess &&
              cudaMemcpy(nb.data(), m->d_n_blocks, 4 * nb.size(), cudaMemcpyDeviceToHost) == cudaSuccess &&
              cudaMemcpy(&top, m->d_free_top, 4, cudaMemcpyDeviceToHost) == cudaSuccess;
    if (!ok) { cudaGetLastError(); return; }
    for (int s = 0; s < m->cfg.max_seqs; s++) { m->h_seq_len[s] = len[s]; m->h_n_blocks[s] = nb[s]; }
    m->h_free = top;
}

// Device half: packing kernel + the transformer stack, reading the step description already in d_step_in.
static int g_graphs = 1;

// pack kernel + the transformer stack for one planned step; n_work = grid sizes of the attention kernels
int enqueue_kernels(vx_model *m, const StepPlan &p, int out_flags, int logit_rows, int n_work[2]) {
    vx_ctx *c = m->c; const vx_model_config &cf = m->cfg;
    PackArgs pa{};
    pa.step_in = m->d_step_in; pa.n_seqs = p.n_seqs; pa.n_rows = p.rows;
    pa.tables = m->d_tables; pa.width = cf.max_blocks_per_seq; pa.seq_len = m->d_seq_len; pa.n_blocks = m->d_n_blocks;
    pa.free_list = m->d_free_list; pa.free_top = m->d_free_top; pa.refcnt = m->d_refcnt; pa.status = m->d_status;
    pa.cu = m->d_cu; pa.row_slot = m->d_row_slot; pa.row_pos = m->d_row_pos; pa.slot_map = m->d_slot_map;
    pa.row_kv_len = m->d_row_kv_len; pa.row_kv_start = m->d_row_kv_start; pa.window = cf.sliding_window;
    pa.row_route = m->d_row_route; pa.last_row = m->d_last_row;
    pa.work0 = m->d_work[0]; pa.work1 = m->d_work[1]; pa.rws0 = m->d_rws[0]; pa.rws1 = m->d_rws[1];
    pa.n_work0 = m->d_n_work[0]; pa.n_work1 = m->d_n_work[1]; pa.chunk0 = p.chunk[0]; pa.chunk1 = p.chunk[1]; pa.max_work = MAX_WORK;
    pack_kernel<<<1, 1024, 0, c->stream>>>(pa);
    VX_LAUNCH_CHECK(c);
    return forward(m, p.rows, p.special, p.plain_rows, n_work, p.chunk, logit_rows, out_flags);
}

// A decode step is ~250-330 small launches, and a thin batch is bound by the host's launch rate rather than by the GPU.
// Steps of the same shape are therefore replayed from a CUDA graph.  The key holds everything that shapes the launches:
// sequence and row counts, the split-K chunk sizes, and the attention grids rounded up to a multiple of 32 work items
// (CTAs beyond the device-side count return at once), so that a key survives many steps while the contexts grow.
// The first step of a key runs eagerly (it also makes every lazy allocation and attribute call), the second is captured.
int enqueue_step(vx_model *m, const StepPlan &p, int out_flags, int logit_rows) {
    vx_ctx *c = m->c;
    m->last_rows = p.rows; m->last_seqs = p.n_seqs;
    if (m->capture_on) m->capture_rows = p.rows;
    int n_work[2] = {p.n_work[0], p.n_work[1]};
    // steps with prefill routes launch one kernel per routed entry, so their launch sequence is not a function of the key
    // (a tensor-parallel step captures its NCCL collectives with the rest: every rank runs the same shapes in the same order,
    // so all of them capture, and later replay, the same step)
    const bool can_graph = g_graphs && p.special.empty() && !m->capture_on && !m->time_on[0] && !m->time_on[1];
    if (can_graph) {
        for (int i = 0; i < 2; i++) if (n_work[i] > 0) n_work[i] = std::min(MAX_WORK, (n_work[i] + 31) / 32 * 32);
        const vx_model::GraphKey key{p.n_seqs, p.rows, logit_rows, p.chunk[0], p.chunk[1], n_work[0], n_work[1], out_flags};
        if (m->graphs.size() > 256) {                    // shapes no longer in use: start over rather than grow without bound
            for (auto &kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
            m->graphs.clear();
        }
        vx_model::GraphEntry &e = m->graphs[key];
        // A key that differs from an instantiated one only in the attention grids (the contexts grew past a chunk boundary)
        // takes that graph over: the step is captured again and the executable graph is updated in place, which costs a
        // fraction of an eager step plus an instantiation.
        vx_model::GraphEntry *sib = nullptr;
        if (!e.exec && e.seen < 1000000)
            for (auto &kv : m->graphs) {
                const vx_model::GraphKey &k = kv.first;
                if (kv.second.exec && k.n_seqs == key.n_seqs && k.rows == key.rows && k.logit_rows == key.logit_rows && k.chunk0 == key.chunk0 &&
                    k.chunk1 == key.chunk1 && k.out_flags == key.out_flags) { sib = &kv.second; break; }
            }
        if (!e.exec && (e.seen >= 1 || sib) && e.seen < 1000000) {
            const uint64_t l0 = c->launches;
            cudaGraph_t g = nullptr;
            bool ok = cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
            int rc = ok ? enqueue_kernels(m, p, out_flags, logit_rows, n_work) : VX_OK;
            if (ok) ok = cudaStreamEndCapture(c->stream, &g) == cudaSuccess && g != nullptr && rc == VX_OK;
            if (ok && sib) {
                cudaGraphExecUpdateResultInfo info;
                if (cudaGraphExecUpdate(sib->exec, g, &info) == cudaSuccess) { e.exec = sib->exec; sib->exec = nullptr; sib->seen = 1; m->graph_updates++; }
                else { cudaGetLastError(); cudaGraphExecDestroy(sib->exec); sib->exec = nullptr; sib->seen = 1; }   // not updatable (a kernel changed): instantiate below
            }
            if (ok && !e.exec) ok = cudaGraphInstantiate(&e.exec, g, 0) == cudaSuccess;
            if (g) cudaGraphDestroy(g);
            e.launches = c->launches - l0;
            c->launches = l0;                            // nothing ran while capturing
            if (!ok) { cudaGetLastError(); e.exec = nullptr; e.seen = 1000000; }     // this shape stays eager
        }
        if (e.exec) {
            VX_CUDA(c, cudaGraphLaunch(e.exec, c->stream));
            c->launches += e.launches;
            m->graph_replays++;
            m->steps++;
            return VX_OK;
        }
        if (e.seen < 1000000) e.seen++;
    }
    VX_TRY(enqueue_kernels(m, p, out_flags, logit_rows, n_work));
    m->steps++;
    return VX_OK;
}

// step flags of the C ABI (vexel_cuda.h) -> what the stack has to produce
int run_step_planned(vx_model *m, const StepPlan &p, int n_seqs, const int *slots, const int32_t *tokens, const int32_t *positions,
                     const int32_t *q_lens, int out_flags, int logit_rows, int32_t *out_tokens, float *logits, const vx_sample_params *sample,
                     float *hidden) {
    vx_ctx *c = m->c; const vx_model_config &cf = m->cfg;
    int32_t *h = m->h_step_in;
    for (int i = 0; i < n_seqs; i++) {
        h[i] = slots[i]; h[n_seqs + i] = q_lens ? q_lens[i] : 1; h[2 * n_seqs + i] = positions[i]; h[3 * n_seqs + i] = p.routes[i];
    }
    memcpy(h + 4 * n_seqs, tokens, sizeof(int32_t) * p.rows);
    VX_CUDA(c, cudaMemcpyAsync(m->d_step_in, h, sizeof(int32_t) * (4 * n_seqs + p.rows), cudaMemcpyHostToDevice, c->stream));
    VX_TRY(enqueue_step(m, p, out_flags, logit_rows));
    if (logits && cf.final_softcap > 0.f) {
        long n = (long)logit_rows * cf.vocab;
        final_softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, c->stream>>>(m->logits, n, cf.final_softcap);
        VX_LAUNCH_CHECK(c);
    }
    if (logits) VX_CUDA(c, cudaMemcpyAsync(logits, m->logits, sizeof(float) * (size_t)logit_rows * cf.vocab, cudaMemcpyDeviceToHost, c->stream));
    if (hidden) VX_CUDA(c, cudaMemcpyAsync(hidden, m->d_hidden, sizeof(float) * (size_t)logit_rows * cf.hidden, cudaMemcpyDeviceToHost, c->stream));
    if (sample) {
        // rows with temperature 0 keep the argmax; the others are drawn on the device from the logits in place
        // (scheduler.go:783-820 copies the logits to the host and samples there)
        VX_CUDA(c, cudaMemcpyAsync(m->d_sample, sample, sizeof(vx_sample_params) * (size_t)logit_rows, cudaMemcpyHostToDevice, c->stream));
        VX_TRY(vxs_sample_rows(c, m->logits, cf.vocab, logit_rows, cf.vocab, m->d_sample, logits ? 0.f : cf.final_softcap, m->d_out_tok));
    }
    VX_CUDA(c, cudaMemcpyAsync(m->h_out_tok, m->d_out_tok, sizeof(int32_t) * logit_rows, cudaMemcpyDeviceToHost, c->stream));
    VX_TRY(check_status(m));   // synchronises the stream
    time_collect(m);
    if (out_tokens) memcpy(out_tokens, m->h_out_tok, sizeof(int32_t) * logit_rows);
    return VX_OK;
}

// flags: VX_STEP_* of the C ABI.  logit_rows_req > 0: outputs for that many trailing rows only (prefill: 1).
int run_step(vx_model *m, int n_seqs, const int *slots, const int32_t *tokens, const int32_t *positions, const int32_t *q_lens,
             int flags, int logit_rows_req, int32_t *out_tokens, float *logits, const vx_sample_params *sample = nullptr,
             float *hidden = nullptr) {
    if (m->tp && sample) return vx_fail(m->c, VX_E_UNSUPPORTED, "sampling from a vocabulary-split output head is not implemented: tensor-parallel steps are greedy");
    StepPlan p;
    VX_TRY(plan_step(m, n_seqs, slots, positions, q_lens, (flags & VX_STEP_PROMPT_ROWS) != 0, &p));
    int out_flags = hidden ? OUT_HIDDEN : 0;
    int logit_rows = p.rows;
    if (logit_rows_req > 0) logit_rows = logit_rows_req;
    else if (flags & VX_STEP_LAST_ROWS) { logit_rows = n_seqs; if (n_seqs != p.rows) out_flags |= OUT_LAST_ROWS; }   // no gather when every entry has one row
    int rc = run_step_planned(m, p, n_seqs, slots, tokens, positions, q_lens, out_flags, logit_rows, out_tokens, logits, sample, hidden);
    if (rc != VX_OK) resync_mirror(m);
    return rc;
}

int get_slot(vx_model *m, int64_t id, bool create, int *slot) {
    auto it = m->seq_slot.find(id);
    if (it != m->seq_slot.end()) { *slot = it->second; return VX_OK; }
    if (!create) return vx_fail(m->c, VX_E_NO_SEQ, "sequence %lld not found", (long long)id);
    if (m->free_slots.empty()) return vx_fail(m->c, VX_E_OOM, "all %d sequence slots are in use", m->cfg.max_seqs);
    int s = m->free_slots.back(); m->free_slots.pop_back();
    m->seq_slot[id] = s; m->h_seq_len[s] = 0; m->h_n_blocks[s] = 0;
    // device state of a free slot is already zero (reset by delete / creation)
    *slot = s;
    return VX_OK;
}

}  // namespace

extern "C" {

int vx_model_create(vx_ctx *c, const vx_model_config *cfg, vx_model **out) {
    if (!c || !cfg || !out) return VX_E_BAD_ARG;
    VxGuard g(c);
    *out = nullptr;
    VX_REQUIRE(c, cfg->n_layers > 0 && cfg->hidden > 0 && cfg->n_heads > 0 && cfg->n_kv_heads > 0 && cfg->head_dim > 0 && cfg->ffn > 0 && cfg->vocab > 0, "non-positive dimension");
    VX_REQUIRE(c, cfg->n_heads % cfg->n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads");
    VX_REQUIRE(c, cfg->head_dim % 8 == 0 && cfg->head_dim <= 256, "head_dim must be a multiple of 8, at most 256");
    VX_REQUIRE(c, cfg->hidden % 32 == 0 && cfg->ffn % 32 == 0, "hidden and ffn must be multiples of 32");
    VX_REQUIRE(c, cfg->hidden <= 8192 && cfg->ffn <= 32768, "hidden <= 8192 and ffn <= 32768");
    VX_REQUIRE(c, cfg->max_blocks > 0 && cfg->max_seqs > 0 && cfg->max_batch_tokens > 0 && cfg->max_blocks_per_seq > 0, "non-positive pool limits");
    vx_model *m = new vx_model();
    m->c = c; m->cfg = *cfg;
    m->raw.resize((size_t)cfg->n_layers * VX_W_PER_LAYER + 3);
    m->layers.resize(cfg->n_layers);
    auto fail = [&](int rc) { vx_model_destroy(m); return rc; };
    const int T = cfg->max_batch_tokens, H = cfg->hidden, D = cfg->head_dim, F = cfg->ffn;
    const int qd = cfg->n_heads * D, kvd = cfg->n_kv_heads * D, nqkv = qd + 2 * kvd;
    int rc;
#define MA(expr) if ((rc = (expr)) != VX_OK) return fail(rc)
    // ---- pool: [layer][block][K|V][16][Hkv][D] fp16, zero-filled so every byte is a finite fp16
    m->layer_stride = (size_t)cfg->max_blocks * 2 * BS * kvd;
    MA(model_alloc_t(m, m->layer_stride * cfg->n_layers, &m->pool));
    if (cudaMemsetAsync(m->pool, 0, m->layer_stride * cfg->n_layers * sizeof(__half), c->stream) != cudaSuccess) return fail(VX_E_CUDA);
    MA(model_alloc_t(m, (size_t)cfg->max_seqs * cfg->max_blocks_per_seq, &m->d_tables));
    MA(model_alloc_t(m, (size_t)cfg->max_seqs, &m->d_table_ptrs));
    MA(model_alloc_t(m, (size_t)cfg->max_seqs, &m->d_seq_len));
    MA(model_alloc_t(m, (size_t)cfg->max_seqs, &m->d_n_blocks));
    MA(model_alloc_t(m, (size_t)cfg->max_blocks, &m->d_free_list));
    MA(model_alloc_t(m, (size_t)cfg->max_blocks, &m->d_refcnt));
    MA(model_alloc_t(m, 4, &m->d_free_top));
    MA(model_alloc_t(m, 4, &m->d_status));
    cudaMemsetAsync(m->d_tables, 0, sizeof(int32_t) * (size_t)cfg->max_seqs * cfg->max_blocks_per_seq, c->stream);
    cudaMemsetAsync(m->d_seq_len, 0, sizeof(int32_t) * cfg->max_seqs, c->stream);
    cudaMemsetAsync(m->d_n_blocks, 0, sizeof(int32_t) * cfg->max_seqs, c->stream);
    cudaMemsetAsync(m->d_refcnt, 0, sizeof(int32_t) * cfg->max_blocks, c->stream);
    cudaMemsetAsync(m->d_status, 0, 16, c->stream);
    init_free_list_kernel<<<ceil_div(cfg->max_blocks, 256), 256, 0, c->stream>>>(m->d_free_list, cfg->max_blocks);
    init_table_ptrs_kernel<<<ceil_div(cfg->max_seqs, 256), 256, 0, c->stream>>>(m->d_table_ptrs, m->d_tables, cfg->max_blocks_per_seq, cfg->max_seqs);
    cudaMemcpyAsync(m->d_free_top, &cfg->max_blocks, 4, cudaMemcpyHostToDevice, c->stream);
    m->h_free = cfg->max_blocks;
    m->h_seq_len.assign(cfg->max_seqs, 0); m->h_n_blocks.assign(cfg->max_seqs, 0);
    for (int s = cfg->max_seqs - 1; s >= 0; s--) m->free_slots.push_back(s);
    // ---- step buffers
    const size_t step_ints = (size_t)4 * cfg->max_seqs + T;
    MA(model_alloc_t(m, step_ints, &m->d_step_in));
    if (cudaMallocHost(&m->h_step_in, step_ints * 4) != cudaSuccess || cudaMallocHost(&m->h_out_tok, (size_t)(T + 8) * 4) != cudaSuccess) return fail(VX_E_OOM);
    MA(model_alloc_t(m, (size_t)cfg->max_seqs + 1, &m->d_cu));
    MA(model_alloc_t(m, (size_t)T, &m->d_row_slot)); MA(model_alloc_t(m, (size_t)T, &m->d_row_pos));
    MA(model_alloc_t(m, (size_t)T, &m->d_slot_map)); MA(model_alloc_t(m, (size_t)T, &m->d_row_kv_len));
    MA(model_alloc_t(m, (size_t)std::max(T, cfg->max_seqs) + 1, &m->d_row_kv_start));
    MA(model_alloc_t(m, (size_t)T, &m->d_row_route)); MA(model_alloc_t(m, (size_t)T, &m->d_row_bound)); MA(model_alloc_t(m, (size_t)cfg->max_seqs, &m->d_last_row));
    MA(model_alloc_t(m, (size_t)T * H, &m->d_hidden));
    {
        const int G = cfg->n_heads / cfg->n_kv_heads;
        m->fast_attn_shape = (D == 64 || D == 128 || D == 256) && (G == 1 || G == 2 || G == 4 || G == 8) && (nqkv % 4 == 0);
    }
    for (int i = 0; i < 2; i++) {
        MA(model_alloc_t(m, (size_t)MAX_WORK, &m->d_work[i]));
        MA(model_alloc_t(m, (size_t)T + 1, &m->d_rws[i]));
        MA(model_alloc_t(m, 4, &m->d_n_work[i]));
    }
    // partials: rows cut into >1 chunk only exist when contexts are long; size for the planner's worst case
    {
        size_t max_items = std::min<size_t>(MAX_WORK, (size_t)T * ((size_t)ceil_div(cfg->max_blocks_per_seq, 4) + 1));
        MA(model_alloc_t(m, max_items * cfg->n_heads * (D + 2), &m->d_partials));
    }
    MA(model_alloc_t(m, (size_t)T * (D / 2), &m->d_cos)); MA(model_alloc_t(m, (size_t)T * (D / 2), &m->d_sin));
    MA(model_alloc_t(m, (size_t)(D / 2), &m->d_freq));
    {
        std::vector<float> fr(D / 2);   // backend/cpu/cpu.go:253-254
        for (int j = 0; j < D / 2; j++) fr[j] = (float)(1.0 / pow((double)cfg->rope_theta, (double)(2 * j) / (double)D));
        cudaMemcpyAsync(m->d_freq, fr.data(), sizeof(float) * fr.size(), cudaMemcpyHostToDevice, c->stream);
        cudaStreamSynchronize(c->stream);
    }
    MA(model_alloc_t(m, (size_t)T * H, &m->x)); MA(model_alloc_t(m, (size_t)T * nqkv, &m->qkv));
    MA(model_alloc_t(m, (size_t)T * qd, &m->attn)); MA(model_alloc_t(m, (size_t)T * cfg->vocab, &m->logits));
    m->parts_cap = (size_t)MAX_PARTS * T * std::max(std::max(H, nqkv), 2 * F);
    MA(model_alloc_t(m, m->parts_cap, &m->parts));
    MA(model_alloc_t(m, (size_t)T, &m->d_out_tok));
    { int32_t *sp = nullptr; MA(model_alloc_t(m, (size_t)T * 4, &sp)); m->d_sample = sp; }
    auto mk_split = [&](int k, VxSplit *s) {
        size_t hi, lo, so, bo; int kp;
        size_t bytes = vxq_split_bytes(T, k, &hi, &lo, &so, &bo, &kp);
        void *p; int r = model_alloc(m, bytes, &p); if (r != VX_OK) return r;
        cudaMemsetAsync(p, 0, bytes, c->stream);
        char *b = (char *)p;
        *s = VxSplit{(__half *)(b + hi), (__half *)(b + lo), (float *)(b + so), (float *)(b + bo), kp};
        return (int)VX_OK;
    };
    MA(mk_split(H, &m->sp_h)); MA(mk_split(qd, &m->sp_q)); MA(mk_split(F, &m->sp_f));
#undef MA
    if (cudaStreamSynchronize(c->stream) != cudaSuccess) return fail(VX_E_CUDA);
    *out = m;
    return VX_OK;
}

int vx_model_destroy(vx_model *m) {
    if (!m) return VX_E_BAD_ARG;
    VxGuard g(m->c);
    cudaStreamSynchronize(m->c->stream);
    for (void *p : m->owned) cudaFree(p);
    for (auto &r : m->raw) if (r.dev) cudaFree(r.dev);
    if (m->h_step_in) cudaFreeHost(m->h_step_in);
    if (m->h_out_tok) cudaFreeHost(m->h_out_tok);
    if (m->d_run_out) cudaFree(m->d_run_out);
    for (auto e : m->ev_pool) cudaEventDestroy(e);
    for (auto &kv : m->graphs) if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    delete m;
    return VX_OK;
}

vx_ctx *vx_model_ctx(vx_model *m) { return m ? m->c : nullptr; }

int vx_model_get_config(vx_model *m, vx_model_config *out) {
    if (!m || !out) return VX_E_BAD_ARG;
    *out = m->cfg;
    return VX_OK;
}

int vx_model_set_tensor(vx_model *m, int layer, int slot, int type, const void *data, size_t bytes, int on_device) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, !m->finalized, "model already finalized");
    VX_REQUIRE(c, data != nullptr, "nil tensor data");
    int n, k; size_t idx;
    if (layer < 0) {
        VX_REQUIRE(c, slot >= 0 && slot < 3, "bad global slot");
        n = slot == VX_G_FINAL_NORM ? 1 : (slot == VX_G_EMBED && m->tp) ? m->vocab_full : m->cfg.vocab; k = m->cfg.hidden;
        idx = (size_t)m->cfg.n_layers * VX_W_PER_LAYER + slot;
    } else {
        VX_REQUIRE(c, layer < m->cfg.n_layers && slot >= 0 && slot < VX_W_PER_LAYER, "bad layer/slot");
        slot_dims(m->cfg, slot, &n, &k);
        idx = (size_t)layer * VX_W_PER_LAYER + slot;
    }
    size_t want = type_row_bytes(type, k) * (size_t)n;
    if (want == 0) return vx_fail(c, VX_E_UNSUPPORTED, "unsupported GGUF tensor type %d", type);
    if (bytes != want) return vx_fail(c, VX_E_BAD_ARG, "tensor (layer %d slot %d type %d) has %zu bytes, expected %zu", layer, slot, type, bytes, want);
    RawTensor &r = m->raw[idx];
    if (r.dev) { cudaFree(r.dev); r.dev = nullptr; }
    cudaError_t e = cudaMalloc(&r.dev, bytes);
    if (e != cudaSuccess) { cudaGetLastError(); return vx_fail(c, VX_E_OOM, "cudaMalloc(%zu) for weights failed", bytes); }
    VX_CUDA(c, cudaMemcpyAsync(r.dev, data, bytes, on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    r.type = type; r.bytes = bytes;
    return VX_OK;
}

// Repacks the projection matrices for the MMA kernel, concatenating Wq|Wk|Wv and W1|W3 row-wise
// (rows are independent in the GGUF row-major block layout), and releases the raw copies.
// Marks the model as one rank's slice of a tensor-parallel model (call before any tensor is set, on a context that has
// run vx_tp_init).  The model's config holds the LOCAL head / FFN / vocabulary counts; vocab_full is the whole vocabulary,
// which the (replicated) embedding table covers.
int vx_model_enable_tp(vx_model *m, int vocab_full) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, !m->finalized, "model already finalized");
    VX_REQUIRE(c, c->tp != nullptr, "vx_tp_init has not been called on this context");
    VX_REQUIRE(c, vocab_full == m->cfg.vocab * vxtp_world(c), "the local vocabulary must be vocab_full / world");
    for (auto &r : m->raw) VX_REQUIRE(c, r.dev == nullptr, "enable tensor parallelism before setting tensors");
    m->tp = true; m->vocab_full = vocab_full;
    VX_TRY(model_alloc_t(m, (size_t)m->cfg.max_batch_tokens * m->cfg.hidden, &m->ar_buf));
    float2 *sc = nullptr;
    VX_TRY(model_alloc_t(m, (size_t)m->cfg.max_batch_tokens * (1 + vxtp_world(c)), &sc));
    m->tp_scratch = sc;
    return VX_OK;
}

int vx_model_finalize(vx_model *m) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, !m->finalized, "model already finalized");
    const vx_model_config &cf = m->cfg;
    auto raw_at = [&](int layer, int slot) -> RawTensor & { return m->raw[(size_t)layer * VX_W_PER_LAYER + slot]; };
    auto norm_f32 = [&](RawTensor &r, float **dst) -> int {
        if (!r.dev) { *dst = nullptr; return VX_OK; }
        if (r.type != VX_T_F32) return vx_fail(c, VX_E_UNSUPPORTED, "norm weights must be F32 (got type %d)", r.type);
        *dst = (float *)r.dev; m->owned.push_back(r.dev); r.dev = nullptr;   // ownership moves to the model
        return VX_OK;
    };
    // concatenated repack of row groups that share k and the block format
    auto build = [&](std::vector<RawTensor *> srcs, std::vector<int> ns, int k, VxWeight *w) -> int {
        int n_total = 0;
        for (int n : ns) n_total += n;
        const int type = srcs[0]->type;
        for (RawTensor *r : srcs) {
            if (!r->dev) return vx_fail(c, VX_E_BAD_ARG, "a projection tensor was never set");
            if (r->type != type) return vx_fail(c, VX_E_BAD_ARG, "internal: mixed block formats in one fused matrix");
        }
        VxRepackLayout L;
        if (!vxq_layout(type, n_total, k, &L)) return vx_fail(c, VX_E_UNSUPPORTED, "projection type %d: no device kernel (Q4_0, Q4_K, Q6_K)", type);
        void *p; VX_TRY(model_alloc(m, L.total, &p));
        int row = 0;
        for (size_t i = 0; i < srcs.size(); i++) {
            VX_TRY(vxq_repack_rows(c, type, srcs[i]->dev, ns[i], k, p, L, row));
            row += ns[i];
        }
        vxq_weight_view(type, n_total, k, p, L, w);
        m->weight_bytes += w->bytes;
        VX_CUDA(c, cudaStreamSynchronize(c->stream));
        for (RawTensor *r : srcs) { cudaFree(r->dev); r->dev = nullptr; }
        return VX_OK;
    };
    const int qd = cf.n_heads * cf.head_dim, kvd = cf.n_kv_heads * cf.head_dim;
    for (int l = 0; l < cf.n_layers; l++) {
        LayerW &L = m->layers[l];
        VX_TRY(norm_f32(raw_at(l, VX_W_ATTN_NORM), &L.attn_norm));
        VX_TRY(norm_f32(raw_at(l, VX_W_FFN_NORM), &L.ffn_norm));
        VX_TRY(norm_f32(raw_at(l, VX_W_POST_ATTN_NORM), &L.post_attn_norm));
        VX_TRY(norm_f32(raw_at(l, VX_W_POST_FFN_NORM), &L.post_ffn_norm));
        VX_REQUIRE(c, L.attn_norm && L.ffn_norm, "attn_norm / ffn_norm missing");
        if (cf.post_norms) VX_REQUIRE(c, L.post_attn_norm && L.post_ffn_norm, "post norms missing");
        {   // fuse consecutive Q/K/V tensors of the same block format (Q4_K_M keeps attn_v in Q6_K)
            RawTensor *t3[3] = {&raw_at(l, VX_W_WQ), &raw_at(l, VX_W_WK), &raw_at(l, VX_W_WV)};
            const int n3[3] = {qd, kvd, kvd};
            for (int i = 0, col = 0; i < 3;) {
                std::vector<RawTensor *> grp; std::vector<int> ns; int cols = 0, j = i;
                for (; j < 3 && t3[j]->type == t3[i]->type; j++) { grp.push_back(t3[j]); ns.push_back(n3[j]); cols += n3[j]; }
                ColW cw; cw.col = col;
                VX_TRY(build(grp, ns, cf.hidden, &cw.w));
                L.wqkv.push_back(cw);
                col += cols; i = j;
            }
        }
        VX_TRY(build({&raw_at(l, VX_W_WO)}, {cf.hidden}, qd, &L.wo));
        if (raw_at(l, VX_W_W1).type != raw_at(l, VX_W_W3).type) return vx_fail(c, VX_E_UNSUPPORTED, "ffn_gate and ffn_up must share a block format");
        VX_TRY(build({&raw_at(l, VX_W_W1), &raw_at(l, VX_W_W3)}, {cf.ffn, cf.ffn}, cf.hidden, &L.w13));
        VX_TRY(build({&raw_at(l, VX_W_W2)}, {cf.hidden}, cf.ffn, &L.w2));
        m->weight_bytes += (size_t)cf.hidden * 4 * (cf.post_norms ? 4 : 2);
    }
    size_t gi = (size_t)cf.n_layers * VX_W_PER_LAYER;
    RawTensor &emb = m->raw[gi + VX_G_EMBED], &fn = m->raw[gi + VX_G_FINAL_NORM], &outw = m->raw[gi + VX_G_OUTPUT];
    VX_REQUIRE(c, emb.dev && fn.dev, "token embedding / final norm missing");
    VX_REQUIRE(c, emb.type == VX_T_Q4_0 || emb.type == VX_T_F32, "token embedding must be Q4_0 or F32");
    VX_TRY(norm_f32(fn, &m->final_norm));
    m->weight_bytes += (size_t)cf.hidden * 4;
    if (outw.dev) {
        VX_TRY(build({&outw}, {cf.vocab}, cf.hidden, &m->w_out));
    } else {   // tied output head (runtime/loader.go:596-600)
        VX_REQUIRE(c, emb.type == VX_T_Q4_0, "tied output head needs a Q4_0 embedding");
        RawTensor copy = emb;
        void *dup; VX_CUDA(c, cudaMalloc(&dup, emb.bytes));
        VX_CUDA(c, cudaMemcpyAsync(dup, emb.dev, emb.bytes, cudaMemcpyDeviceToDevice, c->stream));
        copy.dev = dup;
        VX_TRY(build({&copy}, {cf.vocab}, cf.hidden, &m->w_out));   // frees the duplicate
    }
    m->embed = emb; m->owned.push_back(emb.dev); emb.dev = nullptr;
    m->finalized = true;
    return VX_OK;
}

int vx_seq_create(vx_model *m, int64_t id) {
    if (!m) return VX_E_BAD_ARG;
    VxGuard g(m->c);
    if (m->seq_slot.count(id)) {   // re-creating an id starts it from empty; its blocks go back to the pool
        VX_TRY(vx_seq_truncate(m, id, 0));
        return VX_OK;
    }
    int s;
    return get_slot(m, id, true, &s);
}

int vx_seq_delete(vx_model *m, int64_t id) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    auto it = m->seq_slot.find(id);
    if (it == m->seq_slot.end()) return VX_OK;   // unknown ids are ignored (runtime/gpu_block_pool.go:144-147)
    int s = it->second;
    seq_release_kernel<<<1, 1, 0, c->stream>>>(m->d_tables, m->cfg.max_blocks_per_seq, m->d_n_blocks, m->d_seq_len, m->d_free_list,
                                               m->d_free_top, m->d_refcnt, s, 0, 0);
    VX_LAUNCH_CHECK(c);
    m->seq_slot.erase(it); m->free_slots.push_back(s);
    m->h_seq_len[s] = 0; m->h_n_blocks[s] = 0;
    return refresh_free(m);
}

int vx_seq_truncate(vx_model *m, int64_t id, int new_len) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    auto it = m->seq_slot.find(id);
    if (it == m->seq_slot.end()) return VX_OK;                          // runtime/gpu_block_pool.go:169-172
    int s = it->second;
    if (new_len < 0 || new_len >= m->h_seq_len[s]) return VX_OK;
    int keep = new_len > 0 ? (new_len - 1) / BS + 1 : 0;
    seq_release_kernel<<<1, 1, 0, c->stream>>>(m->d_tables, m->cfg.max_blocks_per_seq, m->d_n_blocks, m->d_seq_len, m->d_free_list,
                                               m->d_free_top, m->d_refcnt, s, keep, new_len);
    VX_LAUNCH_CHECK(c);
    m->h_seq_len[s] = new_len; m->h_n_blocks[s] = std::min(m->h_n_blocks[s], keep);
    return refresh_free(m);
}

int vx_seq_share(vx_model *m, int64_t src, int64_t dst, int n_tokens) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    int a, b;
    VX_TRY(get_slot(m, src, false, &a));
    VX_TRY(get_slot(m, dst, false, &b));
    int nb = (n_tokens + BS - 1) / BS;
    if (nb > m->h_n_blocks[a]) return vx_fail(c, VX_E_BAD_ARG, "source seq has %d blocks, need %d", m->h_n_blocks[a], nb);
    if (m->h_n_blocks[b] + nb > m->cfg.max_blocks_per_seq) return vx_fail(c, VX_E_OOM_BLOCKS, "destination block table is full");
    seq_share_kernel<<<1, 1, 0, c->stream>>>(m->d_tables, m->cfg.max_blocks_per_seq, m->d_n_blocks, m->d_seq_len, m->d_refcnt, a, b, nb, n_tokens);
    VX_LAUNCH_CHECK(c);
    m->h_n_blocks[b] += nb;
    if (n_tokens > m->h_seq_len[b]) m->h_seq_len[b] = n_tokens;
    return VX_OK;
}

int vx_seq_len(vx_model *m, int64_t id, int *out_len) {
    if (!m || !out_len) return VX_E_BAD_ARG;
    VxGuard g(m->c);
    int s;
    VX_TRY(get_slot(m, id, false, &s));
    *out_len = m->h_seq_len[s];
    return VX_OK;
}

int vx_seq_block_table(vx_model *m, int64_t id, int32_t *out, int cap, int *out_n) {
    if (!m || !out_n) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    int s;
    VX_TRY(get_slot(m, id, false, &s));
    int32_t nb = 0;
    VX_CUDA(c, cudaMemcpyAsync(&nb, m->d_n_blocks + s, 4, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    *out_n = nb;
    int n = std::min(nb, cap);
    if (out && n > 0) {
        VX_CUDA(c, cudaMemcpyAsync(out, m->d_tables + (size_t)s * m->cfg.max_blocks_per_seq, 4 * (size_t)n, cudaMemcpyDeviceToHost, c->stream));
        VX_CUDA(c, cudaStreamSynchronize(c->stream));
    }
    return VX_OK;
}

int vx_pool_stats(vx_model *m, int *total, int *free_blocks, int *shared) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_TRY(refresh_free(m));
    // every layer's pool evolves identically, so totals are per-layer counts times n_layers (gpu_block_pool.go:610-625)
    if (total) *total = m->cfg.max_blocks * m->cfg.n_layers;
    if (free_blocks) *free_blocks = m->h_free * m->cfg.n_layers;
    if (shared) {
        std::vector<int32_t> rc(m->cfg.max_blocks);
        VX_CUDA(c, cudaMemcpy(rc.data(), m->d_refcnt, 4 * rc.size(), cudaMemcpyDeviceToHost));
        int n = 0;
        for (int v : rc) n += v > 1;
        *shared = n * m->cfg.n_layers;
    }
    return VX_OK;
}

// the free list as the stack it is, bottom first: the next block handed out is the last entry (gpu_block_pool.go:200-208)
int vx_pool_free_list(vx_model *m, int32_t *out, int cap, int *n_out) {
    if (!m || !n_out) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_TRY(refresh_free(m));
    *n_out = m->h_free;
    const int n = std::min(m->h_free, cap);
    if (out && n > 0) {
        VX_CUDA(c, cudaMemcpyAsync(out, m->d_free_list, 4 * (size_t)n, cudaMemcpyDeviceToHost, c->stream));
        VX_CUDA(c, cudaStreamSynchronize(c->stream));
    }
    return VX_OK;
}

int vx_pool_layer_ptr(vx_model *m, int layer, vx_dptr *out, size_t *bytes) {
    if (!m || !out || layer < 0 || layer >= m->cfg.n_layers) return VX_E_BAD_ARG;
    *out = (vx_dptr)(uintptr_t)(m->pool + (size_t)layer * m->layer_stride);
    if (bytes) *bytes = m->layer_stride * sizeof(__half);
    return VX_OK;
}

int vx_pool_shuffle_free_list(vx_model *m, uint32_t seed) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->seq_slot.empty() && m->h_free == m->cfg.max_blocks, "the free list can only be shuffled while no sequence holds blocks");
    int32_t *tmp;
    VX_CUDA(c, cudaMalloc(&tmp, sizeof(int32_t) * m->cfg.max_blocks));
    shuffle_free_list_kernel<<<std::min(1024, ceil_div(m->cfg.max_blocks, 128)), 128, 0, c->stream>>>(m->d_free_list, tmp, m->cfg.max_blocks, seed);
    cudaMemcpyAsync(m->d_free_list, tmp, sizeof(int32_t) * m->cfg.max_blocks, cudaMemcpyDeviceToDevice, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return vx_cuda_fail(c, e, "shuffle free list");
    return VX_OK;
}

int vx_seq_fill_synthetic(vx_model *m, int64_t id, int len, uint32_t seed) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    int s;
    VX_TRY(get_slot(m, id, true, &s));
    VX_REQUIRE(c, len > 0 && len >= m->h_seq_len[s], "length must grow");
    int nb = (len + BS - 1) / BS;
    if (nb > m->cfg.max_blocks_per_seq || nb - m->h_n_blocks[s] > m->h_free) return vx_fail(c, VX_E_OOM_BLOCKS, "not enough free blocks for %d tokens", len);
    seq_grow_kernel<<<1, 1, 0, c->stream>>>(m->d_tables, m->cfg.max_blocks_per_seq, m->d_n_blocks, m->d_seq_len, m->d_free_list, m->d_free_top,
                                            m->d_refcnt, s, len, m->d_status);
    VX_LAUNCH_CHECK(c);
    m->h_free -= nb - m->h_n_blocks[s]; m->h_n_blocks[s] = nb; m->h_seq_len[s] = len;
    int hs = m->cfg.n_kv_heads * m->cfg.head_dim;
    fill_noise_kernel<<<c->sm_count * 8, 256, 0, c->stream>>>(m->pool, m->layer_stride, m->cfg.n_layers,
                                                              m->d_tables + (size_t)s * m->cfg.max_blocks_per_seq, len, hs, seed);
    VX_LAUNCH_CHECK(c);
    return check_status(m);
}

int vx_decode_step(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                   const int32_t *q_lens, int32_t *out_tokens, float *logits) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->finalized, "model not finalized");
    VX_REQUIRE(c, n_seqs > 0 && n_seqs <= m->cfg.max_seqs && seq_ids && tokens && positions, "bad arguments");
    std::vector<int> slots(n_seqs);
    for (int i = 0; i < n_seqs; i++) VX_TRY(get_slot(m, seq_ids[i], true, &slots[i]));   // created on first use (runtime/decode.go:362-364)
    return run_step(m, n_seqs, slots.data(), tokens, positions, q_lens, 0, 0, out_tokens, logits);
}

// vx_decode_step with options.  flags: VX_STEP_LAST_ROWS = outputs (tokens, logits, hidden, sampling records) cover the last
// row of every batch entry only, n_seqs rows in batch order; VX_STEP_PROMPT_ROWS = multi-row entries are prompt chunks
// (PrefillWithPagedKV, runtime/decode.go:961-1096): an entry that starts at position 0 attends over its fresh float32 K/V.
// hidden (optional, host): post-final-norm hidden states of the output rows, [rows, hidden] float32, what
// VerifySpeculativeWithPagedKVAndHidden hands to the Medusa heads (runtime/decode.go:1543-1557).
int vx_decode_step_ex(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                      const int32_t *q_lens, int flags, const vx_sample_params *params, int32_t *out_tokens, float *logits, float *hidden) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->finalized, "model not finalized");
    VX_REQUIRE(c, n_seqs > 0 && n_seqs <= m->cfg.max_seqs && seq_ids && tokens && positions, "bad arguments");
    VX_REQUIRE(c, (flags & ~(VX_STEP_LAST_ROWS | VX_STEP_PROMPT_ROWS)) == 0, "unknown step flag");
    std::vector<int> slots(n_seqs);
    for (int i = 0; i < n_seqs; i++) VX_TRY(get_slot(m, seq_ids[i], true, &slots[i]));
    return run_step(m, n_seqs, slots.data(), tokens, positions, q_lens, flags, 0, out_tokens, logits, params, hidden);
}

// vx_decode_step followed by Sampler.Sample (pkg/sampler/sampler.go:49-76) on the device: one parameter record per
// packed row, the uniform draw supplied by the caller.  Rows with temperature 0 are greedy.
int vx_decode_step_sampled(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                           const int32_t *q_lens, const vx_sample_params *params, int32_t *out_tokens, float *logits) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->finalized, "model not finalized");
    VX_REQUIRE(c, n_seqs > 0 && n_seqs <= m->cfg.max_seqs && seq_ids && tokens && positions && params, "bad arguments");
    std::vector<int> slots(n_seqs);
    for (int i = 0; i < n_seqs; i++) VX_TRY(get_slot(m, seq_ids[i], true, &slots[i]));
    return run_step(m, n_seqs, slots.data(), tokens, positions, q_lens, 0, 0, out_tokens, logits, params);
}

// Greedy generation for a fixed batch with the token feedback kept on the device: step s+1 is fed the
// argmax of step s without a host round trip.  Only the first step's inputs cross PCIe; all produced
// tokens come back in one copy at the end.  device_ms (optional) is the CUDA-event time of the n_steps
// steps on the context's stream, measured after the first step's inputs are resident.
int vx_decode_run(vx_model *m, int n_seqs, const int64_t *seq_ids, const int32_t *tokens, const int32_t *positions,
                  int n_steps, int32_t *out_tokens, float *device_ms) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->finalized, "model not finalized");
    VX_REQUIRE(c, n_seqs > 0 && n_seqs <= m->cfg.max_seqs && n_seqs <= m->cfg.max_batch_tokens && seq_ids && tokens && positions && n_steps > 0, "bad arguments");
    std::vector<int> slots(n_seqs);
    for (int i = 0; i < n_seqs; i++) VX_TRY(get_slot(m, seq_ids[i], true, &slots[i]));
    // admission for the whole run up front: blocks needed after n_steps tokens
    long need = 0;
    for (int i = 0; i < n_seqs; i++) {
        if (positions[i] != m->h_seq_len[slots[i]]) return vx_fail(c, VX_E_BAD_ARG, "position %d of batch entry %d != sequence length %d", positions[i], i, m->h_seq_len[slots[i]]);
        int nb = (positions[i] + n_steps + BS - 1) / BS;
        if (nb > m->cfg.max_blocks_per_seq) return vx_fail(c, VX_E_OOM_BLOCKS, "sequence would need %d blocks (table width %d)", nb, m->cfg.max_blocks_per_seq);
        need += std::max(0, nb - m->h_n_blocks[slots[i]]);
    }
    if (need > m->h_free) return vx_fail(c, VX_E_OOM_BLOCKS, "no free blocks: need %ld, have %d (max=%d)", need, m->h_free, m->cfg.max_blocks);
    if (m->run_out_cap < (size_t)n_steps * n_seqs) {
        if (m->d_run_out) { cudaStreamSynchronize(c->stream); cudaFree(m->d_run_out); m->d_run_out = nullptr; }
        VX_CUDA(c, cudaMalloc(&m->d_run_out, sizeof(int32_t) * (size_t)n_steps * n_seqs));
        m->run_out_cap = (size_t)n_steps * n_seqs;
    }
    int32_t *h = m->h_step_in;
    for (int i = 0; i < n_seqs; i++) { h[i] = slots[i]; h[n_seqs + i] = 1; h[2 * n_seqs + i] = positions[i]; h[3 * n_seqs + i] = 0; h[4 * n_seqs + i] = tokens[i]; }
    VX_CUDA(c, cudaMemcpyAsync(m->d_step_in, h, sizeof(int32_t) * 5 * n_seqs, cudaMemcpyHostToDevice, c->stream));
    cudaEvent_t e0, e1;
    VX_CUDA(c, cudaEventCreate(&e0)); VX_CUDA(c, cudaEventCreate(&e1));
    cudaEventRecord(e0, c->stream);
    std::vector<int32_t> pos(positions, positions + n_seqs);
    int rc = VX_OK;
    for (int st = 0; st < n_steps && rc == VX_OK; st++) {
        StepPlan p;
        rc = plan_step(m, n_seqs, slots.data(), pos.data(), nullptr, false, &p);
        if (rc != VX_OK) break;
        if (st > 0) {
            advance_step_kernel<<<ceil_div(n_seqs, 256), 256, 0, c->stream>>>(m->d_step_in, n_seqs, m->d_out_tok);
            c->launches++;
        }
        rc = enqueue_step(m, p, 0, n_seqs);
        if (rc != VX_OK) break;
        cudaMemcpyAsync(m->d_run_out + (size_t)st * n_seqs, m->d_out_tok, sizeof(int32_t) * n_seqs, cudaMemcpyDeviceToDevice, c->stream);
        for (int i = 0; i < n_seqs; i++) pos[i]++;
    }
    cudaEventRecord(e1, c->stream);
    int rc2 = check_status(m);
    time_collect(m);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (device_ms) *device_ms = ms;
    if (rc != VX_OK || rc2 != VX_OK) resync_mirror(m);
    if (rc != VX_OK) return rc;
    if (rc2 != VX_OK) return rc2;
    if (out_tokens) VX_CUDA(c, cudaMemcpy(out_tokens, m->d_run_out, sizeof(int32_t) * (size_t)n_steps * n_seqs, cudaMemcpyDeviceToHost));
    return VX_OK;
}

static int prefill_impl(vx_model *m, int64_t id, const int32_t *tokens, int n_tokens, int start_pos, const vx_sample_params *sample,
                        int32_t *out_token, float *logits) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->finalized, "model not finalized");
    VX_REQUIRE(c, tokens && n_tokens > 0 && start_pos >= 0, "bad arguments");
    int slot;
    VX_TRY(get_slot(m, id, true, &slot));
    const int T = m->cfg.max_batch_tokens;
    int done = 0;
    while (done < n_tokens) {
        int n = std::min(T, n_tokens - done);
        int pos = start_pos + done, ql = n;
        bool last = done + n == n_tokens;
        // the first chunk of a prompt that starts at 0 attends over its own float32 K/V (SDPAPrefill);
        // later chunks read the paged fp16 cache like the multi-query verify path
        VX_TRY(run_step(m, 1, &slot, tokens + done, &pos, &ql, VX_STEP_PROMPT_ROWS, 1, last ? out_token : nullptr, last ? logits : nullptr,
                        last ? sample : nullptr));
        done += n;
    }
    return VX_OK;
}

int vx_prefill(vx_model *m, int64_t id, const int32_t *tokens, int n_tokens, int start_pos, int32_t *out_token, float *logits) {
    return prefill_impl(m, id, tokens, n_tokens, start_pos, nullptr, out_token, logits);
}

// vx_prefill whose first generated token is drawn by Sampler.Sample from the last prompt position's logits
int vx_prefill_sampled(vx_model *m, int64_t id, const int32_t *tokens, int n_tokens, int start_pos, const vx_sample_params *params,
                       int32_t *out_token, float *logits) {
    if (!params) return VX_E_BAD_ARG;
    return prefill_impl(m, id, tokens, n_tokens, start_pos, params, out_token, logits);
}

int vx_model_set_capture(vx_model *m, int enable) {
    if (!m) return VX_E_BAD_ARG;
    VxGuard g(m->c);
    if (enable && !m->capture) {
        size_t n = (size_t)(m->cfg.n_layers + 1) * m->cfg.max_batch_tokens * m->cfg.hidden;
        VX_TRY(model_alloc_t(m, n, &m->capture));
    }
    m->capture_on = enable != 0;
    return VX_OK;
}

int vx_model_get_capture(vx_model *m, float *host_out, size_t n_floats) {
    if (!m || !host_out) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, m->capture != nullptr, "capture was never enabled");
    size_t have = (size_t)(m->cfg.n_layers + 1) * m->capture_rows * m->cfg.hidden;
    VX_REQUIRE(c, n_floats >= have, "capture buffer too small");
    VX_CUDA(c, cudaMemcpyAsync(host_out, m->capture, have * 4, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    return VX_OK;
}

int vx_model_get_packing(vx_model *m, int32_t *cu, int32_t *slot_map, int32_t *row_kv_len, int n_seqs, int n_rows) {
    if (!m) return VX_E_BAD_ARG;
    vx_ctx *c = m->c;
    VxGuard g(c);
    VX_REQUIRE(c, n_seqs == m->last_seqs && n_rows == m->last_rows, "shape does not match the last step");
    if (cu) VX_CUDA(c, cudaMemcpyAsync(cu, m->d_cu, 4 * (size_t)(n_seqs + 1), cudaMemcpyDeviceToHost, c->stream));
    if (slot_map) VX_CUDA(c, cudaMemcpyAsync(slot_map, m->d_slot_map, 4 * (size_t)n_rows, cudaMemcpyDeviceToHost, c->stream));
    if (row_kv_len) VX_CUDA(c, cudaMemcpyAsync(row_kv_len, m->d_row_kv_len, 4 * (size_t)n_rows, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    return VX_OK;
}

int vx_model_counters(vx_model *m, uint64_t *launches, uint64_t *steps) {
    if (!m) return VX_E_BAD_ARG;
    if (launches) *launches = m->c->launches;
    if (steps) *steps = m->steps;
    return VX_OK;
}

int vx_model_graph_stats(vx_model *m, uint64_t *replays, uint64_t *takeovers) {
    if (!m) return VX_E_BAD_ARG;
    if (replays) *replays = m->graph_replays;
    if (takeovers) *takeovers = m->graph_updates;
    return VX_OK;
}

int vx_model_kernel_time(vx_model *m, int which, int enable, float *ms, uint64_t *launches) {
    if (!m || which < 0 || which > 1) return VX_E_BAD_ARG;
    VxGuard g(m->c);
    if (ms) *ms = m->time_ms[which];
    if (launches) *launches = m->time_n[which];
    if (enable >= 0) {
        if ((enable != 0) != m->time_on[which]) { m->time_ms[which] = 0; m->time_n[which] = 0; }
        m->time_on[which] = enable != 0;
    }
    return VX_OK;
}

int vx_set_graphs(int enable) { g_graphs = enable != 0; return VX_OK; }
int vx_debug_skip(int mask) { g_dbg_skip = mask; return VX_OK; }

int vx_model_max_blocks(vx_model *m) { return m ? m->cfg.max_blocks : 0; }

int vx_model_weight_bytes(vx_model *m, uint64_t *bytes) {
    if (!m || !bytes) return VX_E_BAD_ARG;
    *bytes = m->weight_bytes;
    return VX_OK;
}

}  // extern "C"
