// Interface-level float32 kernels of backend.Backend and the optional capability interfaces
// (inference/backend/backend.go:199-263, 333-390).  Arithmetic follows inference/backend/cpu/cpu.go;
// only the order of long reductions differs (parallel instead of sequential).
#include "vx_common.cuh"

// ------------------------------------------------------------------ elementwise
// transcendental functions are evaluated in float64 and rounded once, as cpu.go does with math.Exp/Tanh
__device__ __forceinline__ float silu_f(float v) {          // cpu.go:378-387
    float sg = 1.0f / (1.0f + (float)exp((double)(-v)));
    return v * sg;
}
__device__ __forceinline__ float gelu_f(float v) {          // cpu.go:440-454
    const float s2pi = 0.7978845608f, coeff = 0.044715f;
    float x3 = __fmul_rn(__fmul_rn(v, v), v);
    float ta = __fmul_rn(s2pi, __fadd_rn(v, __fmul_rn(coeff, x3)));
    float th = (float)tanh((double)ta);
    return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, th));
}

enum { EW_SILU, EW_GELU, EW_SILU_MUL, EW_GELU_MUL, EW_ADD, EW_MUL, EW_SCALE };

template <int OP>
__global__ void ew_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, float s, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    int stride = gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        float r;
        if (OP == EW_SILU) r = silu_f(a[i]);
        else if (OP == EW_GELU) r = gelu_f(a[i]);
        else if (OP == EW_SILU_MUL) r = __fmul_rn(silu_f(a[i]), b[i]);
        else if (OP == EW_GELU_MUL) r = __fmul_rn(gelu_f(a[i]), b[i]);
        else if (OP == EW_ADD) r = __fadd_rn(a[i], b[i]);
        else if (OP == EW_MUL) r = __fmul_rn(a[i], b[i]);
        else r = __fmul_rn(a[i], s);
        out[i] = r;
    }
}

template <int OP>
static int ew_launch(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, float s, int n) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (n <= 0) return VX_OK;
    VX_REQUIRE(c, a != 0 && out != 0, "nil device pointer");
    int blocks = min(ceil_div(n, 256), c->sm_count * 8);
    ew_kernel<OP><<<blocks, 256, 0, c->stream>>>(dp<float>(a), dp<float>(b), dp<float>(out), s, n);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// ------------------------------------------------------------------ RMSNorm (cpu.go:200-220)
__global__ void rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ out,
                               int cols, float eps) {
    __shared__ float red[32];
    const float *xr = x + (size_t)blockIdx.x * cols;
    float *o = out + (size_t)blockIdx.x * cols;
    float ss = 0.f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) { float v = xr[j]; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, red);
    float mean = __fdiv_rn(ss, (float)cols);
    float rms = __fsqrt_rn(__fadd_rn(mean, eps));
    for (int j = threadIdx.x; j < cols; j += blockDim.x) o[j] = __fmul_rn(__fdiv_rn(xr[j], rms), w[j]);
}

// ------------------------------------------------------------------ RoPE (cpu.go:226-375)
// one thread per (vector, rotated pair); vectors = seq_len*heads for q followed by seq_len*kv_heads for k
__global__ void rope_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ freqs,
                            int head_dim, int n_heads, int n_kv_heads, int seq_len, int start_pos,
                            int eff_dim, float theta, int neox) {
    int half = eff_dim / 2;
    int nq = seq_len * n_heads, nk = k ? seq_len * n_kv_heads : 0;
    long total = (long)(nq + nk) * half;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
        int vec = (int)(idx / half), j = (int)(idx % half);
        float *v; int pos;
        if (vec < nq) { v = q + (size_t)vec * head_dim; pos = start_pos + vec / n_heads; }
        else { int kv = vec - nq; v = k + (size_t)kv * head_dim; pos = start_pos + kv / n_kv_heads; }
        float freq;
        if (freqs) freq = freqs[j];
        else freq = (float)(1.0 / pow((double)theta, (double)(2 * j) / (double)eff_dim));
        float angle = __fmul_rn((float)pos, freq);
        float cs = (float)cos((double)angle), sn = (float)sin((double)angle);
        int i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
        float a = v[i0], b = v[i1];
        v[i0] = __fsub_rn(__fmul_rn(a, cs), __fmul_rn(b, sn));
        v[i1] = __fadd_rn(__fmul_rn(a, sn), __fmul_rn(b, cs));
    }
}

// ------------------------------------------------------------------ Softmax (cpu.go:490-518)
__global__ void softmax_kernel(const float *__restrict__ x, float *__restrict__ out, int cols) {
    __shared__ float red[32];
    const float *r = x + (size_t)blockIdx.x * cols;
    float *o = out + (size_t)blockIdx.x * cols;
    float mx = -INFINITY;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) mx = fmaxf(mx, r[j]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) { float e = (float)exp((double)(r[j] - mx)); o[j] = e; sum += e; }
    sum = block_sum(sum, red);
    float inv = __fdiv_rn(1.0f, sum);
    for (int j = threadIdx.x; j < cols; j += blockDim.x) o[j] = __fmul_rn(o[j], inv);
}

// ------------------------------------------------------------------ Embedding (cpu.go:543-555)
__global__ void embedding_kernel(const int32_t *__restrict__ ids, const float *__restrict__ table,
                                 float *__restrict__ out, int vocab, int dim) {
    int id = ids[blockIdx.x];
    if (id < 0 || id >= vocab) return;   // out-of-range ids leave the row untouched
    const float *src = table + (size_t)id * dim;
    float *dst = out + (size_t)blockIdx.x * dim;
    for (int j = threadIdx.x; j < dim; j += blockDim.x) dst[j] = src[j];
}

// ------------------------------------------------------------------ Argmax (pkg/sampler/sampler.go:79-90)
// strict '>' scan: the first index holding the maximum wins; NaNs never win (x > max is false)
__global__ void argmax_rows_kernel(const float *__restrict__ x, int cols, int32_t *__restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const float *r = x + (size_t)blockIdx.x * cols;
    float bv = -3.402823466e+38f; int bi = 0x7fffffff;
    for (int j = threadIdx.x; j < cols; j += blockDim.x) {
        float v = r[j];
        if (v > bv) { bv = v; bi = j; }
    }
    auto better = [](float v, int i, float ov, int oi) { return (ov > v) || (ov == v && oi < i); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(bv, bi, ov, oi)) { bv = ov; bi = oi; }
    }
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        bv = lane < nw ? sv[lane] : -3.402823466e+38f; bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(bv, bi, ov, oi)) { bv = ov; bi = oi; }
        }
        // every element <= -MaxFloat32 (or NaN): sampler.Argmax returns index 0
        if (lane == 0) out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
}

// ------------------------------------------------------------------ plain float32 matmul
// out[i][j] = sum_p a[i][p] * B(p, j); TRANS: B stored [n][k] (cpu.go:158-197) else [k][n] (cpu.go:106-144).
// One warp per output column tile; used for interface completeness and F32 output heads, not the hot path.
template <bool TRANS>
__global__ void matmul_f32_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                  int m, int n, int k) {
    int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    int j = warp;   // output column
    if (j >= n) return;
    for (int i = 0; i < m; i++) {
        float s = 0.f;
        for (int p = lane; p < k; p += 32) {
            float bv = TRANS ? b[(size_t)j * k + p] : b[(size_t)p * n + j];
            s = fmaf(a[(size_t)i * k + p], bv, s);
        }
        s = warp_sum(s);
        if (lane == 0) out[(size_t)i * n + j] = s;
    }
}

// ------------------------------------------------------------------ generic SDPA (contiguous K/V)
// One CTA (256 threads) per (query row, q head).  K/V element (pos, kv head, d) lives at
// base + pos*pos_stride + kvh*head_stride + d.  Online softmax over tiles of 256 positions:
// threads first own positions (scores), then own output dimensions (weighted V sum).
__global__ void sdpa_generic_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                    float *__restrict__ out, int q_ld, int out_ld, int n_q_heads, int n_kv_heads, int head_dim,
                                    long pos_stride, long head_stride, int kv_len_fixed, int causal_rows,
                                    float scale, float softcap) {
    extern __shared__ float sm[];
    float *qs = sm;                 // [head_dim]
    float *ps = sm + head_dim;      // [256]
    __shared__ float red[32];
    int h = blockIdx.x, row = blockIdx.y;
    int kvh = h / (n_q_heads / n_kv_heads);
    int kv_len = causal_rows ? row + 1 : kv_len_fixed;
    const float *qh = q + (size_t)row * q_ld + (size_t)h * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) qs[d] = qh[d];
    __syncthreads();
    float m_run = -INFINITY, l_run = 0.f, acc = 0.f;   // acc: output dim threadIdx.x (head_dim <= 256)
    for (int t0 = 0; t0 < kv_len; t0 += 256) {
        int pos = t0 + threadIdx.x;
        float s = -INFINITY;
        if (pos < kv_len) {
            const float *kp = k + (size_t)pos * pos_stride + (size_t)kvh * head_stride;
            float dot = 0.f;
            for (int d = 0; d < head_dim; d++) dot = fmaf(qs[d], kp[d], dot);
            s = dot * scale;
            if (softcap > 0.f) s = softcap * (float)tanh((double)(s / softcap));
        }
        float tmax = block_max(s, red);
        float m_new = fmaxf(m_run, tmax);
        float p = pos < kv_len ? __expf(s - m_new) : 0.f;
        float corr = __expf(m_run - m_new);
        float psum = block_sum(p, red);
        ps[threadIdx.x] = p;
        __syncthreads();
        l_run = l_run * corr + psum;
        acc *= corr;
        if (threadIdx.x < head_dim) {
            int cnt = min(256, kv_len - t0);
            const float *vp = v + (size_t)t0 * pos_stride + (size_t)kvh * head_stride + threadIdx.x;
            for (int i = 0; i < cnt; i++) acc = fmaf(ps[i], vp[(size_t)i * pos_stride], acc);
        }
        m_run = m_new;
        __syncthreads();
    }
    if (threadIdx.x < head_dim) out[(size_t)row * out_ld + (size_t)h * head_dim + threadIdx.x] = acc / l_run;
}

int vxe_sdpa_strided(vx_ctx *c, const float *q, int q_ld, const float *k, const float *v, float *out, int out_ld, int rows, int kv_len,
                     int causal, int hq, int hkv, int d, long pos_stride, long head_stride, float scale, float softcap) {
    VX_REQUIRE(c, q && k && v && out, "nil device pointer");
    VX_REQUIRE(c, hq > 0 && hkv > 0 && hq % hkv == 0 && d > 0 && d <= 256, "bad head configuration (head_dim <= 256)");
    VX_REQUIRE(c, rows > 0 && (causal || kv_len > 0), "empty attention");
    dim3 grid(hq, rows);
    size_t smem = (size_t)(d + 256) * sizeof(float);
    sdpa_generic_kernel<<<grid, 256, smem, c->stream>>>(q, k, v, out, q_ld, out_ld, hq, hkv, d, pos_stride, head_stride, kv_len, causal,
                                                        scale, softcap);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

static int sdpa_launch(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int rows, int kv_len, int causal,
                       int hq, int hkv, int d, long pos_stride, long head_stride, float scale, float softcap) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    return vxe_sdpa_strided(c, dp<float>(q), hq * d, dp<float>(k), dp<float>(v), dp<float>(out), hq * d, rows, kv_len, causal, hq, hkv, d,
                            pos_stride, head_stride, scale, softcap);
}

int vxe_argmax_rows(vx_ctx *c, const float *x, int rows, int cols, int32_t *out) {
    argmax_rows_kernel<<<rows, 1024, 0, c->stream>>>(x, cols, out);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

extern "C" {

int vx_silu(vx_ctx *c, vx_dptr x, vx_dptr out, int n) { return ew_launch<EW_SILU>(c, x, 0, out, 0.f, n); }
int vx_gelu(vx_ctx *c, vx_dptr x, vx_dptr out, int n) { return ew_launch<EW_GELU>(c, x, 0, out, 0.f, n); }
int vx_silu_mul(vx_ctx *c, vx_dptr gate, vx_dptr up, vx_dptr out, int n) { return ew_launch<EW_SILU_MUL>(c, gate, up, out, 0.f, n); }
int vx_gelu_mul(vx_ctx *c, vx_dptr gate, vx_dptr up, vx_dptr out, int n) { return ew_launch<EW_GELU_MUL>(c, gate, up, out, 0.f, n); }
int vx_add(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int n) { return ew_launch<EW_ADD>(c, a, b, out, 0.f, n); }
int vx_mul(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int n) { return ew_launch<EW_MUL>(c, a, b, out, 0.f, n); }
int vx_scale(vx_ctx *c, vx_dptr buf, float s, int n) { return ew_launch<EW_SCALE>(c, buf, 0, buf, s, n); }

int vx_rmsnorm(vx_ctx *c, vx_dptr x, vx_dptr w, vx_dptr out, int rows, int cols, float eps) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (rows <= 0 || cols <= 0) return VX_OK;
    VX_REQUIRE(c, x && w && out, "nil device pointer");
    rmsnorm_kernel<<<rows, 256, 0, c->stream>>>(dp<float>(x), dp<float>(w), dp<float>(out), cols, eps);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

static int rope_launch(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr freqs, int head_dim, int n_heads, int n_kv_heads,
                       int seq_len, int start_pos, int rope_dim, float theta, int neox) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, q != 0 && head_dim > 0 && n_heads > 0 && seq_len > 0, "bad arguments");
    int eff = rope_dim == 0 ? head_dim : rope_dim;
    VX_REQUIRE(c, eff <= head_dim && eff % 2 == 0, "rope_dim must be even and <= head_dim");
    long total = (long)seq_len * (n_heads + (k ? n_kv_heads : 0)) * (eff / 2);
    long want = (total + 255) / 256, cap = (long)c->sm_count * 16;
    int blocks = (int)(want < cap ? want : cap);
    rope_kernel<<<blocks, 256, 0, c->stream>>>(dp<float>(q), dp<float>(k), dp<float>(freqs), head_dim, n_heads, n_kv_heads,
                                               seq_len, start_pos, eff, theta, neox);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}
int vx_rope(vx_ctx *c, vx_dptr q, vx_dptr k, int head_dim, int n_heads, int n_kv_heads, int seq_len, int start_pos,
            int rope_dim, float theta, int neox) {
    return rope_launch(c, q, k, 0, head_dim, n_heads, n_kv_heads, seq_len, start_pos, rope_dim, theta, neox);
}
int vx_rope_freqs(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr freqs, int head_dim, int n_heads, int n_kv_heads,
                  int seq_len, int start_pos, int neox) {
    if (c && freqs == 0) return vx_fail(c, VX_E_BAD_ARG, "vx_rope_freqs: nil frequency buffer");
    return rope_launch(c, q, k, freqs, head_dim, n_heads, n_kv_heads, seq_len, start_pos, 0, 0.f, neox);
}

int vx_softmax(vx_ctx *c, vx_dptr x, vx_dptr out, int rows, int cols) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (rows <= 0 || cols <= 0) return VX_OK;
    VX_REQUIRE(c, x && out, "nil device pointer");
    softmax_kernel<<<rows, 256, 0, c->stream>>>(dp<float>(x), dp<float>(out), cols);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

int vx_embedding(vx_ctx *c, vx_dptr ids, int n_tokens, vx_dptr table, vx_dptr out, int vocab, int dim) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (n_tokens <= 0) return VX_OK;
    VX_REQUIRE(c, ids && table && out && dim > 0, "bad arguments");
    embedding_kernel<<<n_tokens, 256, 0, c->stream>>>(dp<int32_t>(ids), dp<float>(table), dp<float>(out), vocab, dim);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

int vx_argmax_rows(vx_ctx *c, vx_dptr x, int rows, int cols, vx_dptr out) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, x && out && rows > 0 && cols > 0, "bad arguments");
    argmax_rows_kernel<<<rows, 1024, 0, c->stream>>>(dp<float>(x), cols, dp<int32_t>(out));
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// synchronous like the reference's Metal Argmax (dispatch, Sync, read 4 bytes: backend/metal/backend.go:1795-1811)
int vx_argmax(vx_ctx *c, vx_dptr x, int n, int *out_index) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, x && out_index && n > 0, "bad arguments");
    argmax_rows_kernel<<<1, 1024, 0, c->stream>>>(dp<float>(x), n, c->d_int_result);
    VX_LAUNCH_CHECK(c);
    VX_CUDA(c, cudaMemcpyAsync(c->h_int_result, c->d_int_result, 4, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    *out_index = *c->h_int_result;
    return VX_OK;
}

static int matmul_f32_launch(vx_ctx *c, bool trans, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (m <= 0 || n <= 0) return VX_OK;
    VX_REQUIRE(c, a && b && out && k > 0, "bad arguments");
    int blocks = ceil_div(n * 32, 256);
    if (trans) matmul_f32_kernel<true><<<blocks, 256, 0, c->stream>>>(dp<float>(a), dp<float>(b), dp<float>(out), m, n, k);
    else matmul_f32_kernel<false><<<blocks, 256, 0, c->stream>>>(dp<float>(a), dp<float>(b), dp<float>(out), m, n, k);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}
int vx_matmul_f32(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) { return matmul_f32_launch(c, false, a, b, out, m, n, k); }
int vx_matmul_f32_t(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) { return matmul_f32_launch(c, true, a, b, out, m, n, k); }

// head-major cache: element (pos, kvh, d) at kvh*kv_head_stride + pos*head_dim + d (cpu.go:568-592)
int vx_sdpa(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int kv_len, int hq, int hkv, int d, float scale, int kv_head_stride) {
    return sdpa_launch(c, q, k, v, out, 1, kv_len, 0, hq, hkv, d, d, kv_head_stride, scale, 0.f);
}
int vx_sdpa_softcap(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int kv_len, int hq, int hkv, int d, float scale,
                    float softcap, int kv_head_stride) {
    return sdpa_launch(c, q, k, v, out, 1, kv_len, 0, hq, hkv, d, d, kv_head_stride, scale, softcap);
}
// token-major Q/K/V with causal masking (cpu.go:635-701)
int vx_sdpa_prefill(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int seq_len, int hq, int hkv, int d, float scale) {
    return sdpa_launch(c, q, k, v, out, seq_len, 0, 1, hq, hkv, d, (long)hkv * d, d, scale, 0.f);
}
int vx_sdpa_prefill_softcap(vx_ctx *c, vx_dptr q, vx_dptr k, vx_dptr v, vx_dptr out, int seq_len, int hq, int hkv, int d,
                            float scale, float softcap) {
    return sdpa_launch(c, q, k, v, out, seq_len, 0, 1, hq, hkv, d, (long)hkv * d, d, scale, softcap);
}

}  // extern "C"
