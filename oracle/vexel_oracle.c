/*
 * vexel_oracle.c -- CPU restatement of the reference's batched paged-KV decode path.
 *
 * TEST INFRASTRUCTURE ONLY (see vexel_oracle.h).  Built with
 *   gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC
 * so that every float32 multiply/add rounds on its own, as Go does on amd64.
 *
 * Threads: the reference splits matmuls over the M (token) rows only
 * (backend/cpu/cpu.go:115-143).  Here the loops over *independent output
 * elements* (output columns, heads) are additionally split with OpenMP.  Each
 * output element is still produced by one thread with the reference's exact
 * operation order, so results do not depend on the thread count.
 */
#include "vexel_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ scalar */

/* pkg/gguf/dequant.go:231-261 (same mapping as backend/cpu/cpu.go:962-992 for finite values) */
float vo_f16_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu, f;
    if (exp == 0) {
        if (mant == 0) {
            f = sign << 31;
        } else {
            exp = 127 - 14;
            while ((mant & 0x400u) == 0) { mant <<= 1; exp--; }
            mant &= 0x3FFu;
            f = (sign << 31) | (exp << 23) | (mant << 13);
        }
    } else if (exp == 0x1F) {
        f = (sign << 31) | (0xFFu << 23) | (mant << 13);
    } else {
        f = (sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13);
    }
    float r; memcpy(&r, &f, 4); return r;
}

/* IEEE-754 binary32 -> binary16, round to nearest even (the Metal `(half)x` cast used by
 * reshape_paged_kv_f16, backend/metal/metal_bridge_darwin.m:8641). */
uint16_t vo_f32_to_f16(float fl) {
    uint32_t x; memcpy(&x, &fl, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t e = (x >> 23) & 0xFFu, m = x & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? (0x200u | (m >> 13)) : 0));
    int32_t ne = (int32_t)e - 127 + 15;
    if (ne >= 31) return (uint16_t)(sign | 0x7C00u);
    if (ne <= 0) {
        if (ne < -10) return (uint16_t)sign;
        m |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - ne);
        uint32_t hm = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hm = m >> 13, rem = m & 0x1FFFu;
    uint16_t h = (uint16_t)(sign | ((uint32_t)ne << 10) | hm);
    if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) h++;   /* carry may roll into the exponent: correct */
    return h;
}

/* --------------------------------------------------------------- dequantize */

size_t vo_type_row_bytes(int type, int64_t k) {
    switch (type) {
    case VO_F32:  return (size_t)k * 4;
    case VO_F16:  return (size_t)k * 2;
    case VO_Q4_0: return (size_t)(k / 32) * 18;
    case VO_Q4_K: return (size_t)(k / 256) * 144;
    case VO_Q6_K: return (size_t)(k / 256) * 210;
    default: return 0;
    }
}

/* pkg/gguf/dequant.go:16-56: low nibbles -> elements 0..15, high -> 16..31, w = scale*float32(q-8) */
void vo_dequant_q4_0(const uint8_t *data, int64_t n, float *out) {
    int64_t nb = (n + 31) / 32;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 18;
        float scale = vo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        for (int i = 0; i < 16; i++) {
            uint8_t bv = blk[2 + i];
            int64_t idx = b * 32 + i;
            if (idx < n) out[idx] = scale * (float)((int)(bv & 0x0F) - 8);
            idx = b * 32 + i + 16;
            if (idx < n) out[idx] = scale * (float)((int)((bv >> 4) & 0x0F) - 8);
        }
    }
}

/* pkg/gguf/dequant.go:400-409 */
void vo_scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63; *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* pkg/gguf/dequant.go:342-396: w = d1*float32(q) - dm1 with d1 = d*sc, dm1 = dmin*m (two roundings) */
void vo_dequant_q4_k(const uint8_t *data, int64_t n, float *out) {
    int64_t nb = (n + 255) / 256;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *blk = data + b * 144;
        float d = vo_f16_to_f32((uint16_t)(blk[0] | (blk[1] << 8)));
        float dmin = vo_f16_to_f32((uint16_t)(blk[2] | (blk[3] << 8)));
        const uint8_t *sc = blk + 4, *qs = blk + 16;
        int qoff = 0, is = 0;
        for (int j = 0; j < 256; j += 64) {
            uint8_t s1, m1, s2, m2;
            vo_scale_min_k4(is + 0, sc, &s1, &m1);
            float d1 = d * (float)s1, dm1 = dmin * (float)m1;
            vo_scale_min_k4(is + 1, sc, &s2, &m2);
            float d2 = d * (float)s2, dm2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) {
                int64_t i1 = b * 256 + j + l, i2 = i1 + 32;
                if (i1 < n) out[i1] = d1 * (float)(qs[qoff + l] & 0x0F) - dm1;
                if (i2 < n) out[i2] = d2 * (float)(qs[qoff + l] >> 4) - dm2;
            }
            qoff += 32; is += 2;
        }
    }
}

/* pkg/gguf/dequant.go:272-331: w = (d*float32(sc))*float32(q), q in [-32,31] */
void vo_dequant_q6_k(const uint8_t *data, int64_t n, float *out) {
    int64_t nb = (n + 255) / 256;
    for (int64_t b = 0; b < nb; b++) {
        const uint8_t *ql = data + b * 210, *qh = ql + 128;
        const int8_t *scales = (const int8_t *)(ql + 192);
        float d = vo_f16_to_f32((uint16_t)(ql[208] | (ql[209] << 8)));
        for (int h = 0; h < 2; h++) {
            const uint8_t *l4 = ql + h * 64, *h2 = qh + h * 32;
            const int8_t *sc = scales + h * 8;
            int64_t y = b * 256 + h * 128;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((l4[l] & 0xF) | (((h2[l] >> 0) & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((l4[l + 32] & 0xF) | (((h2[l] >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((l4[l] >> 4) | (((h2[l] >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((l4[l + 32] >> 4) | (((h2[l] >> 6) & 3) << 4)) - 32;
                if (y + l < n)      out[y + l]      = d * (float)sc[is + 0] * (float)q1;
                if (y + l + 32 < n) out[y + l + 32] = d * (float)sc[is + 2] * (float)q2;
                if (y + l + 64 < n) out[y + l + 64] = d * (float)sc[is + 4] * (float)q3;
                if (y + l + 96 < n) out[y + l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
        }
    }
}

void vo_dequant(int type, const uint8_t *data, int64_t n, float *out) {
    switch (type) {
    case VO_F32: memcpy(out, data, (size_t)n * 4); break;
    case VO_F16: for (int64_t i = 0; i < n; i++) out[i] = vo_f16_to_f32(((const uint16_t *)data)[i]); break;
    case VO_Q4_0: vo_dequant_q4_0(data, n, out); break;
    case VO_Q4_K: vo_dequant_q4_k(data, n, out); break;
    case VO_Q6_K: vo_dequant_q6_k(data, n, out); break;
    default: break;
    }
}

/* ------------------------------------------------------------------ kernels */

static int g_threads = 0;
void vo_set_threads(int n) {
    g_threads = n;
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

/* backend/cpu/cpu.go:106-144 */
void vo_matmul(const float *a, const float *b, float *out, int m, int n, int k) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            float sum = 0;
            for (int p = 0; p < k; p++) sum += a[(size_t)i * k + p] * b[(size_t)p * n + j];
            out[(size_t)i * n + j] = sum;
        }
}

/* backend/cpu/cpu.go:158-197 */
void vo_matmul_transposed(const float *a, const float *b, float *out, int m, int n, int k) {
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; j++) {
        const float *br = b + (size_t)j * k;
        for (int i = 0; i < m; i++) {
            const float *ar = a + (size_t)i * k;
            float sum = 0;
            for (int p = 0; p < k; p++) sum += ar[p] * br[p];
            out[(size_t)i * n + j] = sum;
        }
    }
}

/* backend/cpu/cpu.go:842-911: one f32 sum per output; per block byte i: low nibble
 * (elem i) then high nibble (elem i+16); weight = float32(q-8)*scale. */
void vo_matmul_q4_0(const float *a, const uint8_t *bq, float *out, int m, int n, int k) {
    int bpr = k / 32;
#pragma omp parallel for schedule(static)
    for (int j = 0; j < n; j++) {
        const uint8_t *row = bq + (size_t)j * bpr * 18;
        for (int i = 0; i < m; i++) {
            const float *ar = a + (size_t)i * k;
            float sum = 0;
            for (int blk = 0; blk < bpr; blk++) {
                const uint8_t *p = row + blk * 18;
                float scale = vo_f16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
                int base = blk * 32;
                for (int bi = 0; bi < 16; bi++) {
                    uint8_t bv = p[2 + bi];
                    float lo = (float)((int)(bv & 0x0F) - 8) * scale;
                    sum += ar[base + bi] * lo;
                    float hi = (float)((int)((bv >> 4) & 0x0F) - 8) * scale;
                    sum += ar[base + bi + 16] * hi;
                }
            }
            out[(size_t)i * n + j] = sum;
        }
    }
}

/* backend/cpu/cpu.go:200-220 */
void vo_rmsnorm(const float *x, const float *w, float *out, int rows, int cols, float eps) {
    for (int i = 0; i < rows; i++) {
        const float *xr = x + (size_t)i * cols;
        float *o = out + (size_t)i * cols;
        float ss = 0;
        for (int j = 0; j < cols; j++) { float v = xr[j]; ss += v * v; }
        float mean = ss / (float)cols;
        float rms = (float)sqrt((double)(mean + eps));
        for (int j = 0; j < cols; j++) o[j] = (xr[j] / rms) * w[j];
    }
}

static void rope_one(float *data, int total_vectors, int heads, int head_dim, int start_pos,
                     int half, int eff_dim, float theta, const float *freqs, int neox) {
    for (int i = 0; i < total_vectors; i++) {
        int pos = start_pos + i / heads;
        float *v = data + (size_t)i * head_dim;
        for (int j = 0; j < half; j++) {
            int i0 = neox ? j : 2 * j, i1 = neox ? j + half : 2 * j + 1;
            float freq;
            if (freqs) freq = freqs[j];
            else {
                double e = (double)(2 * j) / (double)eff_dim;
                freq = (float)(1.0 / pow((double)theta, e));
            }
            float angle = (float)pos * freq;
            float c = (float)cos((double)angle), s = (float)sin((double)angle);
            float a = v[i0], b = v[i1];
            v[i0] = a * c - b * s;
            v[i1] = a * s + b * c;
        }
    }
}

/* backend/cpu/cpu.go:226-303 */
void vo_rope(float *q, float *k, int head_dim, int n_heads, int n_kv_heads, int seq_len,
             int start_pos, int rope_dim, float theta, int neox) {
    int eff = rope_dim == 0 ? head_dim : rope_dim;
    rope_one(q, seq_len * n_heads, n_heads, head_dim, start_pos, eff / 2, eff, theta, NULL, neox);
    if (k) rope_one(k, seq_len * n_kv_heads, n_kv_heads, head_dim, start_pos, eff / 2, eff, theta, NULL, neox);
}

/* backend/cpu/cpu.go:308-375 */
void vo_rope_freqs(float *q, float *k, const float *freqs, int head_dim, int n_heads,
                   int n_kv_heads, int seq_len, int start_pos, int neox) {
    rope_one(q, seq_len * n_heads, n_heads, head_dim, start_pos, head_dim / 2, head_dim, 0.f, freqs, neox);
    if (k) rope_one(k, seq_len * n_kv_heads, n_kv_heads, head_dim, start_pos, head_dim / 2, head_dim, 0.f, freqs, neox);
}

/* backend/cpu/cpu.go:378-387 */
void vo_silu(const float *x, float *out, int n) {
    for (int i = 0; i < n; i++) {
        float v = x[i];
        float sg = 1.0f / (1.0f + (float)exp((double)(-v)));
        out[i] = v * sg;
    }
}
/* backend/cpu/cpu.go:390-400 */
void vo_silu_mul(const float *g, const float *u, float *out, int n) {
    for (int i = 0; i < n; i++) {
        float v = g[i];
        float sg = 1.0f / (1.0f + (float)exp((double)(-v)));
        out[i] = (v * sg) * u[i];
    }
}
/* backend/cpu/cpu.go:440-454.  Go's untyped constants 0.7978845608 and 0.044715 become float32
 * when combined with float32 operands. */
static inline float gelu1(float v) {
    const float s2pi = 0.7978845608f, coeff = 0.044715f;
    float x3 = v * v * v;
    float ta = s2pi * (v + coeff * x3);
    float th = (float)tanh((double)ta);
    return 0.5f * v * (1.0f + th);
}
void vo_gelu(const float *x, float *out, int n) { for (int i = 0; i < n; i++) out[i] = gelu1(x[i]); }
/* backend/cpu/cpu.go:457-473 */
void vo_gelu_mul(const float *g, const float *u, float *out, int n) {
    for (int i = 0; i < n; i++) out[i] = gelu1(g[i]) * u[i];
}
/* backend/cpu/cpu.go:490-518 */
void vo_softmax(const float *x, float *out, int rows, int cols) {
    for (int i = 0; i < rows; i++) {
        const float *r = x + (size_t)i * cols; float *o = out + (size_t)i * cols;
        float mx = r[0];
        for (int j = 0; j < cols; j++) if (r[j] > mx) mx = r[j];
        float sum = 0;
        for (int j = 0; j < cols; j++) { float e = (float)exp((double)(r[j] - mx)); o[j] = e; sum += e; }
        float inv = 1.0f / sum;
        for (int j = 0; j < cols; j++) o[j] *= inv;
    }
}
void vo_add(const float *a, const float *b, float *out, int n) { for (int i = 0; i < n; i++) out[i] = a[i] + b[i]; }
void vo_mul(const float *a, const float *b, float *out, int n) { for (int i = 0; i < n; i++) out[i] = a[i] * b[i]; }
void vo_scale(float *x, float s, int n) { for (int i = 0; i < n; i++) x[i] *= s; }

/* backend/cpu/cpu.go:543-555: an id outside [0,vocab) leaves its output row untouched */
void vo_embedding(const int32_t *ids, int n_tok, const float *table, float *out, int vocab, int dim) {
    for (int i = 0; i < n_tok; i++) {
        int id = ids[i];
        if (id < 0 || id >= vocab) continue;
        memcpy(out + (size_t)i * dim, table + (size_t)id * dim, (size_t)dim * 4);
    }
}

/* Shared tail of every SDPA variant: max-subtracted softmax over scores[0..n), exp in float64
 * (cpu.go:595-612), then out = sum_pos w*v accumulated position-major (cpu.go:614-630). */
static void softmax_inplace(float *scores, int n) {
    float mx = scores[0];
    for (int i = 0; i < n; i++) if (scores[i] > mx) mx = scores[i];
    float sum = 0;
    for (int i = 0; i < n; i++) { scores[i] = (float)exp((double)(scores[i] - mx)); sum += scores[i]; }
    float inv = 1.0f / sum;
    for (int i = 0; i < n; i++) scores[i] *= inv;
}

/* backend/cpu/cpu.go:568-632 (softcap<=0) and :705-767 (softcap>0); head-major K/V */
void vo_sdpa(const float *q, const float *k, const float *v, float *out, int kv_len,
             int n_q_heads, int n_kv_heads, int head_dim, float scale, float softcap,
             int kv_head_stride) {
    int hpk = n_q_heads / n_kv_heads;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_q_heads; h++) {
        float *scores = (float *)malloc(sizeof(float) * (size_t)kv_len);
        const float *qh = q + (size_t)h * head_dim;
        float *oh = out + (size_t)h * head_dim;
        size_t base = (size_t)(h / hpk) * kv_head_stride;
        for (int pos = 0; pos < kv_len; pos++) {
            const float *kv = k + base + (size_t)pos * head_dim;
            float dot = 0;
            for (int d = 0; d < head_dim; d++) dot += qh[d] * kv[d];
            float sc = dot * scale;
            if (softcap > 0) sc = softcap * (float)tanh((double)(sc / softcap));
            scores[pos] = sc;
        }
        softmax_inplace(scores, kv_len);
        for (int d = 0; d < head_dim; d++) oh[d] = 0;
        for (int pos = 0; pos < kv_len; pos++) {
            const float *vv = v + base + (size_t)pos * head_dim;
            float w = scores[pos];
            for (int d = 0; d < head_dim; d++) oh[d] += w * vv[d];
        }
        free(scores);
    }
}

/* backend/cpu/cpu.go:635-701 and :770-838; token-major Q/K/V, causal */
void vo_sdpa_prefill(const float *q, const float *k, const float *v, float *out, int seq_len,
                     int n_q_heads, int n_kv_heads, int head_dim, float scale, float softcap) {
    int hpk = n_q_heads / n_kv_heads;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int qp = 0; qp < seq_len; qp++)
        for (int h = 0; h < n_q_heads; h++) {
            int kvh = h / hpk, n = qp + 1;
            float *scores = (float *)malloc(sizeof(float) * (size_t)n);
            const float *qh = q + ((size_t)qp * n_q_heads + h) * head_dim;
            float *oh = out + ((size_t)qp * n_q_heads + h) * head_dim;
            for (int kp = 0; kp < n; kp++) {
                const float *kv = k + ((size_t)kp * n_kv_heads + kvh) * head_dim;
                float dot = 0;
                for (int d = 0; d < head_dim; d++) dot += qh[d] * kv[d];
                float sc = dot * scale;
                if (softcap > 0) sc = softcap * (float)tanh((double)(sc / softcap));
                scores[kp] = sc;
            }
            softmax_inplace(scores, n);
            for (int d = 0; d < head_dim; d++) oh[d] = 0;
            for (int kp = 0; kp < n; kp++) {
                const float *vv = v + ((size_t)kp * n_kv_heads + kvh) * head_dim;
                float w = scores[kp];
                for (int d = 0; d < head_dim; d++) oh[d] += w * vv[d];
            }
            free(scores);
        }
}

/* pkg/sampler/sampler.go:79-90: strict '>' so the first maximum wins */
int vo_argmax(const float *x, int n) {
    float mv = -3.40282346638528859811704183484516925440e+38f; int mi = 0;
    for (int i = 0; i < n; i++) if (x[i] > mv) { mv = x[i]; mi = i; }
    return mi;
}

/* runtime/model.go:340-349 */
void vo_final_softcap(float *logits, int n, float cap) {
    if (cap <= 0) return;
    double inv = 1.0 / (double)cap;
    for (int i = 0; i < n; i++) logits[i] = (float)((double)cap * tanh((double)logits[i] * inv));
}

/* ------------------------------------------------------------------ sampler */
typedef struct { int idx; float p; } idxp;
static int cmp_f_desc(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b; return (x < y) - (x > y);
}
static int cmp_ip_desc(const void *a, const void *b) {
    const idxp *x = a, *y = b;
    if (x->p != y->p) return (x->p < y->p) - (x->p > y->p);
    return (x->idx > y->idx) - (x->idx < y->idx);   /* Go's sort is unstable; ties broken by index here */
}
/* pkg/sampler/sampler.go:49-204.  r replaces rng.Float32() (the Go math/rand stream is not restated). */
int vo_sample(const float *logits, int n, float temperature, int top_k, float top_p, float r) {
    if (temperature == 0) return vo_argmax(logits, n);
    float *p = (float *)malloc(sizeof(float) * (size_t)n);
    for (int i = 0; i < n; i++) p[i] = logits[i] / temperature;
    float mx = -3.40282346638528859811704183484516925440e+38f;
    for (int i = 0; i < n; i++) if (p[i] > mx) mx = p[i];
    float sum = 0;
    for (int i = 0; i < n; i++) { p[i] = (float)exp((double)(p[i] - mx)); sum += p[i]; }
    for (int i = 0; i < n; i++) p[i] /= sum;
    if (top_k > 0 && top_k < n) {
        float *s = (float *)malloc(sizeof(float) * (size_t)n);
        memcpy(s, p, sizeof(float) * (size_t)n);
        qsort(s, (size_t)n, sizeof(float), cmp_f_desc);
        float thr = s[top_k - 1]; free(s);
        float sm = 0;
        for (int i = 0; i < n; i++) { if (p[i] < thr) p[i] = 0; else sm += p[i]; }
        if (sm > 0) for (int i = 0; i < n; i++) p[i] /= sm;
    }
    if (top_p > 0 && top_p < 1.0f) {
        idxp *pr = (idxp *)malloc(sizeof(idxp) * (size_t)n);
        for (int i = 0; i < n; i++) { pr[i].idx = i; pr[i].p = p[i]; }
        qsort(pr, (size_t)n, sizeof(idxp), cmp_ip_desc);
        float cs = 0; int cut = n;
        for (int i = 0; i < n; i++) { cs += pr[i].p; if (cs > top_p) { cut = i + 1; break; } }
        char *keep = (char *)calloc((size_t)n, 1);
        for (int i = 0; i < cut; i++) keep[pr[i].idx] = 1;
        float sm = 0;
        for (int i = 0; i < n; i++) { if (!keep[i]) p[i] = 0; else sm += p[i]; }
        if (sm > 0) for (int i = 0; i < n; i++) p[i] /= sm;
        free(pr); free(keep);
    }
    float cs = 0; int pick = n - 1;
    for (int i = 0; i < n; i++) { cs += p[i]; if (r < cs) { pick = i; break; } }
    free(p);
    return pick;
}

/* --------------------------------------------------------- paged KV kernels */

/* backend/metal/metal_bridge_darwin.m:8539-8601 */
void vo_reshape_paged_kv_f32(const float *src, float *pool, const int32_t *blk, const int32_t *off,
                             int n_tok, int n_kv_heads, int head_dim, int block_size, int is_v) {
    size_t hs = (size_t)n_kv_heads * head_dim, part = (size_t)block_size * hs;
    for (int t = 0; t < n_tok; t++)
        for (size_t e = 0; e < hs; e++)
            pool[(size_t)blk[t] * 2 * part + (is_v ? part : 0) + (size_t)off[t] * hs + e] = src[(size_t)t * hs + e];
}
/* backend/metal/metal_bridge_darwin.m:8607-8642 */
void vo_reshape_paged_kv_f16(const float *src, uint16_t *pool, const int32_t *blk, const int32_t *off,
                             int n_tok, int n_kv_heads, int head_dim, int block_size, int is_v) {
    size_t hs = (size_t)n_kv_heads * head_dim, part = (size_t)block_size * hs;
    for (int t = 0; t < n_tok; t++)
        for (size_t e = 0; e < hs; e++)
            pool[(size_t)blk[t] * 2 * part + (is_v ? part : 0) + (size_t)off[t] * hs + e] =
                vo_f32_to_f16(src[(size_t)t * hs + e]);
}

/* Paged decode attention: the arithmetic of CPUBackend.SDPA / SDPASoftCap (cpu.go:568-632, 705-767)
 * with the block-table addressing of sdpa_paged_decode_f32/_f16
 * (backend/metal/metal_bridge_darwin.m:11074-11198, 8655-8755); GQA kvHead = qHead/(Hq/Hkv).
 * kv_start > 0 restricts to the sliding window as runtime/block.go:925-929 does. */
void vo_sdpa_paged(const float *q, const void *pool, int pool_is_f16, const int32_t *table,
                   float *out, int kv_start, int kv_len, int block_size, int n_q_heads,
                   int n_kv_heads, int head_dim, float scale, float softcap) {
    int hpk = n_q_heads / n_kv_heads, n = kv_len - kv_start;
    size_t hs = (size_t)n_kv_heads * head_dim, part = (size_t)block_size * hs;
    const float *pf = (const float *)pool; const uint16_t *ph = (const uint16_t *)pool;
#pragma omp parallel for schedule(static)
    for (int h = 0; h < n_q_heads; h++) {
        float *scores = (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
        int kvh = h / hpk;
        const float *qh = q + (size_t)h * head_dim;
        float *oh = out + (size_t)h * head_dim;
        for (int i = 0; i < n; i++) {
            int pos = kv_start + i;
            size_t base = (size_t)table[pos / block_size] * 2 * part + (size_t)(pos % block_size) * hs + (size_t)kvh * head_dim;
            float dot = 0;
            for (int d = 0; d < head_dim; d++) {
                float kv = pool_is_f16 ? vo_f16_to_f32(ph[base + d]) : pf[base + d];
                dot += qh[d] * kv;
            }
            float sc = dot * scale;
            if (softcap > 0) sc = softcap * (float)tanh((double)(sc / softcap));
            scores[i] = sc;
        }
        softmax_inplace(scores, n);
        for (int d = 0; d < head_dim; d++) oh[d] = 0;
        for (int i = 0; i < n; i++) {
            int pos = kv_start + i;
            size_t base = (size_t)table[pos / block_size] * 2 * part + part + (size_t)(pos % block_size) * hs + (size_t)kvh * head_dim;
            float w = scores[i];
            for (int d = 0; d < head_dim; d++) {
                float vv = pool_is_f16 ? vo_f16_to_f32(ph[base + d]) : pf[base + d];
                oh[d] += w * vv;
            }
        }
        free(scores);
    }
}

/* ------------------------------------------------------------- block pool */

typedef struct {
    int64_t id; int used; int seq_len;
    int32_t **tables; int *n_blocks;   /* per layer */
} vo_seq;

struct vo_pool {
    int n_layers, n_kv_heads, head_dim, block_size, max_blocks, f16;
    void **data;              /* per layer pool buffer */
    int32_t **free_list; int *n_free;   /* per layer stack, pop from the end (gpu_block_pool.go:200-208) */
    int **refcnt;
    vo_seq *seqs; int n_seqs, cap_seqs;
};

/* runtime/gpu_block_pool.go:66-126: free list initialised ascending, so the first pop is max_blocks-1 */
vo_pool *vo_pool_create(int n_layers, int n_kv_heads, int head_dim, int block_size, int max_blocks, int f16) {
    vo_pool *p = (vo_pool *)calloc(1, sizeof(*p));
    p->n_layers = n_layers; p->n_kv_heads = n_kv_heads; p->head_dim = head_dim;
    p->block_size = block_size; p->max_blocks = max_blocks; p->f16 = f16;
    size_t bytes = (size_t)max_blocks * 2 * block_size * n_kv_heads * head_dim * (f16 ? 2 : 4);
    p->data = (void **)calloc((size_t)n_layers, sizeof(void *));
    p->free_list = (int32_t **)calloc((size_t)n_layers, sizeof(int32_t *));
    p->n_free = (int *)calloc((size_t)n_layers, sizeof(int));
    p->refcnt = (int **)calloc((size_t)n_layers, sizeof(int *));
    for (int l = 0; l < n_layers; l++) {
        p->data[l] = calloc(1, bytes);
        p->free_list[l] = (int32_t *)malloc(sizeof(int32_t) * (size_t)max_blocks);
        p->refcnt[l] = (int *)calloc((size_t)max_blocks, sizeof(int));
        for (int j = 0; j < max_blocks; j++) p->free_list[l][j] = j;
        p->n_free[l] = max_blocks;
    }
    return p;
}
static void seq_free(vo_pool *p, vo_seq *s) {
    for (int l = 0; l < p->n_layers; l++) free(s->tables[l]);
    free(s->tables); free(s->n_blocks); s->used = 0;
}
void vo_pool_destroy(vo_pool *p) {
    if (!p) return;
    for (int i = 0; i < p->n_seqs; i++) if (p->seqs[i].used) seq_free(p, &p->seqs[i]);
    for (int l = 0; l < p->n_layers; l++) { free(p->data[l]); free(p->free_list[l]); free(p->refcnt[l]); }
    free(p->data); free(p->free_list); free(p->n_free); free(p->refcnt); free(p->seqs); free(p);
}
static vo_seq *find_seq(vo_pool *p, int64_t id) {
    for (int i = 0; i < p->n_seqs; i++) if (p->seqs[i].used && p->seqs[i].id == id) return &p->seqs[i];
    return NULL;
}
/* runtime/gpu_block_pool.go:129-137 (creating an existing id replaces its state without releasing blocks) */
void vo_pool_create_seq(vo_pool *p, int64_t id) {
    vo_seq *s = find_seq(p, id);
    if (s) seq_free(p, s);
    else {
        for (int i = 0; i < p->n_seqs && !s; i++) if (!p->seqs[i].used) s = &p->seqs[i];
        if (!s) {
            if (p->n_seqs == p->cap_seqs) {
                p->cap_seqs = p->cap_seqs ? p->cap_seqs * 2 : 16;
                p->seqs = (vo_seq *)realloc(p->seqs, sizeof(vo_seq) * (size_t)p->cap_seqs);
            }
            s = &p->seqs[p->n_seqs++];
        }
    }
    s->id = id; s->used = 1; s->seq_len = 0;
    s->tables = (int32_t **)calloc((size_t)p->n_layers, sizeof(int32_t *));
    s->n_blocks = (int *)calloc((size_t)p->n_layers, sizeof(int));
    for (int l = 0; l < p->n_layers; l++) s->tables[l] = (int32_t *)malloc(sizeof(int32_t) * (size_t)p->max_blocks);
}
/* runtime/gpu_block_pool.go:210-219 */
static void release_block(vo_pool *p, int layer, int32_t b) {
    int rc = p->refcnt[layer][b];
    if (rc <= 1) { p->refcnt[layer][b] = 0; p->free_list[layer][p->n_free[layer]++] = b; }
    else p->refcnt[layer][b] = rc - 1;
}
/* runtime/gpu_block_pool.go:140-160: blocks go back in table order, logical block 0 first */
void vo_pool_delete_seq(vo_pool *p, int64_t id) {
    vo_seq *s = find_seq(p, id);
    if (!s) return;
    for (int l = 0; l < p->n_layers; l++)
        for (int i = 0; i < s->n_blocks[l]; i++) release_block(p, l, s->tables[l][i]);
    seq_free(p, s);
}
/* runtime/gpu_block_pool.go:165-190 */
void vo_pool_truncate(vo_pool *p, int64_t id, int new_len) {
    vo_seq *s = find_seq(p, id);
    if (!s || new_len >= s->seq_len) return;
    int nb = new_len > 0 ? (new_len - 1) / p->block_size + 1 : 0;
    for (int l = 0; l < p->n_layers; l++) {
        for (int i = nb; i < s->n_blocks[l]; i++) release_block(p, l, s->tables[l][i]);
        if (nb < s->n_blocks[l]) s->n_blocks[l] = nb;
    }
    s->seq_len = new_len;
}
/* runtime/gpu_block_pool.go:572-607 */
int vo_pool_share(vo_pool *p, int64_t src, int64_t dst, int n_tokens) {
    vo_seq *a = find_seq(p, src), *b = find_seq(p, dst);
    if (!a || !b) return -1;
    int nb = (n_tokens + p->block_size - 1) / p->block_size;
    for (int l = 0; l < p->n_layers; l++) {
        if (nb > a->n_blocks[l]) return -2;
        for (int i = 0; i < nb; i++) {
            int32_t id = a->tables[l][i];
            b->tables[l][b->n_blocks[l]++] = id;
            p->refcnt[l][id]++;
        }
    }
    if (n_tokens > b->seq_len) b->seq_len = n_tokens;
    return 0;
}
/* runtime/gpu_block_pool.go:223-323 */
int vo_pool_store_kv(vo_pool *p, int layer, int64_t id, int start_pos, const float *k,
                     const float *v, int n_tok) {
    vo_seq *s = find_seq(p, id);
    if (!s) return -1;
    int end = start_pos + n_tok, last = (end - 1) / p->block_size;
    while (s->n_blocks[layer] <= last) {
        if (p->n_free[layer] == 0) return -2;
        int32_t b = p->free_list[layer][--p->n_free[layer]];
        p->refcnt[layer][b] = 1;
        s->tables[layer][s->n_blocks[layer]++] = b;
    }
    for (int i = 0; k && v && i < n_tok; i++) {   /* k == NULL: allocate the blocks only (test set-up copies whole pages in) */
        int pos = start_pos + i;
        int32_t blk = s->tables[layer][pos / p->block_size], off = pos % p->block_size;
        size_t hs = (size_t)p->n_kv_heads * p->head_dim;
        if (p->f16) {
            vo_reshape_paged_kv_f16(k + i * hs, (uint16_t *)p->data[layer], &blk, &off, 1, p->n_kv_heads, p->head_dim, p->block_size, 0);
            vo_reshape_paged_kv_f16(v + i * hs, (uint16_t *)p->data[layer], &blk, &off, 1, p->n_kv_heads, p->head_dim, p->block_size, 1);
        } else {
            vo_reshape_paged_kv_f32(k + i * hs, (float *)p->data[layer], &blk, &off, 1, p->n_kv_heads, p->head_dim, p->block_size, 0);
            vo_reshape_paged_kv_f32(v + i * hs, (float *)p->data[layer], &blk, &off, 1, p->n_kv_heads, p->head_dim, p->block_size, 1);
        }
    }
    if (end > s->seq_len) s->seq_len = end;
    return 0;
}
int vo_pool_seq_len(vo_pool *p, int64_t id) { vo_seq *s = find_seq(p, id); return s ? s->seq_len : -1; }
int vo_pool_table(vo_pool *p, int layer, int64_t id, int32_t *out, int cap) {
    vo_seq *s = find_seq(p, id);
    if (!s) return -1;
    int n = s->n_blocks[layer];
    for (int i = 0; i < n && i < cap; i++) out[i] = s->tables[layer][i];
    return n;
}
int vo_pool_free_blocks(vo_pool *p, int layer) { return p->n_free[layer]; }
/* Test set-up: replace every layer's free stack (bottom first) while no sequence holds a block.  The reference starts from
 * the ascending list (gpu_block_pool.go:114-116); a serving pool that has run for a while hands out blocks in whatever
 * order they came back, and tests reproduce such an order on both sides with this. */
int vo_pool_set_free_list(vo_pool *p, const int32_t *ids, int n) {
    if (n != p->max_blocks) return -1;
    for (int l = 0; l < p->n_layers; l++) {
        if (p->n_free[l] != p->max_blocks) return -2;
        memcpy(p->free_list[l], ids, sizeof(int32_t) * (size_t)n);
    }
    return 0;
}
void *vo_pool_layer_data(vo_pool *p, int layer) { return p->data[layer]; }

/* runtime/gpu_block_pool.go:337-389 (kv_len<=0 -> seq_len), attention math as vo_sdpa_paged */
int vo_pool_attention(vo_pool *p, int layer, int64_t id, const float *q, float *out,
                      int n_q_heads, float scale, float softcap, int window, int kv_len) {
    vo_seq *s = find_seq(p, id);
    if (!s || s->n_blocks[layer] == 0) return -1;
    int eff = kv_len > 0 ? kv_len : s->seq_len;
    int start = 0;
    if (window > 0 && eff - 1 >= window) start = eff - 1 - window + 1;   /* runtime/block.go:925-929 */
    vo_sdpa_paged(q, p->data[layer], p->f16, s->tables[layer], out, start, eff, p->block_size,
                  n_q_heads, p->n_kv_heads, p->head_dim, scale, softcap);
    return 0;
}

/* ------------------------------------------------------------------ model */

typedef struct { int type; void *raw; float *f32; } vo_tensor;

struct vo_model {
    vo_config c;
    vo_tensor *layer_t;      /* [n_layers][VO_T_PER_LAYER] */
    vo_tensor glob[3];
    vo_pool *pool;
};

vo_model *vo_model_create(const vo_config *cfg) {
    vo_model *m = (vo_model *)calloc(1, sizeof(*m));
    m->c = *cfg;
    m->layer_t = (vo_tensor *)calloc((size_t)cfg->n_layers * VO_T_PER_LAYER, sizeof(vo_tensor));
    m->pool = vo_pool_create(cfg->n_layers, cfg->n_kv_heads, cfg->head_dim, 16, cfg->max_blocks, cfg->kv_f16);
    return m;
}
static void tensor_free(vo_tensor *t) { free(t->raw); free(t->f32); t->raw = NULL; t->f32 = NULL; }
void vo_model_destroy(vo_model *m) {
    if (!m) return;
    for (int i = 0; i < m->c.n_layers * VO_T_PER_LAYER; i++) tensor_free(&m->layer_t[i]);
    for (int i = 0; i < 3; i++) tensor_free(&m->glob[i]);
    vo_pool_destroy(m->pool); free(m->layer_t); free(m);
}
vo_pool *vo_model_pool(vo_model *m) { return m->pool; }

static void slot_dims(const vo_config *c, int slot, int64_t *n, int64_t *k) {
    int qd = c->n_heads * c->head_dim, kvd = c->n_kv_heads * c->head_dim;
    switch (slot) {
    case VO_T_WQ: *n = qd; *k = c->hidden; break;
    case VO_T_WK: case VO_T_WV: *n = kvd; *k = c->hidden; break;
    case VO_T_WO: *n = c->hidden; *k = qd; break;
    case VO_T_W1: case VO_T_W3: *n = c->ffn; *k = c->hidden; break;
    case VO_T_W2: *n = c->hidden; *k = c->ffn; break;
    default: *n = 1; *k = c->hidden; break;   /* norm vectors */
    }
}
/* runtime/loader.go:81-212: projection matrices stay raw when Q4_0 (fused matmul available on CPU);
 * anything else quantized is dequantized to F32 (the reference's LoadWeightsF32 route, loader.go:214-271,
 * because CPUBackend.MatMulQ4_K/Q6_K panic, cpu.go:916-928). */
static int set_tensor(vo_tensor *t, int type, const void *data, int64_t n, int64_t k, int keep_q4_0_raw) {
    tensor_free(t);
    t->type = type;
    size_t bytes = vo_type_row_bytes(type, k) * (size_t)n;
    if (bytes == 0) return -1;
    if (type == VO_Q4_0 && keep_q4_0_raw) {
        t->raw = malloc(bytes); memcpy(t->raw, data, bytes);
    } else {
        t->f32 = (float *)malloc(sizeof(float) * (size_t)(n * k));
        vo_dequant(type, (const uint8_t *)data, n * k, t->f32);
    }
    return 0;
}
int vo_model_set_layer_tensor(vo_model *m, int layer, int slot, int type, const void *data) {
    int64_t n, k; slot_dims(&m->c, slot, &n, &k);
    return set_tensor(&m->layer_t[layer * VO_T_PER_LAYER + slot], type, data, n, k, 1);
}
/* runtime/loader.go:275-288: embedding always F32; a Q4_0 output head is dequantized to F32 */
int vo_model_set_global_tensor(vo_model *m, int which, int type, const void *data) {
    int64_t n = which == VO_G_FINAL_NORM ? 1 : m->c.vocab;
    return set_tensor(&m->glob[which], type, data, n, m->c.hidden, 0);
}

/* runtime/block.go:506-552 */
static void proj(const vo_tensor *w, const float *a, float *out, int m, int n, int k) {
    if (w->raw) vo_matmul_q4_0(a, (const uint8_t *)w->raw, out, m, n, k);
    else vo_matmul_transposed(a, w->f32, out, m, n, k);
}

/* runtime/block.go:464-476 */
static int layer_slides(const vo_config *c, int layer) {
    if (c->sliding_window <= 0) return 0;
    return c->window_alternating ? (layer % 2 == 1) : 1;
}

/* One pass of runtime/decode.go:339-461 (n_tok==1), :961-1096 (prefill) or :1446-1569 (verify), with the
 * layer body of runtime/block.go:763-1081 on the device-pool branch (:866-895). */
int vo_model_forward(vo_model *m, int64_t seq, const int32_t *tokens, int n_tok, int start_pos,
                     int all_logits, float *logits, float *hidden) {
    const vo_config *c = &m->c;
    int H = c->hidden, Hq = c->n_heads, Hkv = c->n_kv_heads, D = c->head_dim, F = c->ffn, T = n_tok;
    int qd = Hq * D, kvd = Hkv * D;
    if (vo_pool_seq_len(m->pool, seq) < 0) vo_pool_create_seq(m->pool, seq);   /* decode.go:362-364 */
    float *x = (float *)calloc((size_t)T * H, 4), *nrm = (float *)malloc((size_t)T * H * 4);
    float *q = (float *)malloc((size_t)T * qd * 4), *k = (float *)malloc((size_t)T * kvd * 4);
    float *v = (float *)malloc((size_t)T * kvd * 4), *att = (float *)malloc((size_t)T * qd * 4);
    float *gate = (float *)malloc((size_t)T * F * 4), *up = (float *)malloc((size_t)T * F * 4);
    int rc = 0;
    vo_embedding(tokens, T, m->glob[VO_G_EMBED].f32, x, c->vocab, H);          /* decode.go:405-407 */
    if (c->embed_scale != 0) vo_scale(x, c->embed_scale, T * H);               /* decode.go:408 */
    if (hidden) memcpy(hidden, x, (size_t)T * H * 4);
    float scale = (float)(1.0 / sqrt((double)D));                              /* block.go:862 */
    for (int l = 0; l < c->n_layers && rc == 0; l++) {
        vo_tensor *t = &m->layer_t[l * VO_T_PER_LAYER];
        vo_rmsnorm(x, t[VO_T_ATTN_NORM].f32, nrm, T, H, c->rms_eps);           /* block.go:836 */
        proj(&t[VO_T_WQ], nrm, q, T, qd, H);                                   /* block.go:841-854 */
        proj(&t[VO_T_WK], nrm, k, T, kvd, H);
        proj(&t[VO_T_WV], nrm, v, T, kvd, H);
        vo_rope(q, k, D, Hq, Hkv, T, start_pos, 0, c->rope_theta, c->rope_neox); /* block.go:858 */
        rc = vo_pool_store_kv(m->pool, l, seq, start_pos, k, v, T);            /* block.go:868, 878 */
        if (rc) break;
        int window = layer_slides(c, l) ? c->sliding_window : 0;
        if (T == 1) {
            vo_pool_attention(m->pool, l, seq, q, att, Hq, scale, c->attn_softcap, window, 0);   /* block.go:872 */
        } else if (start_pos > 0) {
            for (int i = 0; i < T; i++)                                        /* block.go:881-890, kvLens[i]=startPos+i+1 */
                vo_pool_attention(m->pool, l, seq, q + (size_t)i * qd, att + (size_t)i * qd, Hq, scale,
                                  c->attn_softcap, window, start_pos + i + 1);
        } else {
            vo_sdpa_prefill(q, k, v, att, T, Hq, Hkv, D, scale, c->attn_softcap);   /* block.go:891-895 */
        }
        proj(&t[VO_T_WO], att, nrm, T, H, qd);                                 /* block.go:983 */
        if (c->post_norms) vo_rmsnorm(nrm, t[VO_T_POST_ATTN_NORM].f32, nrm, T, H, c->rms_eps);   /* :985-987 */
        vo_add(x, nrm, x, T * H);                                              /* :990 */
        vo_rmsnorm(x, t[VO_T_FFN_NORM].f32, nrm, T, H, c->rms_eps);            /* :997 */
        proj(&t[VO_T_W1], nrm, gate, T, F, H);                                 /* :1045-1049 */
        proj(&t[VO_T_W3], nrm, up, T, F, H);
        if (c->geglu) vo_gelu_mul(gate, up, gate, T * F);                      /* :1051-1057 */
        else vo_silu_mul(gate, up, gate, T * F);
        proj(&t[VO_T_W2], gate, nrm, T, H, F);                                 /* :1060 */
        if (c->post_norms) vo_rmsnorm(nrm, t[VO_T_POST_FFN_NORM].f32, nrm, T, H, c->rms_eps);    /* :1067-1070 */
        vo_add(x, nrm, x, T * H);                                              /* :1077 */
        if (hidden) memcpy(hidden + (size_t)(l + 1) * T * H, x, (size_t)T * H * 4);
    }
    if (rc == 0 && logits) {
        if (T == 1 || all_logits) {
            vo_rmsnorm(x, m->glob[VO_G_FINAL_NORM].f32, x, T, H, c->rms_eps);  /* decode.go:442 */
            vo_matmul_transposed(x, m->glob[VO_G_OUTPUT].f32, logits, T, c->vocab, H);   /* model.go:421 */
        } else {                                                               /* decode.go:1057-1086: last token only */
            float *last = x + (size_t)(T - 1) * H;
            vo_rmsnorm(last, m->glob[VO_G_FINAL_NORM].f32, last, 1, H, c->rms_eps);
            vo_matmul_transposed(last, m->glob[VO_G_OUTPUT].f32, logits, 1, c->vocab, H);
        }
    }
    free(x); free(nrm); free(q); free(k); free(v); free(att); free(gate); free(up);
    return rc;
}
