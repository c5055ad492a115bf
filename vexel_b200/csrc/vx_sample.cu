// Temperature / top-k / top-p sampling on the device, one CTA per logits row.
//
// Follows pkg/sampler/sampler.go:49-204: scaled = logit / T; softmax (exp evaluated in f64, cast to f32);
// top-k keeps everything >= the k-th largest probability (ties at the threshold survive) and renormalises;
// top-p keeps the shortest prefix of the descending order whose running sum exceeds p and renormalises;
// the token is the first index whose running sum exceeds the uniform draw r, else the last index.
// The caller supplies r (the reference draws it from math/rand on the host), so a given (logits, r) pair
// maps to one token.  The reference sorts; here the k-th value and the top-p cut are found by a three-pass
// radix select over the f32 bit pattern (probabilities are non-negative, so the patterns order like the values),
// which visits each row a constant number of times and needs no O(V log V) work.
//
// The reference accumulates its normalisation sums and the sampling CDF sequentially in float32, in index
// order.  Those running sums decide which token a draw maps to (a vocabulary-wide CDF has boundaries only
// ~1e-5 apart), so they are reproduced bit for bit: one thread adds the row in index order (adding a zeroed
// entry is exact, so filtered rows cost only the scan).  The one place where float64 stands in for the
// reference's float32 arithmetic is the top-p cut, whose running sum over the *sorted* probabilities is
// evaluated from per-bin float64 sums: a cut whose running sum lands within float32 rounding of p may keep
// one entry more or less than the reference would.
#include "vx_common.cuh"

namespace {

constexpr int ST = 1024;                 // threads per row
constexpr int NW = ST / 32;
constexpr int NB = 2048;                 // bins per radix pass: 11 + 11 + 10 bits

struct SampleRow { float temperature; int32_t top_k; float top_p; float u; };

__device__ __forceinline__ int pass_bin(uint32_t b, int pass) { return pass == 0 ? (int)(b >> 21) : pass == 1 ? (int)((b >> 10) & 2047u) : (int)(b & 1023u); }
__device__ __forceinline__ uint32_t pass_mask(int pass) { return pass == 0 ? 0u : pass == 1 ? 0xFFE00000u : 0xFFFFFC00u; }
__device__ __forceinline__ int pass_shift(int pass) { return pass == 0 ? 21 : pass == 1 ? 10 : 0; }

struct Smem {
    double hsum[NB];
    unsigned hcnt[NB];
    double wtmp[NW + 1];
    double red[NW];
    unsigned long long chosen;           // (bin << 32) | valid
    double above_sum; unsigned above_cnt;
    unsigned eq_cnt; unsigned prefix;
    int keep_all; int pick;
    float fsum;
};

__device__ __forceinline__ float block_max(float v, Smem &s) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if (lane == 0) s.red[w] = (double)v;
    __syncthreads();
    float t = (float)s.red[0];
#pragma unroll
    for (int i = 1; i < NW; i++) t = fmaxf(t, (float)s.red[i]);
    return t;
}

// sum of p[0..n) accumulated left to right in float32, as `sum += probs[i]` does (sampler.go:106-109, 131-137, 188-195)
__device__ float seq_sum_f32(const float *p, int n) {
    float s = 0.f; int i = 0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0)
        for (; i + 8 <= n; i += 8) {
            float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
            s += a.x; s += a.y; s += a.z; s += a.w; s += b.x; s += b.y; s += b.z; s += b.w;
        }
    for (; i < n; i++) s += p[i];
    return s;
}

__device__ __forceinline__ float seq_sum_bcast(const float *p, int n, Smem &s) {
    __syncthreads();
    if (threadIdx.x == 0) s.fsum = seq_sum_f32(p, n);
    __syncthreads();
    return s.fsum;
}

// first index whose float32 running sum exceeds r, else n - 1 (sampler.go:206-218)
__device__ int seq_pick_f32(const float *p, int n, float r) {
    float cs = 0.f; int i = 0;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0)
        for (; i + 8 <= n; i += 8) {
            float4 a = *reinterpret_cast<const float4 *>(p + i), b = *reinterpret_cast<const float4 *>(p + i + 4);
            float c0 = cs + a.x, c1 = c0 + a.y, c2 = c1 + a.z, c3 = c2 + a.w, c4 = c3 + b.x, c5 = c4 + b.y, c6 = c5 + b.z, c7 = c6 + b.w;
            if (r < c7) {                          // the running sum never decreases, so the first crossing is in this group
                if (r < c0) return i;     if (r < c1) return i + 1; if (r < c2) return i + 2; if (r < c3) return i + 3;
                if (r < c4) return i + 4; if (r < c5) return i + 5; if (r < c6) return i + 6; return i + 7;
            }
            cs = c7;
        }
    for (; i < n; i++) { cs += p[i]; if (r < cs) return i; }
    return n - 1;
}

// exclusive scan over the block of a (sum, count) pair; every thread also learns the totals
__device__ __forceinline__ void block_excl_scan2(double v, unsigned c, Smem &s, double *ev, unsigned *ec) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    double iv = v; unsigned ic = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        double tv = __shfl_up_sync(0xffffffffu, iv, o); unsigned tc = __shfl_up_sync(0xffffffffu, ic, o);
        if (lane >= o) { iv += tv; ic += tc; }
    }
    __shared__ double wv[NW]; __shared__ unsigned wc[NW];
    __syncthreads();
    if (lane == 31) { wv[w] = iv; wc[w] = ic; }
    __syncthreads();
    double bv = 0; unsigned bc = 0;
    for (int i = 0; i < w; i++) { bv += wv[i]; bc += wc[i]; }
    *ev = bv + iv - v; *ec = bc + ic - c;
}

// One radix pass.  by_sum = false: find the bin holding the element of descending rank `target_cnt`
// (1-based, counted among elements that match the prefix, after `above_cnt` larger ones).  by_sum = true:
// find the bin in which above_sum + running sum first exceeds `p`.
__device__ void radix_pass(const float *pr, int n, int pass, bool by_sum, unsigned target_cnt, double p, Smem &s) {
    for (int i = threadIdx.x; i < NB; i += ST) { s.hsum[i] = 0.0; s.hcnt[i] = 0u; }
    if (threadIdx.x == 0) s.chosen = 0ull;
    __syncthreads();
    const uint32_t mask = pass_mask(pass), prefix = s.prefix;
    for (int i = threadIdx.x; i < n; i += ST) {
        float v = pr[i]; uint32_t b = __float_as_uint(v);
        if ((b & mask) == prefix) {
            int bin = pass_bin(b, pass);
            atomicAdd(&s.hcnt[bin], 1u);
            if (by_sum) atomicAdd(&s.hsum[bin], (double)v);
        }
    }
    __syncthreads();
    // descending order: thread t owns bins NB-1-2t and NB-2-2t
    const int b0 = NB - 1 - 2 * (int)threadIdx.x, b1 = b0 - 1;
    double s0 = s.hsum[b0], s1 = s.hsum[b1]; unsigned c0 = s.hcnt[b0], c1 = s.hcnt[b1];
    double ev; unsigned ec;
    block_excl_scan2(s0 + s1, c0 + c1, s, &ev, &ec);
    const double as = s.above_sum; const unsigned ac = s.above_cnt;
    int pick = -1; double add_s = 0; unsigned add_c = 0;
    if (!by_sum) {
        unsigned lo = ac + ec;
        if (lo < target_cnt && target_cnt <= lo + c0) { pick = b0; add_c = ec; add_s = ev; }
        else if (lo + c0 < target_cnt && target_cnt <= lo + c0 + c1) { pick = b1; add_c = ec + c0; add_s = ev + s0; }
    } else {
        double lo = as + ev;
        if (c0 && lo <= p && lo + s0 > p) { pick = b0; add_c = ec; add_s = ev; }
        else if (c1 && lo + s0 <= p && lo + s0 + s1 > p) { pick = b1; add_c = ec + c0; add_s = ev + s0; }
    }
    __syncthreads();
    if (pick >= 0) {
        // at most one thread gets here for a count target; for a sum target f64 rounding keeps it to one as well
        unsigned long long rec = ((unsigned long long)(unsigned)pick << 32) | 1ull;
        if (atomicCAS(&s.chosen, 0ull, rec) == 0ull) {
            s.above_sum = as + add_s; s.above_cnt = ac + add_c;
            s.eq_cnt = (pick == b0) ? c0 : c1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!(s.chosen & 1ull)) {
            if (pass == 0) s.keep_all = 1;           // the running sum never exceeds p: everything stays
            else {
                // rounding between passes hid the crossing: it is in the lowest occupied bin of this range
                int b = 0; while (b < NB - 1 && s.hcnt[b] == 0u) b++;
                double sa = 0; unsigned ca = 0;
                for (int j = NB - 1; j > b; j--) { sa += s.hsum[j]; ca += s.hcnt[j]; }
                s.above_sum = as + sa; s.above_cnt = ac + ca; s.eq_cnt = s.hcnt[b];
                s.chosen = ((unsigned long long)(unsigned)b << 32) | 1ull;
            }
        }
        if (s.chosen & 1ull) s.prefix = prefix | ((uint32_t)(s.chosen >> 32) << pass_shift(pass));
    }
    __syncthreads();
}

// zeroes everything below the threshold pattern `thr`; of the `eq_cnt` entries equal to it keeps the first
// `keep_eq` in index order; renormalises by the kept sum (sampler.go:131-143, 186-200)
__device__ void apply_threshold(float *pr, int n, uint32_t thr, unsigned eq_cnt, unsigned keep_eq, Smem &s) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int seg = ((n + NW - 1) / NW + 31) & ~31;
    const int lo = min(n, w * seg), hi = min(n, lo + seg);
    unsigned base = 0;
    if (keep_eq < eq_cnt) {
        unsigned cnt = 0;
        for (int i = lo + lane; i < hi; i += 32) cnt += (__float_as_uint(pr[i]) == thr);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
        __syncthreads();
        if (lane == 0) s.hcnt[w] = cnt;
        __syncthreads();
        for (int i = 0; i < w; i++) base += s.hcnt[i];
        __syncthreads();
    }
    for (int i0 = lo; i0 < hi; i0 += 32) {
        int i = i0 + lane;
        float v = i < hi ? pr[i] : 0.f;
        uint32_t b = __float_as_uint(v);
        bool tie = (i < hi) && b == thr;
        bool keep = (i < hi) && b > thr;
        if (keep_eq < eq_cnt) {
            unsigned bal = __ballot_sync(0xffffffffu, tie);
            unsigned rank = base + __popc(bal & ((1u << lane) - 1u));
            keep = keep || (tie && rank < keep_eq);
            base += __popc(bal);
        } else keep = keep || tie;
        if (i < hi && !keep) pr[i] = 0.f;
    }
    const float sm = seq_sum_bcast(pr, n, s);
    if (sm > 0.f) for (int i = threadIdx.x; i < n; i += ST) pr[i] = pr[i] / sm;
    __syncthreads();
}

__global__ void __launch_bounds__(ST) sample_rows_kernel(float *logits, long ld, int n, const SampleRow *rows, float final_softcap,
                                                         int32_t *out) {
    __shared__ Smem s;
    const SampleRow R = rows[blockIdx.x];
    if (R.temperature == 0.f) return;                                   // greedy rows keep their argmax (sampler.go:51-53)
    float *pr = logits + (size_t)blockIdx.x * ld;

    // scaled logits and their maximum (sampler.go:56-59, 95-100)
    float mx = -3.40282346638528859811704183484516925440e+38f;
    const double cap = (double)final_softcap, inv_cap = final_softcap > 0.f ? 1.0 / cap : 0.0;
    for (int i = threadIdx.x; i < n; i += ST) {
        float v = pr[i];
        if (final_softcap > 0.f) v = (float)(cap * tanh((double)v * inv_cap));      // runtime/model.go:340-349
        v = v / R.temperature;
        pr[i] = v; mx = fmaxf(mx, v);
    }
    mx = block_max(mx, s);
    for (int i = threadIdx.x; i < n; i += ST) pr[i] = (float)exp((double)(pr[i] - mx));
    const float sum = seq_sum_bcast(pr, n, s);
    for (int i = threadIdx.x; i < n; i += ST) pr[i] = pr[i] / sum;
    __syncthreads();

    if (R.top_k > 0 && R.top_k < n) {                                   // sampler.go:119-144
        if (threadIdx.x == 0) { s.prefix = 0u; s.above_sum = 0.0; s.above_cnt = 0u; s.keep_all = 0; }
        __syncthreads();
        for (int pass = 0; pass < 3; pass++) radix_pass(pr, n, pass, false, (unsigned)R.top_k, 0.0, s);
        const uint32_t thr = s.prefix; const unsigned eq = s.eq_cnt;
        __syncthreads();
        apply_threshold(pr, n, thr, eq, eq, s);                          // every tie at the threshold stays
    }
    if (R.top_p > 0.f && R.top_p < 1.0f) {                              // sampler.go:147-202
        if (threadIdx.x == 0) { s.prefix = 0u; s.above_sum = 0.0; s.above_cnt = 0u; s.keep_all = 0; }
        __syncthreads();
        const double p = (double)R.top_p;
        for (int pass = 0; pass < 3; pass++) { radix_pass(pr, n, pass, true, 0u, p, s); if (s.keep_all) break; }
        if (!s.keep_all) {
            const uint32_t thr = s.prefix; const unsigned eq = s.eq_cnt; const double gt = s.above_sum;
            const double v = (double)__uint_as_float(thr);
            long j = v > 0.0 ? (long)floor((p - gt) / v) + 1 : (long)eq;
            if (j < 1) j = 1; if (j > (long)eq) j = (long)eq;
            while (j > 1 && gt + (double)(j - 1) * v > p) j--;
            while (j < (long)eq && gt + (double)j * v <= p) j++;
            __syncthreads();
            apply_threshold(pr, n, thr, eq, (unsigned)j, s);
        }
        __syncthreads();
    }

    // inverse CDF in index order with the reference's float32 running sum (sampler.go:206-218)
    if (threadIdx.x == 0) out[blockIdx.x] = seq_pick_f32(pr, n, R.u);
}

}  // namespace

int vxe_argmax_rows(vx_ctx *c, const float *x, int rows, int cols, int32_t *out);

// launcher used by the model's step: params on the device, tokens written where the argmax already is
int vxs_sample_rows(vx_ctx *c, float *logits, long ld, int rows, int n, const void *d_params, float final_softcap, int32_t *d_out) {
    VX_REQUIRE(c, rows > 0 && n > 0 && ld >= n, "sample: bad shape");
    sample_rows_kernel<<<rows, ST, 0, c->stream>>>(logits, ld, n, (const SampleRow *)d_params, final_softcap, d_out);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

extern "C" {

// Sampler.Sample (pkg/sampler/sampler.go:49-76) for `rows` logits rows at once; overwrites the rows with their
// probabilities.  Rows with temperature 0 return the first index of the maximum (sampler.go:79-90).
int vx_sample_rows(vx_ctx *c, vx_dptr logits, int rows, int n, const vx_sample_params *params, int32_t *out_tokens) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, logits && params && out_tokens && rows > 0 && n > 0, "vx_sample_rows: bad arguments");
    static_assert(sizeof(vx_sample_params) == sizeof(SampleRow), "parameter record layout");
    vx_dptr d_par = 0, d_out = 0;
    VX_TRY(vx_alloc(c, sizeof(SampleRow) * (size_t)rows, &d_par));
    VX_TRY(vx_alloc(c, sizeof(int32_t) * (size_t)rows, &d_out));
    VX_CUDA(c, cudaMemcpyAsync((void *)d_par, params, sizeof(SampleRow) * (size_t)rows, cudaMemcpyHostToDevice, c->stream));
    VX_TRY(vxe_argmax_rows(c, (const float *)logits, rows, n, (int32_t *)d_out));
    VX_TRY(vxs_sample_rows(c, (float *)logits, n, rows, n, (const void *)d_par, 0.f, (int32_t *)d_out));
    VX_CUDA(c, cudaMemcpyAsync(out_tokens, (const void *)d_out, sizeof(int32_t) * (size_t)rows, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    VX_TRY(vx_check_device_error(c));
    vx_free(c, d_par); vx_free(c, d_out);
    return VX_OK;
}

}  // extern "C"
