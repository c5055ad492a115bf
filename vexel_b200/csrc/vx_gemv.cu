// Thin-batch Q4_0 (and, further down, Q4_K) projection (1 to 4 activation rows): y[m][n] = sum_k x[m][k] * d[n][k/32] * (q[n][k] - 8).
//
// The reference runs its decode projections as one quantised mat-vec per sequence (MatMulQ4_0 with M = 1,
// inference/runtime/block.go:947-1060, kernels metal_bridge_darwin.m matvec_q4_0*).  With a handful of rows the product is
// a stream over the weights, and what limits it is the number of instructions spent per weight byte, so this kernel keeps
// that number low:
//   * a warp owns 16 weight rows; lane (g, c) fetches the 16-byte slot c of rows g and g + 8 of every 128-weight group (the
//     repacked layout of vx_quant.cu) -- exactly the nibbles of its own mma.sync A fragments, so no ldmatrix and no CTA
//     barrier; the copies go through a per-warp cp.async ring, seven groups ahead;
//   * a nibble becomes an fp16 integer with one logic operation and one subtraction (0x6400 | q = 1024 + q); the high
//     nibbles are taken in place, (1024 + 16 q) / 16 - 72 in one exact FMA, so nothing is shifted into position;
//   * the rows keep their fp16 hi and lo parts side by side in the eight columns of one m16n8k16 tile, so that the
//     float32-faithful product costs one MMA per 16 weights (with five or more rows a second tile is needed, and the staged
//     kernel of vx_quant.cu measured faster: 3.81 against 4.43 ms per step at eight rows);
//   * the block scale is applied to the four accumulators of a 32-weight block in float32, as the reference does.
// Activations are read as B fragments straight from the split arrays (the 0,2,1,3 order they are stored in is the fragment
// order).
#include <cuda_fp16.h>

#include "vx_common.cuh"

namespace {

constexpr int GV_WARPS = 4;                 // 64 weight rows per CTA
constexpr int GV_THREADS = GV_WARPS * 32;
constexpr int GV_CTAS_PER_SM = 6;            // bounded by the ring (36 KB per CTA)
constexpr int GV_STAGES = 8;                // 128-weight groups in flight per warp
constexpr int GV_STAGE_BYTES = 1024 + 128;  // 16 rows x 64 bytes of nibbles + 16 rows x 4 scales

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same with a zero addend: starts the sum of a 32-weight block without clearing four registers first
__device__ __forceinline__ void mma16816_first(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// two low nibbles of v (bits 0-3 and 16-19) -> half2 {q0 - 8, q1 - 8}
__device__ __forceinline__ uint32_t lo_nib(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;                                                 // 1024 + q
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6408)));   // - 1032
    return *reinterpret_cast<uint32_t *>(&r);
}
// two high nibbles of v (bits 4-7 and 20-23), taken in place -> half2 {q0 - 8, q1 - 8}: (1024 + 16 q) / 16 - 72, one exact FMA
__device__ __forceinline__ uint32_t hi_nib(uint32_t v) {
    uint32_t h = (v & 0x00F000F0u) | 0x64006400u;
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x2C00)),    // 1/16
                        __half2half2(__ushort_as_half((unsigned short)0xD480)));                                      // -72
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t word_of(const uint4 &v, int b) { return b == 0 ? v.x : b == 1 ? v.y : b == 2 ? v.z : v.w; }

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void *smem, const void *gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// Rows 0-3: hi parts in columns 0-3 and lo parts in columns 4-7 of the tile.
// Weights: every lane copies its own two 16-byte slots of a group (rows g and g + 8) into a ring of GV_STAGES groups per warp
// with cp.async, so that the bytes in flight are not bounded by registers; lanes c = 0, 1 of a quad also copy the block scales
// of rows g, g + 8.  A lane reads back only what its own warp copied: one wait_group and one __syncwarp per group, no CTA
// barrier.  Activations: lane (g, c) reads its B fragments -- row g, columns 32 b + 4 c .. + 3 and the four 16 further on,
// stored in the order 0,2,1,3 -- straight from the split arrays (a few KB per row: they stay in L1).  Columns of the tile that
// stand for no row read the last row instead; what they produce is never stored.
__global__ void __launch_bounds__(GV_THREADS, GV_CTAS_PER_SM)
gemv_q4_0_kernel(const uint4 *__restrict__ qs, const __half *__restrict__ sc, const __half *__restrict__ xh, const __half *__restrict__ xl,
                 const float *__restrict__ xscale, float *__restrict__ out, int M, int N, int k_groups, int groups_per_split, int x_ld,
                 int ld_out, size_t part_stride) {
    // per warp and stage: [32 lanes] slot of row g, [32 lanes] slot of row g + 8, [16 rows] four block scales
    __shared__ __align__(16) unsigned char ring[GV_WARPS][GV_STAGES][GV_STAGE_BYTES];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int r0 = blockIdx.x * (GV_WARPS * 16) + warp * 16;
    const int j_begin = blockIdx.y * groups_per_split;
    const int n_j = min(groups_per_split, k_groups - j_begin);
    // rows past the end of the matrix are read as its last row and never stored
    const int row_a = min(r0 + g, N - 1), row_b = min(r0 + g + 8, N - 1);
    const uint4 *qa = qs + ((size_t)row_a * k_groups + j_begin) * 4 + c;
    const uint4 *qb = qs + ((size_t)row_b * k_groups + j_begin) * 4 + c;
    // lane c = 0 fetches the scales of row g, lane c = 1 those of row g + 8
    const __half *sp = sc + ((size_t)(c == 0 ? row_a : row_b) * k_groups + j_begin) * 4;
    const int xrow = min(g & 3, M - 1);
    const __half *x0 = (g >= 4 ? xl : xh) + (size_t)xrow * x_ld + (size_t)j_begin * 128 + 4 * c;
    unsigned char *my = &ring[warp][0][0];

    auto request = [&](int j) {                              // group j of the slice into stage j % GV_STAGES (an empty group past the end)
        if (j < n_j) {
            unsigned char *st = my + (j % GV_STAGES) * GV_STAGE_BYTES;
            cp_async16(st + lane * 16, qa + (size_t)j * 4);
            cp_async16(st + 512 + lane * 16, qb + (size_t)j * 4);
            if (c < 2) cp_async8(st + 1024 + (g + 8 * c) * 8, sp + (size_t)j * 4);
        }
        cp_async_commit();
    };
    // weights do not depend on the kernel ahead of this one: the ring is filled before waiting for it
#pragma unroll
    for (int j = 0; j < GV_STAGES - 1; j++) request(j);
    vx_pdl_wait();
    vx_pdl_trigger();                                        // (chained launch) the row kernel behind this one may be set up now

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < n_j; j++) {
        cp_async_wait<GV_STAGES - 2>();                      // group j has landed (this lane's copies) ...
        __syncwarp();                                        // ... and every other lane's; stage (j - 1) % GV_STAGES has been read by all
        request(j + GV_STAGES - 1);
        const unsigned char *st = my + (j % GV_STAGES) * GV_STAGE_BYTES;
        const uint4 wa = *reinterpret_cast<const uint4 *>(st + lane * 16), wb = *reinterpret_cast<const uint4 *>(st + 512 + lane * 16);
        const uint2 da = *reinterpret_cast<const uint2 *>(st + 1024 + g * 8), db = *reinterpret_cast<const uint2 *>(st + 1024 + (g + 8) * 8);
        const __half2 dA01 = *reinterpret_cast<const __half2 *>(&da.x), dA23 = *reinterpret_cast<const __half2 *>(&da.y);
        const __half2 dB01 = *reinterpret_cast<const __half2 *>(&db.x), dB23 = *reinterpret_cast<const __half2 *>(&db.y);
        const float sA[4] = {__low2float(dA01), __high2float(dA01), __low2float(dA23), __high2float(dA23)};
        const float sB[4] = {__low2float(dB01), __high2float(dB01), __low2float(dB23), __high2float(dB23)};
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const uint32_t va = word_of(wa, b), vb = word_of(wb, b);
            const uint32_t va8 = va >> 8, vb8 = vb >> 8;
            const uint32_t l0 = lo_nib(va), l1 = lo_nib(vb), l2 = lo_nib(va8), l3 = lo_nib(vb8);   // weights 4c .. 4c+3 of the block
            const uint32_t h0 = hi_nib(va), h1 = hi_nib(vb), h2 = hi_nib(va8), h3 = hi_nib(vb8);   // weights 16 + 4c .. + 3
            const uint2 xa = __ldg(reinterpret_cast<const uint2 *>(x0 + 32 * b)), xb = __ldg(reinterpret_cast<const uint2 *>(x0 + 32 * b + 16));
            float s[4];
            mma16816_first(s, l0, l1, l2, l3, xa.x, xa.y);
            mma16816(s, h0, h1, h2, h3, xb.x, xb.y);
            acc[0] = fmaf(sA[b], s[0], acc[0]); acc[1] = fmaf(sA[b], s[1], acc[1]);
            acc[2] = fmaf(sB[b], s[2], acc[2]); acc[3] = fmaf(sB[b], s[3], acc[3]);
        }
        x0 += 128;
    }
    cp_async_wait<0>();
    // column n (hi part) lives in the lane with c = n / 2, column n + 4 (lo part) in the lane with c + 2
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 2);
    if (c >= 2) return;
    float *o = out + (size_t)blockIdx.y * part_stride;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int m = 2 * c + e;
        if (m < M) {
            const float s = xscale[m];
            if (r0 + g < N) o[(size_t)m * ld_out + r0 + g] = acc[e] * s;
            if (r0 + g + 8 < N) o[(size_t)m * ld_out + r0 + g + 8] = acc[2 + e] * s;
        }
    }
}

// ---- the same design for Q4_K (inference/pkg/gguf/dequant.go:342-396): w = fl(d sc_u) q - fl(dmin m_u) per 32-weight sub-block u.
// The repacked group of a row holds word c of the halves (64-weight group jj, 16-byte half t) = (0,0), (0,1), (1,0), (1,1);
// the low nibbles of a 64-weight group are sub-block 2 jj, the high nibbles sub-block 2 jj + 1, and half t is one K = 16 step.
// q stays unsigned here: the minimum term meets the activations' block sums (one float4 per batch row and group) in the hi
// columns of the tile.  A ring stage carries the nibbles, the scale / minimum bytes and {d, dmin} of 16 rows.
constexpr int GVK_STAGE_BYTES = 1024 + 128 + 64;
// two low nibbles of v -> half2 {q0, q1};  two high nibbles in place -> half2 {q0, q1}: (1024 + 16 q) / 16 - 64
__device__ __forceinline__ uint32_t lo_nibu(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x6400)));
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ uint32_t hi_nibu(uint32_t v) {
    uint32_t h = (v & 0x00F000F0u) | 0x64006400u;
    __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&h), __half2half2(__ushort_as_half((unsigned short)0x2C00)),    // 1/16
                        __half2half2(__ushort_as_half((unsigned short)0xD400)));                                      // -64
    return *reinterpret_cast<uint32_t *>(&r);
}
__device__ __forceinline__ void cp_async4(void *smem, const void *gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}

__global__ void __launch_bounds__(GV_THREADS, 5)
gemv_q4_k_kernel(const uint4 *__restrict__ qs, const uint2 *__restrict__ sc, const __half2 *__restrict__ sup, const __half *__restrict__ xh,
                 const __half *__restrict__ xl, const float *__restrict__ xscale, const float *__restrict__ xbsum, int bsum_ld,
                 float *__restrict__ out, int M, int N, int k_groups, int groups_per_split, int x_ld, int ld_out, size_t part_stride) {
    __shared__ __align__(16) unsigned char ring[GV_WARPS][GV_STAGES][GVK_STAGE_BYTES];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int r0 = blockIdx.x * (GV_WARPS * 16) + warp * 16;
    const int j_begin = blockIdx.y * groups_per_split;
    const int n_j = min(groups_per_split, k_groups - j_begin);
    const int row_a = min(r0 + g, N - 1), row_b = min(r0 + g + 8, N - 1);
    const uint4 *qa = qs + ((size_t)row_a * k_groups + j_begin) * 4 + c;
    const uint4 *qb = qs + ((size_t)row_b * k_groups + j_begin) * 4 + c;
    // lanes c = 0 / 1 fetch the scale bytes of rows g / g + 8, lanes c = 2 / 3 their {d, dmin}
    const int my_row = (c & 1) ? row_b : row_a;
    const uint2 *sp = sc + (size_t)my_row * k_groups + j_begin;
    const __half2 *dp2 = sup + (size_t)my_row * (k_groups >> 1);
    const int xrow = min(g & 3, M - 1);
    const __half *x0 = (g >= 4 ? xl : xh) + (size_t)xrow * x_ld + (size_t)j_begin * 128 + 4 * c;
    // block sums of the two batch rows whose hi columns this lane holds (lanes c >= 2 hold lo columns: no minimum term)
    const float *bs0 = xbsum + (size_t)min(2 * (c & 1), M - 1) * bsum_ld + (size_t)j_begin * 4;
    const float *bs1 = xbsum + (size_t)min(2 * (c & 1) + 1, M - 1) * bsum_ld + (size_t)j_begin * 4;
    const float hi_col = c < 2 ? 1.f : 0.f;
    unsigned char *my = &ring[warp][0][0];

    auto request = [&](int j) {
        if (j < n_j) {
            unsigned char *st = my + (j % GV_STAGES) * GVK_STAGE_BYTES;
            cp_async16(st + lane * 16, qa + (size_t)j * 4);
            cp_async16(st + 512 + lane * 16, qb + (size_t)j * 4);
            if (c < 2) cp_async8(st + 1024 + (g + 8 * c) * 8, sp + j);
            else cp_async4(st + 1152 + (g + 8 * (c - 2)) * 4, dp2 + ((j_begin + j) >> 1));
        }
        cp_async_commit();
    };
#pragma unroll
    for (int j = 0; j < GV_STAGES - 1; j++) request(j);
    vx_pdl_wait();
    vx_pdl_trigger();

    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < n_j; j++) {
        cp_async_wait<GV_STAGES - 2>();
        __syncwarp();
        request(j + GV_STAGES - 1);
        const unsigned char *st = my + (j % GV_STAGES) * GVK_STAGE_BYTES;
        const uint4 wa = *reinterpret_cast<const uint4 *>(st + lane * 16), wb = *reinterpret_cast<const uint4 *>(st + 512 + lane * 16);
        const uint2 ma = *reinterpret_cast<const uint2 *>(st + 1024 + g * 8), mb = *reinterpret_cast<const uint2 *>(st + 1024 + (g + 8) * 8);
        const float2 da = __half22float2(*reinterpret_cast<const __half2 *>(st + 1152 + g * 4));
        const float2 db = __half22float2(*reinterpret_cast<const __half2 *>(st + 1152 + (g + 8) * 4));
        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(bs0 + 4 * j)), b1 = __ldg(reinterpret_cast<const float4 *>(bs1 + 4 * j));
        const float bv0[4] = {b0.x, b0.y, b0.z, b0.w}, bv1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int u = 0; u < 4; u++) {                          // sub-block u = 2 jj + nib
            const int jj = u >> 1, nib = u & 1;
            const uint32_t a0w = word_of(wa, 2 * jj), a1w = word_of(wa, 2 * jj + 1), b0w = word_of(wb, 2 * jj), b1w = word_of(wb, 2 * jj + 1);
            const uint2 xa = __ldg(reinterpret_cast<const uint2 *>(x0 + 32 * u)), xb = __ldg(reinterpret_cast<const uint2 *>(x0 + 32 * u + 16));
            float s[4];
            if (nib == 0) {
                mma16816_first(s, lo_nibu(a0w), lo_nibu(b0w), lo_nibu(a0w >> 8), lo_nibu(b0w >> 8), xa.x, xa.y);
                mma16816(s, lo_nibu(a1w), lo_nibu(b1w), lo_nibu(a1w >> 8), lo_nibu(b1w >> 8), xb.x, xb.y);
            } else {
                mma16816_first(s, hi_nibu(a0w), hi_nibu(b0w), hi_nibu(a0w >> 8), hi_nibu(b0w >> 8), xa.x, xa.y);
                mma16816(s, hi_nibu(a1w), hi_nibu(b1w), hi_nibu(a1w >> 8), hi_nibu(b1w >> 8), xb.x, xb.y);
            }
            const float d1a = __fmul_rn(da.x, (float)((ma.x >> (8 * u)) & 0xFF)), m1a = __fmul_rn(da.y, (float)((ma.y >> (8 * u)) & 0xFF)) * hi_col;
            const float d1b = __fmul_rn(db.x, (float)((mb.x >> (8 * u)) & 0xFF)), m1b = __fmul_rn(db.y, (float)((mb.y >> (8 * u)) & 0xFF)) * hi_col;
            acc[0] = fmaf(d1a, s[0], fmaf(-m1a, bv0[u], acc[0])); acc[1] = fmaf(d1a, s[1], fmaf(-m1a, bv1[u], acc[1]));
            acc[2] = fmaf(d1b, s[2], fmaf(-m1b, bv0[u], acc[2])); acc[3] = fmaf(d1b, s[3], fmaf(-m1b, bv1[u], acc[3]));
        }
        x0 += 128;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < 4; i++) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 2);
    if (c >= 2) return;
    float *o = out + (size_t)blockIdx.y * part_stride;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int m = 2 * c + e;
        if (m < M) {
            const float s = xscale[m];
            if (r0 + g < N) o[(size_t)m * ld_out + r0 + g] = acc[e] * s;
            if (r0 + g + 8 < N) o[(size_t)m * ld_out + r0 + g + 8] = acc[2 + e] * s;
        }
    }
}

int g_gemv = 1;

}  // namespace

// Q4_0 up to four rows; Q4_K up to three (Llama-3-8B-shaped step: 4.14 -> 3.80 ms at one row, 4.18 -> 4.07 at three, no gain at four)
bool vxq_gemv_eligible(const VxWeight &w, int m) { return g_gemv && m >= 1 && ((w.type == VX_T_Q4_0 && m <= 4) || (w.type == VX_T_Q4_K && m <= 3)); }

// out receives [m][ld_out] when *n_parts_out == 1, otherwise `parts` holds [n_parts][m][w.n]
int vxq_gemv(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
             size_t parts_cap_floats) {
    const int k_groups = w.k_pad / 128;
    const int ctas = ceil_div(w.n, GV_WARPS * 16);
    // split K so that the CTAs fill whole waves of the GPU (six resident CTAs per SM): the split with the best wave
    // efficiency wins, fewer partials on ties
    int split = 1;
    if (parts) {
        const long slots = (long)GV_CTAS_PER_SM * c->sm_count;
        double best = 0.0;
        for (int s = 1; s <= 16 && s <= max(1, k_groups / 2); s++) {
            if ((size_t)s * m * w.n > parts_cap_floats) break;
            const int gps = ceil_div(k_groups, s), s_eff = ceil_div(k_groups, gps);
            const long n_cta = (long)ctas * s_eff;
            const double eff = (double)n_cta / (double)(ceil_div64(n_cta, slots) * slots) * ((double)k_groups / (double)(gps * s_eff));
            if (eff > best + 0.03) { best = eff; split = s_eff; }
        }
    }
    const int gps = ceil_div(k_groups, split);
    split = ceil_div(k_groups, gps);
    float *dst = split > 1 ? parts : out;
    const int ld = split > 1 ? w.n : ld_out;
    const size_t pstride = (size_t)m * w.n;
    *n_parts_out = split;
    dim3 grid(ctas, split);
    // the rings of all resident CTAs need most of the SM's shared memory
    static VxPerDevice carveout;
    cudaError_t le = carveout.once(c, [&]() {
        return cudaFuncSetAttribute(gemv_q4_0_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    });
    if (le != cudaSuccess) return vx_cuda_fail(c, le, "thin-batch projection attributes");
    if (w.type == VX_T_Q4_K) {
        static VxPerDevice carveout_k;
        le = carveout_k.once(c, [&]() {
            return cudaFuncSetAttribute(gemv_q4_k_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        });
        if (le != cudaSuccess) return vx_cuda_fail(c, le, "thin-batch projection attributes");
        le = vx_launch_dependent(gemv_q4_k_kernel, grid, dim3(GV_THREADS), 0, c->stream, (const uint4 *)w.qs, (const uint2 *)w.sc, (const __half2 *)w.aux,
                                 (const __half *)x.hi, (const __half *)x.lo, (const float *)x.scale, (const float *)x.bsum, x.k_pad / 32, dst, m, w.n,
                                 k_groups, gps, x.k_pad, ld, pstride);
    } else
    le = vx_launch_dependent(gemv_q4_0_kernel, grid, dim3(GV_THREADS), 0, c->stream, (const uint4 *)w.qs, (const __half *)w.sc, (const __half *)x.hi,
                             (const __half *)x.lo, (const float *)x.scale, dst, m, w.n, k_groups, gps, x.k_pad, ld, pstride);
    if (le != cudaSuccess) return vx_cuda_fail(c, le, "thin-batch projection launch");
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

extern "C" int vx_set_thin_batch_projections(int enable) { g_gemv = enable != 0; return VX_OK; }
