// GGUF block formats on the device: bit-exact dequantisation (inference/pkg/gguf/dequant.go), the
// repacked weight layout, activation splitting and the dequant-fused tensor-core projection kernel
// behind QuantizedMatMul (inference/backend/backend.go:47-81).
//
// Projection arithmetic.  The reference computes sum_k x[k] * (d_b * float32(q_k - 8)) in float32
// (inference/backend/cpu/cpu.go:842-911).  Here, per 32-weight block b,
//     y += d_b * ( sum_{k in b} (q_k - 8) * x_hi[k]  +  sum_{k in b} (q_k - 8) * x_lo[k] )
// where x = s * (x_hi + x_lo) is an exact-to-2^-22 split of the float32 activation into two fp16
// numbers (s a per-row power of two).  (q-8) is exact in fp16, the products are exact in the
// tensor core's float32 accumulator, and d_b is applied in float32 outside the MMA, so the only
// rounding is float32 accumulation, as in the reference.
#include "vx_common.cuh"

// ------------------------------------------------------------------ dequantisation (bit-exact)
__global__ void dequant_q4_0_kernel(const uint8_t *__restrict__ raw, float *__restrict__ out, int64_t n) {
    int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;   // one thread per packed byte
    int64_t nb = (n + 31) / 32;
    if (idx >= nb * 16) return;
    int64_t b = idx >> 4; int i = (int)(idx & 15);
    const uint8_t *blk = raw + b * 18;
    float scale = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    uint8_t bv = blk[2 + i];
    int64_t e0 = b * 32 + i, e1 = e0 + 16;
    if (e0 < n) out[e0] = __fmul_rn(scale, (float)((int)(bv & 0x0F) - 8));       // dequant.go:43
    if (e1 < n) out[e1] = __fmul_rn(scale, (float)((int)(bv >> 4) - 8));         // dequant.go:50
}

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, uint8_t &sc, uint8_t &mn) {   // dequant.go:400-409
    if (j < 4) { sc = q[j] & 63; mn = q[j + 4] & 63; }
    else { sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4); mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

__global__ void dequant_q4_k_kernel(const uint8_t *__restrict__ raw, float *__restrict__ out, int64_t n) {
    int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;   // one thread per qs byte (128 per block)
    int64_t nb = (n + 255) / 256;
    if (idx >= nb * 128) return;
    int64_t b = idx >> 7; int t = (int)(idx & 127);
    int grp = t >> 5, l = t & 31;                                   // 64-element group, byte within it
    const uint8_t *blk = raw + b * 144;
    float d = __half2float(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))));
    float dmin = __half2float(__ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
    uint8_t s1, m1, s2, m2;
    scale_min_k4(2 * grp, blk + 4, s1, m1);
    scale_min_k4(2 * grp + 1, blk + 4, s2, m2);
    float d1 = __fmul_rn(d, (float)s1), dm1 = __fmul_rn(dmin, (float)m1);
    float d2 = __fmul_rn(d, (float)s2), dm2 = __fmul_rn(dmin, (float)m2);
    uint8_t q = blk[16 + grp * 32 + l];
    int64_t i1 = b * 256 + grp * 64 + l, i2 = i1 + 32;
    if (i1 < n) out[i1] = __fsub_rn(__fmul_rn(d1, (float)(q & 0x0F)), dm1);      // dequant.go:383
    if (i2 < n) out[i2] = __fsub_rn(__fmul_rn(d2, (float)(q >> 4)), dm2);        // dequant.go:386
}

__global__ void dequant_q6_k_kernel(const uint8_t *__restrict__ raw, float *__restrict__ out, int64_t n) {
    int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;   // one thread per (half, l): 64 per block
    int64_t nb = (n + 255) / 256;
    if (idx >= nb * 64) return;
    int64_t b = idx >> 6; int t = (int)(idx & 63);
    int hf = t >> 5, l = t & 31, is = l / 16;
    const uint8_t *ql = raw + b * 210 + hf * 64, *qh = raw + b * 210 + 128 + hf * 32;
    const int8_t *sc = (const int8_t *)(raw + b * 210 + 192) + hf * 8;
    const uint8_t *dp2 = raw + b * 210 + 208;
    float d = __half2float(__ushort_as_half((unsigned short)(dp2[0] | (dp2[1] << 8))));
    int q1 = (int)(int8_t)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
    int q2 = (int)(int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
    int q3 = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
    int q4 = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
    int64_t y = b * 256 + hf * 128 + l;
    if (y < n)      out[y]      = __fmul_rn(__fmul_rn(d, (float)sc[is + 0]), (float)q1);   // dequant.go:313
    if (y + 32 < n) out[y + 32] = __fmul_rn(__fmul_rn(d, (float)sc[is + 2]), (float)q2);
    if (y + 64 < n) out[y + 64] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4]), (float)q3);
    if (y + 96 < n) out[y + 96] = __fmul_rn(__fmul_rn(d, (float)sc[is + 6]), (float)q4);
}

__global__ void f16_to_f32_kernel(const __half *__restrict__ in, float *__restrict__ out, int64_t n) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < n) out[i] = __half2float(in[i]);
}

static int dequant_launch(vx_ctx *c, int type, const void *raw, float *out, int64_t n) {
    if (n <= 0) return VX_OK;
    switch (type) {
    case VX_T_F32: VX_CUDA(c, cudaMemcpyAsync(out, raw, (size_t)n * 4, cudaMemcpyDeviceToDevice, c->stream)); return VX_OK;
    case VX_T_F16: f16_to_f32_kernel<<<(unsigned)ceil_div64(n, 256), 256, 0, c->stream>>>((const __half *)raw, out, n); break;
    case VX_T_Q4_0: dequant_q4_0_kernel<<<(unsigned)ceil_div64(ceil_div64(n, 32) * 16, 256), 256, 0, c->stream>>>((const uint8_t *)raw, out, n); break;
    case VX_T_Q4_K: dequant_q4_k_kernel<<<(unsigned)ceil_div64(ceil_div64(n, 256) * 128, 256), 256, 0, c->stream>>>((const uint8_t *)raw, out, n); break;
    case VX_T_Q6_K: dequant_q6_k_kernel<<<(unsigned)ceil_div64(ceil_div64(n, 256) * 64, 256), 256, 0, c->stream>>>((const uint8_t *)raw, out, n); break;
    default: return vx_fail(c, VX_E_UNSUPPORTED, "dequantize: unsupported GGUF type %d", type);
    }
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// ------------------------------------------------------------------ repacked Q4_0 layout
// For row r and group j of four 32-weight blocks (128 weights), 64 bytes are stored as
//   uint4 slot[c], c = 0..3, slot[c] = { word c of block 4j, word c of 4j+1, word c of 4j+2, word c of 4j+3 }
// where word c of a block is its raw nibble bytes [4c, 4c+4) as a little-endian u32.  A fixed byte
// permutation of the GGUF data: dequantising from it gives the same bits.  Scales go to a separate
// half array [n][k_pad/32]; blocks that pad k to a multiple of 128 have scale 0.
__global__ void repack_q4_0_kernel(const uint8_t *__restrict__ raw, uint4 *__restrict__ qs, __half *__restrict__ sc,
                                   int n, int k_blocks, int k_groups) {
    long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;   // (row, group, c)
    long total = (long)n * k_groups * 4;
    if (idx >= total) return;
    int c = (int)(idx & 3); long rg = idx >> 2;
    int j = (int)(rg % k_groups); long r = rg / k_groups;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int blk = 4 * j + i;
        if (blk < k_blocks) {
            const uint8_t *p = raw + ((size_t)r * k_blocks + blk) * 18;
            w[i] = (uint32_t)p[2 + 4 * c] | ((uint32_t)p[3 + 4 * c] << 8) | ((uint32_t)p[4 + 4 * c] << 16) | ((uint32_t)p[5 + 4 * c] << 24);
            if (c == 0) sc[(size_t)r * k_groups * 4 + blk] = __ushort_as_half((unsigned short)(p[0] | (p[1] << 8)));
        } else {
            w[i] = 0x88888888u;
            if (c == 0) sc[(size_t)r * k_groups * 4 + blk] = __ushort_as_half((unsigned short)0);
        }
    }
    qs[idx] = make_uint4(w[0], w[1], w[2], w[3]);
}

// ------------------------------------------------------------------ repacked K-quant layouts
// Q4_K (144 B / 256 weights).  Per row and 128-weight group G (half a super-block): uint4 slot[c] holding the nibble
// words (64-group jj, 16-byte half t') = (0,0),(0,1),(1,0),(1,1), word c of each; the low nibbles of a 64-group are
// sub-block 2j, the high nibbles sub-block 2j+1 (dequant.go:366-392).  sc: 8 bytes per group {sc[4], min[4]} in the
// order u = 2jj + nib, unpacked from the 6-bit fields (dequant.go:400-409).  aux: half2 {d, dmin} per super-block.
__global__ void repack_q4_k_kernel(const uint8_t *__restrict__ raw, uint4 *__restrict__ qs, uint2 *__restrict__ sc,
                                   __half2 *__restrict__ aux, int n, int k_groups) {
    long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (idx >= (long)n * k_groups * 4) return;
    int c = (int)(idx & 3); long rg = idx >> 2;
    int G = (int)(rg % k_groups); long r = rg / k_groups;
    const uint8_t *blk = raw + ((size_t)r * (k_groups / 2) + G / 2) * 144;
    const int hf = G & 1;
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint8_t *p = blk + 16 + 32 * (2 * hf + (i >> 1)) + 16 * (i & 1) + 4 * c;
        w[i] = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    }
    qs[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    if (c == 0) {
        uint32_t s4 = 0, m4 = 0;
        for (int u = 0; u < 4; u++) {
            uint8_t a, b2;
            scale_min_k4(4 * hf + u, blk + 4, a, b2);
            s4 |= (uint32_t)a << (8 * u); m4 |= (uint32_t)b2 << (8 * u);
        }
        sc[(size_t)r * k_groups + G] = make_uint2(s4, m4);
        if (hf == 0) aux[(size_t)r * (k_groups / 2) + G / 2] =
            __halves2half2(__ushort_as_half((unsigned short)(blk[0] | (blk[1] << 8))), __ushort_as_half((unsigned short)(blk[2] | (blk[3] << 8))));
    }
}
// Q6_K (210 B / 256 weights).  Per row and 128-weight half G: element e = 16u + p (sub-block u, position p); lane c owns
// p in {4c..4c+3}.  lo: uint4, word i byte b = low nibble: low 4 bits of element (u=2i, p=4c+b), high nibble: (u=2i+1, p=4c+b).
// hi: uint2, byte u bits [2b+1:2b] = top 2 bits of element (u, 4c+b).  sc: the 8 int8 scales of the half.  aux: half d.
__global__ void repack_q6_k_kernel(const uint8_t *__restrict__ raw, uint4 *__restrict__ lo, uint2 *__restrict__ hi, uint2 *__restrict__ sc,
                                   __half *__restrict__ aux, int n, int k_groups) {
    long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (idx >= (long)n * k_groups * 4) return;
    int c = (int)(idx & 3); long rg = idx >> 2;
    int G = (int)(rg % k_groups); long r = rg / k_groups;
    const uint8_t *blk = raw + ((size_t)r * (k_groups / 2) + G / 2) * 210;
    const int hf = G & 1;
    const uint8_t *ql = blk + 64 * hf, *qh = blk + 128 + 32 * hf;
    auto q6 = [&](int e) -> uint32_t {            // 0..63, dequant.go:300-308
        int l = e & 31, qd = e >> 5;
        uint32_t lo4 = (qd & 1) ? ql[l + 32] : ql[l];
        lo4 = (qd & 2) ? (lo4 >> 4) : (lo4 & 0xF);
        uint32_t hi2 = (qh[l] >> (2 * qd)) & 3;
        return lo4 | (hi2 << 4);
    };
    uint32_t wl[4] = {0, 0, 0, 0}; uint32_t wh[2] = {0, 0};
    for (int u = 0; u < 8; u++)
        for (int b2 = 0; b2 < 4; b2++) {
            uint32_t v = q6(16 * u + 4 * c + b2);
            wl[u >> 1] |= (v & 0xF) << (8 * b2 + 4 * (u & 1));
            wh[u >> 2] |= (v >> 4) << (8 * (u & 3) + 2 * b2);
        }
    lo[idx] = make_uint4(wl[0], wl[1], wl[2], wl[3]);
    hi[idx] = make_uint2(wh[0], wh[1]);
    if (c == 0) {
        const uint8_t *s8 = blk + 192 + 8 * hf;
        sc[(size_t)r * k_groups + G] = make_uint2((uint32_t)s8[0] | ((uint32_t)s8[1] << 8) | ((uint32_t)s8[2] << 16) | ((uint32_t)s8[3] << 24),
                                                  (uint32_t)s8[4] | ((uint32_t)s8[5] << 8) | ((uint32_t)s8[6] << 16) | ((uint32_t)s8[7] << 24));
        if (hf == 0) aux[(size_t)r * (k_groups / 2) + G / 2] = __ushort_as_half((unsigned short)(blk[208] | (blk[209] << 8)));
    }
}

// byte offsets of the four arrays of a repacked [n][k] matrix; every array is row-major by weight row
bool vxq_layout(int type, int n, int k, VxRepackLayout *L) {
    const size_t kg = (size_t)ceil_div(k, 128);
    size_t rb[4] = {0, 0, 0, 0};
    switch (type) {
    case VX_T_Q4_0: rb[0] = kg * 64; rb[1] = kg * 8; break;
    case VX_T_Q4_K: rb[0] = kg * 64; rb[1] = kg * 8; rb[2] = kg / 2 * 4; break;
    case VX_T_Q6_K: rb[0] = kg * 64; rb[1] = kg * 8; rb[2] = kg / 2 * 2; rb[3] = kg * 32; break;
    default: return false;
    }
    size_t off = 0;
    for (int i = 0; i < 4; i++) { L->row_bytes[i] = rb[i]; L->off[i] = off; off += (rb[i] * n + 255) & ~(size_t)255; }
    L->total = off;
    return true;
}

// repacks n_rows raw GGUF rows into rows [row0, row0 + n_rows) of a layout computed for the whole (concatenated) matrix
int vxq_repack_rows(vx_ctx *c, int type, const void *raw_dev, int n_rows, int k, void *base, const VxRepackLayout &L, int row0) {
    const int blk = type == VX_T_Q4_0 ? 32 : 256;
    if (k % blk != 0) return vx_fail(c, VX_E_BAD_ARG, "repack: k=%d is not a multiple of the %d-weight block", k, blk);
    const int k_groups = ceil_div(k, 128);
    char *b0 = (char *)base;
    void *p[4];
    for (int i = 0; i < 4; i++) p[i] = b0 + L.off[i] + L.row_bytes[i] * (size_t)row0;
    long total = (long)n_rows * k_groups * 4;
    unsigned grid = (unsigned)((total + 255) / 256);
    switch (type) {
    case VX_T_Q4_0: repack_q4_0_kernel<<<grid, 256, 0, c->stream>>>((const uint8_t *)raw_dev, (uint4 *)p[0], (__half *)p[1], n_rows, k / 32, k_groups); break;
    case VX_T_Q4_K: repack_q4_k_kernel<<<grid, 256, 0, c->stream>>>((const uint8_t *)raw_dev, (uint4 *)p[0], (uint2 *)p[1], (__half2 *)p[2], n_rows, k_groups); break;
    case VX_T_Q6_K: repack_q6_k_kernel<<<grid, 256, 0, c->stream>>>((const uint8_t *)raw_dev, (uint4 *)p[0], (uint2 *)p[3], (uint2 *)p[1], (__half *)p[2], n_rows, k_groups); break;
    default: return vx_fail(c, VX_E_UNSUPPORTED, "repack: GGUF type %d has no MMA layout", type);
    }
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

void vxq_weight_view(int type, int n, int k, void *base, const VxRepackLayout &L, VxWeight *w) {
    char *b0 = (char *)base;
    w->type = type; w->n = n; w->k = k; w->k_pad = ceil_div(k, 128) * 128;
    w->qs = b0 + L.off[0]; w->sc = b0 + L.off[1]; w->aux = b0 + L.off[2]; w->hi = b0 + L.off[3];
    const double bpw = type == VX_T_Q4_0 ? 18.0 / 32 : type == VX_T_Q4_K ? 144.0 / 256 : 210.0 / 256;
    w->bytes = (size_t)((double)n * k * bpw);
}

// ------------------------------------------------------------------ activation split
size_t vxq_split_bytes(int rows, int k, size_t *hi_off, size_t *lo_off, size_t *scale_off, size_t *bsum_off, int *k_pad) {
    int kp = ceil_div(k, 128) * 128;
    size_t rp = (size_t)((rows + 63) / 64) * 64;
    size_t off = 0;
    *hi_off = off; off += rp * kp * sizeof(__half);
    *lo_off = off; off += rp * kp * sizeof(__half);
    *scale_off = off; off += ((rp * sizeof(float)) + 255) & ~(size_t)255;
    *bsum_off = off; off += ((rp * (kp / 32) * sizeof(float)) + 255) & ~(size_t)255;
    *k_pad = kp;
    return off;
}

// One CTA of 1024 threads per row; the row lives in registers (NC chunks of 4096 columns).
template <int NC>
__global__ void __launch_bounds__(VX_ROW_THREADS) split_rows_kernel(const float *__restrict__ x, int cols, int ld, VxSplit s) {
    __shared__ float red[32];
    vx_pdl_wait();
    vx_pdl_trigger();          // the projection that follows may become resident and fetch its first weights now
    const int row = blockIdx.x;
    const float *xr = x + (size_t)row * ld;
    float4 v[NC];
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
        v[c] = k0 < cols ? *reinterpret_cast<const float4 *>(xr + k0) : make_float4(0.f, 0.f, 0.f, 0.f);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[c].x), fabsf(v[c].y)), fmaxf(fabsf(v[c].z), fabsf(v[c].w))));
    }
    amax = block_max(amax, red);
    float sc, inv;
    vx_row_scale(amax, sc, inv);
    if (threadIdx.x == 0) s.scale[row] = sc;
    __half *hi = s.hi + (size_t)row * s.k_pad, *lo = s.lo + (size_t)row * s.k_pad;
    float *bs = s.bsum + (size_t)row * (s.k_pad / 32);
#pragma unroll
    for (int c = 0; c < NC; c++) {
        int k0 = (c * VX_ROW_THREADS + threadIdx.x) * 4;
        if (k0 < s.k_pad) {
            const float t[4] = {v[c].x * inv, v[c].y * inv, v[c].z * inv, v[c].w * inv};
            vx_split_store4(t, hi, lo, bs, k0);
        }
    }
}

int vxq_split_rows(vx_ctx *c, const float *x, int rows, int cols, int ld, const VxSplit &s) {
    if (rows <= 0) return VX_OK;
    if (cols % 4 != 0 || ld % 4 != 0) return vx_fail(c, VX_E_BAD_ARG, "activation rows must be multiples of 4 columns");
    int nc = ceil_div(s.k_pad, VX_ROW_THREADS * 4);
    switch (nc) {
#define VX_SPLIT_CASE(N) case N: split_rows_kernel<N><<<rows, VX_ROW_THREADS, 0, c->stream>>>(x, cols, ld, s); break;
        VX_SPLIT_CASE(1) VX_SPLIT_CASE(2) VX_SPLIT_CASE(3) VX_SPLIT_CASE(4) VX_SPLIT_CASE(5) VX_SPLIT_CASE(6) VX_SPLIT_CASE(7) VX_SPLIT_CASE(8)
#undef VX_SPLIT_CASE
    default: return vx_fail(c, VX_E_UNSUPPORTED, "activation rows of %d columns are not supported (max 32768)", cols);
    }
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// ------------------------------------------------------------------ the projection kernel
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(gmem));
}
__device__ __forceinline__ void cp_async8(void *smem, const void *gmem) {
    uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(sa), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// two packed nibbles (bits 0-3 and 16-19 of v) -> half2 {q0 - 8, q1 - 8}, exact
__device__ __forceinline__ uint32_t nib2_to_half2(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;          // 1024 + q in each half
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1032.f, 1032.f));
    return *reinterpret_cast<uint32_t *>(&r);
}

constexpr int GEMM_ROWS = 128;      // weight rows per CTA (8 warps x 16)
constexpr int GEMM_XLD = 144;       // smem row stride in halfs: 128 + 16 keeps 8-byte fragment loads conflict-free
// Depth of the cp.async ring (activation tile + the warps' weight words of one 128-weight group per stage).  Thin batches are
// bound by how many weight bytes a CTA keeps in flight, so they get the deepest ring that still leaves three CTAs per SM.
#ifndef VX_RING_MIN_NT
#define VX_RING_MIN_NT 2
#endif
constexpr bool gemm_ring(int nt) { return nt >= VX_RING_MIN_NT; }      // 8-row tiles keep the next group's weights in registers instead
constexpr int gemm_stages(int fmt, int nt) { return !gemm_ring(nt) ? 3 : nt == 1 ? (fmt == 2 ? 4 : 5) : nt == 2 ? 4 : nt == 4 ? (fmt == 2 ? 3 : 4) : 3; }
constexpr int GEMM_W_BYTES = 8 * 64 * 16;     // per stage: 8 warps x (rows g and g + 8) x 32 lanes x 16 bytes of nibbles
constexpr int GEMM_SC_BYTES = 8 * 16 * 8;     // 8 warps x 16 rows x 8 bytes of block / sub-block scales
constexpr int gemm_h_bytes(int fmt) { return fmt == 2 ? 8 * 64 * 8 : 0; }   // Q6_K: the top two bits, 8 bytes per lane and row
constexpr int gemm_stage_bytes(int fmt, int nt, int terms) {
    return terms * 8 * nt * GEMM_XLD * 2 + (fmt == 1 ? 8 * nt * 16 : 0) + (gemm_ring(nt) ? GEMM_W_BYTES + GEMM_SC_BYTES + gemm_h_bytes(fmt) : 0);
}

// 6-bit variant of nib2_to_half2: v carries the low nibbles (bits 0-3, 16-19), h6 the top two bits already at bits 4-5 and
// 20-21 -> half2 {q0 - 32, q1 - 32}, exact
__device__ __forceinline__ uint32_t q6_to_half2(uint32_t v, uint32_t h6) {
    uint32_t h = (v & 0x000F000Fu) | h6 | 0x64006400u;      // 1024 + q
    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1056.f, 1056.f));
    return *reinterpret_cast<uint32_t *>(&r);
}

enum { FMT_Q4_0 = 0, FMT_Q4_K = 1, FMT_Q6_K = 2 };
struct GemmW { const uint4 *qs; const void *sc; const void *aux; const uint2 *hi; };

// One kernel for the three block formats.  Per 128-weight group a warp runs eight K=16 MMA steps on exact small
// integers (q-8, q, q-32 in fp16) against the fp16 activation split and applies the block scales in float32 outside the
// MMA, so the only rounding is float32 accumulation as in the reference:
//   Q4_0  y += d_b * S_b                               S_b = sum over a 32-block of (q-8)*x     (cpu.go:842-911)
//   Q4_K  y += fl(d*sc_u) * S_u - fl(dmin*m_u) * X_u    S_u = sum q*x, X_u = sum x over sub-block u (dequant.go:342-396)
//   Q6_K  y += fl(d*sc_u) * S_u                         S_u = sum (q-32)*x over a 16-weight sub-block (dequant.go:272-331)
// grid: (ceil(N/128), split_k, ceil(M / (8*NT))).  out layout: [split][M][ld_out]
template <int FMT, int NT, int TERMS>
__global__ void __launch_bounds__(256, NT == 1 ? 3 : 2)
gemm_quant_kernel(GemmW W, const __half *__restrict__ xh, const __half *__restrict__ xl, const float *__restrict__ xscale,
                  const float *__restrict__ xbsum, float *__restrict__ out, int M, int N, int k_groups, int groups_per_split,
                  int x_ld, int ld_out, size_t part_stride) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int MT = 8 * NT;
    constexpr int BS_FLOATS = FMT == FMT_Q4_K ? MT * 4 : 0;                 // per-32-block activation sums of the group
    constexpr int X_BYTES = TERMS * MT * GEMM_XLD * 2 + BS_FLOATS * 4;                  // activation part of a stage
    constexpr int STAGE_BYTES = gemm_stage_bytes(FMT, NT, TERMS), GEMM_STAGES = gemm_stages(FMT, NT);
    constexpr bool RING = gemm_ring(NT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int m0 = blockIdx.z * MT;
    const int g_begin = blockIdx.y * groups_per_split;
    const int g_end = min(k_groups, g_begin + groups_per_split);
    const int n_iter = g_end - g_begin;
    const int r0 = blockIdx.x * GEMM_ROWS + warp * 16;
    const int rowA = min(r0 + g, N - 1), rowB = min(r0 + g + 8, N - 1);
    const uint4 *qA = W.qs + ((size_t)rowA * k_groups) * 4 + c;
    const uint4 *qB = W.qs + ((size_t)rowB * k_groups) * 4 + c;
    const uint2 *sA = reinterpret_cast<const uint2 *>(W.sc) + (size_t)rowA * k_groups;
    const uint2 *sB = reinterpret_cast<const uint2 *>(W.sc) + (size_t)rowB * k_groups;
    const uint2 *hA = FMT == FMT_Q6_K ? W.hi + ((size_t)rowA * k_groups) * 4 + c : nullptr;
    const uint2 *hB = FMT == FMT_Q6_K ? W.hi + ((size_t)rowB * k_groups) * 4 + c : nullptr;

    auto load_x = [&](int stage, int grp) {
        unsigned char *st = smem_raw + (size_t)stage * STAGE_BYTES;
        constexpr int CHUNKS = TERMS * MT * 16;      // TERMS * MT rows of 256 bytes = 16 chunks of 16 bytes each
        for (int i = threadIdx.x; i < CHUNKS; i += 256) {
            int term = i / (MT * 16), rem = i % (MT * 16), r = rem >> 4, ch = rem & 15;
            int m = min(m0 + r, M - 1);
            const __half *src = (term == 0 ? xh : xl) + (size_t)m * x_ld + (size_t)grp * 128 + ch * 8;
            cp_async16(reinterpret_cast<__half *>(st) + (term * MT + r) * GEMM_XLD + ch * 8, src);
        }
        if (FMT == FMT_Q4_K)
            for (int r = threadIdx.x; r < MT; r += 256) {
                int m = min(m0 + r, M - 1);
                cp_async16(st + TERMS * MT * GEMM_XLD * 2 + r * 16, xbsum + (size_t)m * (x_ld / 32) + (size_t)grp * 4);
            }
    };

    // the weight words of a group travel through the same ring: every lane copies the 16 bytes of its two rows (and lane c = 0
    // the rows' 8 bytes of scales), so a CTA has GEMM_STAGES - 1 groups of weights in flight without holding them in registers
    auto load_w = [&](int stage, int grp) {
        unsigned char *st = smem_raw + (size_t)stage * STAGE_BYTES + X_BYTES;
        cp_async16(st + (warp * 64 + lane) * 16, qA + (size_t)grp * 4);
        cp_async16(st + (warp * 64 + 32 + lane) * 16, qB + (size_t)grp * 4);
        if (c == 0) {
            cp_async8(st + GEMM_W_BYTES + (warp * 16 + g) * 8, sA + grp);
            cp_async8(st + GEMM_W_BYTES + (warp * 16 + 8 + g) * 8, sB + grp);
        }
        if (FMT == FMT_Q6_K) {
            cp_async8(st + GEMM_W_BYTES + GEMM_SC_BYTES + (warp * 64 + lane) * 8, hA + (size_t)grp * 4);
            cp_async8(st + GEMM_W_BYTES + GEMM_SC_BYTES + (warp * 64 + 32 + lane) * 8, hB + (size_t)grp * 4);
        }
    };

    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; t++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[t][i] = 0.f;

    // the weights do not depend on the kernel before this one in the stream: the ring's first groups are requested before the
    // wait for that kernel (one commit group, older than every activation group)
    uint4 wA = make_uint4(0, 0, 0, 0), wB = wA; uint2 dA = make_uint2(0, 0), dB = dA, eA = dA, eB = dA;
    if (RING) {
#pragma unroll
        for (int s = 0; s < GEMM_STAGES - 1; s++)
            if (s < n_iter) load_w(s, g_begin + s);
        cp_async_commit();
    } else if (n_iter > 0) {
        wA = __ldg(qA + (size_t)g_begin * 4); wB = __ldg(qB + (size_t)g_begin * 4); dA = __ldg(sA + g_begin); dB = __ldg(sB + g_begin);
        if (FMT == FMT_Q6_K) { eA = __ldg(hA + (size_t)g_begin * 4); eB = __ldg(hB + (size_t)g_begin * 4); }
    }
    vx_pdl_wait();
#pragma unroll
    for (int s = 0; s < GEMM_STAGES - 1; s++) {
        if (s < n_iter) load_x(s, g_begin + s);
        cp_async_commit();
    }

    for (int it = 0; it < n_iter; it++) {
        const int grp = g_begin + it;
        uint4 nA = wA, nB = wB; uint2 ndA = dA, ndB = dB, neA = eA, neB = eB;
        if (!RING && it + 1 < n_iter) {      // prefetch the next group's weights into registers
            nA = __ldg(qA + (size_t)(grp + 1) * 4); nB = __ldg(qB + (size_t)(grp + 1) * 4); ndA = __ldg(sA + grp + 1); ndB = __ldg(sB + grp + 1);
            if (FMT == FMT_Q6_K) { neA = __ldg(hA + (size_t)(grp + 1) * 4); neB = __ldg(hB + (size_t)(grp + 1) * 4); }
        }
        // super-block scales (one or two halves per 256 weights); L1/L2 resident, read once per group
        float supA = 0.f, supB = 0.f, supminA = 0.f, supminB = 0.f;
        if (FMT == FMT_Q4_K) {
            const __half2 a2 = reinterpret_cast<const __half2 *>(W.aux)[(size_t)rowA * (k_groups / 2) + (grp >> 1)];
            const __half2 b2 = reinterpret_cast<const __half2 *>(W.aux)[(size_t)rowB * (k_groups / 2) + (grp >> 1)];
            supA = __low2float(a2); supminA = __high2float(a2); supB = __low2float(b2); supminB = __high2float(b2);
        } else if (FMT == FMT_Q6_K) {
            supA = __half2float(reinterpret_cast<const __half *>(W.aux)[(size_t)rowA * (k_groups / 2) + (grp >> 1)]);
            supB = __half2float(reinterpret_cast<const __half *>(W.aux)[(size_t)rowB * (k_groups / 2) + (grp >> 1)]);
        }
        cp_async_wait<GEMM_STAGES - 2>();
        __syncthreads();
        if (it + GEMM_STAGES - 1 < n_iter) {                 // refill the freed stage
            if (RING) load_w((it + GEMM_STAGES - 1) % GEMM_STAGES, grp + GEMM_STAGES - 1);
            load_x((it + GEMM_STAGES - 1) % GEMM_STAGES, grp + GEMM_STAGES - 1);
        }
        cp_async_commit();

        const unsigned char *stp = smem_raw + (size_t)(it % GEMM_STAGES) * STAGE_BYTES;
        const __half *xst = reinterpret_cast<const __half *>(stp);
        const unsigned char *wst = stp + X_BYTES;
        if (RING) {
            wA = *reinterpret_cast<const uint4 *>(wst + (warp * 64 + lane) * 16); wB = *reinterpret_cast<const uint4 *>(wst + (warp * 64 + 32 + lane) * 16);
            dA = *reinterpret_cast<const uint2 *>(wst + GEMM_W_BYTES + (warp * 16 + g) * 8); dB = *reinterpret_cast<const uint2 *>(wst + GEMM_W_BYTES + (warp * 16 + 8 + g) * 8);
            if (FMT == FMT_Q6_K) {
                eA = *reinterpret_cast<const uint2 *>(wst + GEMM_W_BYTES + GEMM_SC_BYTES + (warp * 64 + lane) * 8);
                eB = *reinterpret_cast<const uint2 *>(wst + GEMM_W_BYTES + GEMM_SC_BYTES + (warp * 64 + 32 + lane) * 8);
            }
        }
        const float *bss = reinterpret_cast<const float *>(stp + TERMS * MT * GEMM_XLD * 2);
        const uint32_t wa[4] = {wA.x, wA.y, wA.z, wA.w}, wb[4] = {wB.x, wB.y, wB.z, wB.w};
        const uint32_t da[2] = {dA.x, dA.y}, db[2] = {dB.x, dB.y};
        const uint32_t ea[2] = {eA.x, eA.y}, eb[2] = {eB.x, eB.y};

        // one scaling unit = the MMA steps that share a scale: two for the 4-bit formats, one for Q6_K
        auto run_steps = [&](float (&blk)[NT][4], const uint32_t (&a)[4], int xoff) {
#pragma unroll
            for (int t = 0; t < NT; t++) {
                const __half *p = xst + (8 * t + g) * GEMM_XLD + xoff + 4 * c;
                uint2 b = *reinterpret_cast<const uint2 *>(p);
                mma_f16(blk[t], a, b.x, b.y);
                if (TERMS == 2) {
                    uint2 bl = *reinterpret_cast<const uint2 *>(p + MT * GEMM_XLD);
                    mma_f16(blk[t], a, bl.x, bl.y);
                }
            }
        };
        if (FMT == FMT_Q4_0) {
#pragma unroll
            for (int i = 0; i < 4; i++) {                       // block i of the group; word i holds its 32 nibbles' lane share
                float blk[NT][4];
#pragma unroll
                for (int t = 0; t < NT; t++) { blk[t][0] = blk[t][1] = blk[t][2] = blk[t][3] = 0.f; }
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    uint32_t va = wa[i] >> (4 * nib), vb = wb[i] >> (4 * nib);
                    uint32_t a[4];
                    a[0] = nib2_to_half2(va); a[2] = nib2_to_half2(va >> 8);
                    a[1] = nib2_to_half2(vb); a[3] = nib2_to_half2(vb >> 8);
                    run_steps(blk, a, 32 * i + 16 * nib);
                }
                uint32_t dpa = da[i >> 1], dpb = db[i >> 1];
                float fa = __half2float(__ushort_as_half((unsigned short)((i & 1) ? (dpa >> 16) : (dpa & 0xFFFF))));
                float fb = __half2float(__ushort_as_half((unsigned short)((i & 1) ? (dpb >> 16) : (dpb & 0xFFFF))));
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    acc[t][0] = fmaf(fa, blk[t][0], acc[t][0]); acc[t][1] = fmaf(fa, blk[t][1], acc[t][1]);
                    acc[t][2] = fmaf(fb, blk[t][2], acc[t][2]); acc[t][3] = fmaf(fb, blk[t][3], acc[t][3]);
                }
            }
        } else if (FMT == FMT_Q4_K) {
#pragma unroll
            for (int u = 0; u < 4; u++) {                       // sub-block u = 2*jj + nib of the group: elements 32u .. 32u+31
                const int jj = u >> 1, nib = u & 1;
                float blk[NT][4];
#pragma unroll
                for (int t = 0; t < NT; t++) { blk[t][0] = blk[t][1] = blk[t][2] = blk[t][3] = 0.f; }
#pragma unroll
                for (int tp = 0; tp < 2; tp++) {
                    uint32_t va = wa[2 * jj + tp] >> (4 * nib), vb = wb[2 * jj + tp] >> (4 * nib);
                    uint32_t a[4];       // unsigned nibbles: undo the -8 of nib2_to_half2 by using the raw magic form
                    uint32_t ha = (va & 0x000F000Fu) | 0x64006400u, hb2 = ((va >> 8) & 0x000F000Fu) | 0x64006400u;
                    uint32_t hc = (vb & 0x000F000Fu) | 0x64006400u, hd = ((vb >> 8) & 0x000F000Fu) | 0x64006400u;
                    const __half2 k1024 = __floats2half2_rn(1024.f, 1024.f);
                    __half2 r0 = __hsub2(*reinterpret_cast<__half2 *>(&ha), k1024), r2 = __hsub2(*reinterpret_cast<__half2 *>(&hb2), k1024);
                    __half2 r1 = __hsub2(*reinterpret_cast<__half2 *>(&hc), k1024), r3 = __hsub2(*reinterpret_cast<__half2 *>(&hd), k1024);
                    a[0] = *reinterpret_cast<uint32_t *>(&r0); a[2] = *reinterpret_cast<uint32_t *>(&r2);
                    a[1] = *reinterpret_cast<uint32_t *>(&r1); a[3] = *reinterpret_cast<uint32_t *>(&r3);
                    run_steps(blk, a, 32 * u + 16 * tp);
                }
                const float fa = __fmul_rn(supA, (float)((da[0] >> (8 * u)) & 0xFF)), ma = __fmul_rn(supminA, (float)((da[1] >> (8 * u)) & 0xFF));
                const float fb = __fmul_rn(supB, (float)((db[0] >> (8 * u)) & 0xFF)), mb = __fmul_rn(supminB, (float)((db[1] >> (8 * u)) & 0xFF));
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    const float x0 = bss[(8 * t + 2 * c) * 4 + u], x1 = bss[(8 * t + 2 * c + 1) * 4 + u];
                    acc[t][0] += fa * blk[t][0] - ma * x0; acc[t][1] += fa * blk[t][1] - ma * x1;
                    acc[t][2] += fb * blk[t][2] - mb * x0; acc[t][3] += fb * blk[t][3] - mb * x1;
                }
            }
        } else {
#pragma unroll
            for (int u = 0; u < 8; u++) {                       // 16-weight sub-block u: elements 16u .. 16u+15, one MMA step
                float blk[NT][4];
#pragma unroll
                for (int t = 0; t < NT; t++) { blk[t][0] = blk[t][1] = blk[t][2] = blk[t][3] = 0.f; }
                const uint32_t va = wa[u >> 1] >> (4 * (u & 1)), vb = wb[u >> 1] >> (4 * (u & 1));
                const uint32_t ha = (ea[u >> 2] >> (8 * (u & 3))) & 0xFF, hb2 = (eb[u >> 2] >> (8 * (u & 3))) & 0xFF;
                uint32_t a[4];
                a[0] = q6_to_half2(va, ((ha & 0x03) << 4) | ((ha & 0x30) << 16));
                a[2] = q6_to_half2(va >> 8, ((ha & 0x0C) << 2) | ((ha & 0xC0) << 14));
                a[1] = q6_to_half2(vb, ((hb2 & 0x03) << 4) | ((hb2 & 0x30) << 16));
                a[3] = q6_to_half2(vb >> 8, ((hb2 & 0x0C) << 2) | ((hb2 & 0xC0) << 14));
                run_steps(blk, a, 16 * u);
                const float fa = __fmul_rn(supA, (float)(int)(int8_t)((da[u >> 2] >> (8 * (u & 3))) & 0xFF));
                const float fb = __fmul_rn(supB, (float)(int)(int8_t)((db[u >> 2] >> (8 * (u & 3))) & 0xFF));
#pragma unroll
                for (int t = 0; t < NT; t++) {
                    acc[t][0] = fmaf(fa, blk[t][0], acc[t][0]); acc[t][1] = fmaf(fa, blk[t][1], acc[t][1]);
                    acc[t][2] = fmaf(fb, blk[t][2], acc[t][2]); acc[t][3] = fmaf(fb, blk[t][3], acc[t][3]);
                }
            }
        }
        if (!RING) { wA = nA; wB = nB; dA = ndA; dB = ndB; eA = neA; eB = neB; }
    }
    cp_async_wait<0>();

    float *o = out + (size_t)blockIdx.y * part_stride;
    const int nA = r0 + g, nB = r0 + g + 8;
#pragma unroll
    for (int t = 0; t < NT; t++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            int m = m0 + 8 * t + 2 * c + e;
            if (m < M) {
                float s = xscale[m];
                if (nA < N) o[(size_t)m * ld_out + nA] = acc[t][e] * s;
                if (nB < N) o[(size_t)m * ld_out + nB] = acc[t][2 + e] * s;
            }
        }
    }
}

template <int FMT, int NT, int TERMS>
static int gemm_launch_nt(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int split,
                          int gps, size_t part_stride) {
    constexpr int MT = 8 * NT;
    size_t smem = (size_t)gemm_stages(FMT, NT) * gemm_stage_bytes(FMT, NT, TERMS);
    auto kern = gemm_quant_kernel<FMT, NT, TERMS>;
    if (smem > 48 * 1024) VX_CUDA(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(ceil_div(w.n, GEMM_ROWS), split, ceil_div(m, MT));
    GemmW W{(const uint4 *)w.qs, w.sc, w.aux, (const uint2 *)w.hi};
    cudaError_t le = vx_launch_dependent(kern, grid, dim3(256), smem, c->stream, W, (const __half *)x.hi, (const __half *)x.lo, (const float *)x.scale,
                                         (const float *)x.bsum, out, m, w.n, w.k_pad / 128, gps, x.k_pad, ld_out, part_stride);
    if (le != cudaSuccess) return vx_cuda_fail(c, le, "projection launch");
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}
template <int FMT>
static int gemm_launch_fmt(vx_ctx *c, int nt, int terms, const VxWeight &w, const VxSplit &x, int m, float *dst, int ld, int split, int gps,
                           size_t pstride) {
#define VX_GEMM_CASE(NTV)                                                                                   \
    case NTV:                                                                                               \
        return terms == 2 ? gemm_launch_nt<FMT, NTV, 2>(c, w, x, m, dst, ld, split, gps, pstride)           \
                          : gemm_launch_nt<FMT, NTV, 1>(c, w, x, m, dst, ld, split, gps, pstride);
    switch (nt) {
        VX_GEMM_CASE(1) VX_GEMM_CASE(2) VX_GEMM_CASE(4) VX_GEMM_CASE(8)
    }
#undef VX_GEMM_CASE
    return VX_E_BAD_ARG;
}

static int g_gemm_terms = 2;   // 2: x = hi + lo (float32-faithful); 1: fp16 activations only
int g_vx_pdl = 1;               // projections start under the tail of the kernel before them (programmatic dependent launch)
static int g_q4k_tc_floor = 17;  // Q4_K: 33 while it ran on the one-CTA-per-tile kernel; on the persistent kernel 17 like the others
                                 // (70B-shaped step at 32 rows 10.46 -> 8.80 ms, 8B-shaped at 24 rows 3.57 -> 3.29 ms)
static int g_tc_min_rows = 17;  // batches of at least this many rows use the tcgen05 kernel (0 = never)

// out receives [m][ld_out] when *n_parts_out == 1, otherwise `parts` holds [n_parts][m][w.n]
int vxq_gemm(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out,
             float *parts, size_t parts_cap_floats) {
    if (w.type != VX_T_Q4_0 && w.type != VX_T_Q4_K && w.type != VX_T_Q6_K)
        return vx_fail(c, VX_E_UNSUPPORTED, "projection: weight type %d has no MMA kernel", w.type);
    if (x.k_pad != w.k_pad) return vx_fail(c, VX_E_BAD_ARG, "projection: activation row stride %d != weight k_pad %d", x.k_pad, w.k_pad);
    // measured crossover to the tcgen05 kernels (whose cost per weight does not depend on the batch): 17 rows
    if (g_gemm_terms == 2 && vxq_gemv_eligible(w, m)) return vxq_gemv(c, w, x, m, out, ld_out, n_parts_out, parts, parts_cap_floats);
    const int tc_rows = (w.type == VX_T_Q4_K && g_tc_min_rows > 0) ? max(g_tc_min_rows, g_q4k_tc_floor) : g_tc_min_rows;
    if (tc_rows > 0 && m >= tc_rows && g_gemm_terms == 2)
        return vxq_gemm_tc(c, w, x, m, out, ld_out, n_parts_out, parts, parts_cap_floats);
    int k_groups = w.k_pad / 128;
    int nt = m <= 8 ? 1 : m <= 16 ? 2 : m <= 32 ? 4 : 8;
    int ctas = ceil_div(w.n, GEMM_ROWS) * ceil_div(m, 8 * nt);
    // split-K so that the CTAs fill whole waves of the GPU (two resident CTAs per SM): pick the split with the best
    // wave efficiency, preferring fewer partials on ties
    int split = 1;
    if (parts) {
        const int slots = 2 * c->sm_count;
        double best = 0.0;
        for (int s = 1; s <= 8 && s <= max(1, k_groups / 4); s++) {
            if ((size_t)s * m * w.n > parts_cap_floats) break;
            int gps_s = ceil_div(k_groups, s), s_eff = ceil_div(k_groups, gps_s);
            long n_cta = (long)ctas * s_eff;
            double eff = (double)n_cta / (double)(ceil_div64(n_cta, slots) * slots) * ((double)k_groups / (double)(gps_s * s_eff));
            if (eff > best + 0.03) { best = eff; split = s; }
        }
    }
    int gps = ceil_div(k_groups, split);
    split = ceil_div(k_groups, gps);
    float *dst = split > 1 ? parts : out;
    int ld = split > 1 ? w.n : ld_out;
    size_t pstride = (size_t)m * w.n;
    *n_parts_out = split;
    switch (w.type) {
    case VX_T_Q4_0: return gemm_launch_fmt<FMT_Q4_0>(c, nt, g_gemm_terms, w, x, m, dst, ld, split, gps, pstride);
    case VX_T_Q4_K: return gemm_launch_fmt<FMT_Q4_K>(c, nt, g_gemm_terms, w, x, m, dst, ld, split, gps, pstride);
    default:        return gemm_launch_fmt<FMT_Q6_K>(c, nt, g_gemm_terms, w, x, m, dst, ld, split, gps, pstride);
    }
}

__global__ void reduce_parts_kernel(const float *__restrict__ parts, int n_parts, int m, int n, float *__restrict__ out, int ld_out) {
    long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (idx >= (long)m * n) return;
    float s = 0.f;
    for (int p = 0; p < n_parts; p++) s += parts[(size_t)p * m * n + idx];
    out[(size_t)(idx / n) * ld_out + idx % n] = s;
}

int vxq_reduce_parts(vx_ctx *c, const float *parts, int n_parts, int m, int n, float *out, int ld_out) {
    long total = (long)m * n;
    reduce_parts_kernel<<<(unsigned)((total + 255) / 256), 256, 0, c->stream>>>(parts, n_parts, m, n, out, ld_out);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// ------------------------------------------------------------------ synthetic Q4_0 weights
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull; z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull; z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
// one thread per 32-weight block: draw ~N(0, sigma) with a counter hash + Box-Muller, then quantise with
// d = signed-absmax / -8 (stored as fp16), q = clamp(round(x/d) + 8, 0, 15)
__global__ void synth_q4_0_kernel(uint8_t *__restrict__ dst, int64_t n_blocks, uint64_t seed, float sigma) {
    int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    float x[32]; float amax = 0.f, vmax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        uint64_t r = mix64(seed ^ mix64((uint64_t)b * 16 + i / 2));
        float u1 = ((uint32_t)(r >> 40) + 1.0f) * (1.0f / 16777217.0f), u2 = (uint32_t)(r & 0xFFFFFF) * (1.0f / 16777216.0f);
        float rad = sqrtf(-2.0f * __logf(u1)) * sigma;
        float sn, cs; __sincosf(6.283185307f * u2, &sn, &cs);
        x[i] = rad * cs; x[i + 1] = rad * sn;
    }
#pragma unroll
    for (int i = 0; i < 32; i++) if (fabsf(x[i]) > amax) { amax = fabsf(x[i]); vmax = x[i]; }
    float d = vmax / -8.0f;
    float id = d != 0.f ? 1.0f / d : 0.f;
    uint8_t *p = dst + b * 18;
    unsigned short dh = __half_as_ushort(__float2half_rn(d));
    p[0] = (uint8_t)(dh & 0xFF); p[1] = (uint8_t)(dh >> 8);
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int q0 = min(15, max(0, (int)floorf(x[i] * id + 8.5f)));
        int q1 = min(15, max(0, (int)floorf(x[i + 16] * id + 8.5f)));
        p[2 + i] = (uint8_t)(q0 | (q1 << 4));
    }
}

extern "C" {

int vx_dequantize(vx_ctx *c, int type, vx_dptr raw, vx_dptr out, int64_t n) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, raw && out && n >= 0, "bad arguments");
    return dequant_launch(c, type, dp<void>(raw), dp<float>(out), n);
}

int vx_synth_q4_0(vx_ctx *c, vx_dptr dst, int64_t n, uint64_t seed, float sigma) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, dst && n > 0 && n % 32 == 0, "element count must be a positive multiple of 32");
    int64_t nb = n / 32;
    synth_q4_0_kernel<<<(unsigned)ceil_div64(nb, 128), 128, 0, c->stream>>>(dp<uint8_t>(dst), nb, seed, sigma);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// Valid Q4_K / Q6_K blocks with hashed payload bytes, for benchmarks that need weights of a K-quant model's shape and
// byte size without a host-side encoder in the loop.  Every byte pattern of the quant and scale fields is a valid
// block; only the fp16 super-scales are chosen, so that the dequantised weights have a standard deviation near sigma
// (Q4_K: w = d*sc*q - dmin*m with sc, m in [0,63], q in [0,15]; Q6_K: w = d*sc*q with sc in [-128,127], q in [-32,31]).
__global__ void synth_kquant_kernel(uint8_t *__restrict__ dst, int64_t n_blocks, int type, uint64_t seed, float sigma) {
    int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    const int bytes = type == VX_T_Q4_K ? 144 : 210;
    uint8_t *p = dst + b * bytes;
    for (int i = 0; i < bytes; i += 8) {
        uint64_t r = mix64(seed ^ mix64((uint64_t)b * 32 + i / 8));
        for (int j = 0; j < 8 && i + j < bytes; j++) p[i + j] = (uint8_t)(r >> (8 * j));
    }
    if (type == VX_T_Q4_K) {
        unsigned short d = __half_as_ushort(__float2half_rn(sigma / 200.f)), dm = __half_as_ushort(__float2half_rn(7.5f * sigma / 200.f));
        p[0] = (uint8_t)(d & 0xFF); p[1] = (uint8_t)(d >> 8); p[2] = (uint8_t)(dm & 0xFF); p[3] = (uint8_t)(dm >> 8);
    } else {
        unsigned short d = __half_as_ushort(__float2half_rn(sigma / 1370.f));
        p[208] = (uint8_t)(d & 0xFF); p[209] = (uint8_t)(d >> 8);
    }
}

int vx_synth_kquant(vx_ctx *c, vx_dptr dst, int type, int64_t n, uint64_t seed, float sigma) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, dst && n > 0 && n % 256 == 0 && (type == VX_T_Q4_K || type == VX_T_Q6_K), "Q4_K or Q6_K, element count a positive multiple of 256");
    int64_t nb = n / 256;
    synth_kquant_kernel<<<(unsigned)ceil_div64(nb, 128), 128, 0, c->stream>>>(dp<uint8_t>(dst), nb, type, seed, sigma);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// QuantizedMatMul on raw GGUF bytes: repack + split into the context scratch, then the MMA kernel.
static int matmul_quant(vx_ctx *c, int type, vx_dptr a, vx_dptr b_raw, vx_dptr out, int m, int n, int k) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (m <= 0 || n <= 0) return VX_OK;
    VX_REQUIRE(c, a && b_raw && out, "nil device pointer");
    const int blk = type == VX_T_Q4_0 ? 32 : 256;
    if (k <= 0 || k % blk != 0) return vx_fail(c, VX_E_BAD_ARG, "k=%d must be a positive multiple of %d", k, blk);
    VxRepackLayout L;
    vxq_layout(type, n, k, &L);
    size_t hi, lo, so, bo; int kp;
    size_t sbytes = vxq_split_bytes(m, k, &hi, &lo, &so, &bo, &kp);
    size_t parts_floats = (size_t)8 * m * n;
    // The repacked weights: kept across calls for tensors that live in a permanent allocation (the reference hands the same
    // weight buffers to MatMulQ* on every token; repacking them each time would double the traffic of a mat-vec), rebuilt
    // in the scratch buffer otherwise.  An entry goes when the API overwrites or frees the raw bytes (vx_repack_invalidate).
    const void *raw = dp<void>(b_raw);
    const double bpw = type == VX_T_Q4_0 ? 18.0 / 32 : type == VX_T_Q4_K ? 144.0 / 256 : 210.0 / 256;
    const size_t raw_bytes = (size_t)((double)n * k * bpw);
    char *wbuf = nullptr;
    if (c->repack_cache) {
        auto it = c->repacked.find(raw);
        if (it != c->repacked.end() && (it->second.type != type || it->second.n != n || it->second.k != k)) {
            vx_repack_invalidate(c, raw, 1);
            it = c->repacked.end();
        }
        if (it != c->repacked.end()) wbuf = (char *)it->second.buf;
        else {
            bool permanent = false;
            for (const auto &pa : c->permanent)
                if ((const char *)raw >= (const char *)pa.first && (const char *)raw + raw_bytes <= (const char *)pa.first + pa.second) { permanent = true; break; }
            void *nb = nullptr;
            if (permanent && cudaMalloc(&nb, L.total) == cudaSuccess) {
                int rc = vxq_repack_rows(c, type, raw, n, k, nb, L, 0);
                if (rc != VX_OK) { cudaFree(nb); return rc; }
                c->repacked[raw] = vx_ctx::Repacked{type, n, k, raw_bytes, nb};
                wbuf = (char *)nb;
            } else cudaGetLastError();
        }
    }
    void *base;
    VX_TRY(vx_scratch(c, (wbuf ? 0 : L.total) + sbytes + parts_floats * 4 + 1024, &base));
    char *p = (char *)base;
    if (!wbuf) VX_TRY(vxq_repack_rows(c, type, raw, n, k, p, L, 0));
    VxWeight w;
    vxq_weight_view(type, n, k, wbuf ? wbuf : p, L, &w);
    char *sp = p + (wbuf ? 0 : L.total);
    VxSplit s{(__half *)(sp + hi), (__half *)(sp + lo), (float *)(sp + so), (float *)(sp + bo), kp};
    VX_TRY(vxq_split_rows(c, dp<float>(a), m, k, k, s));
    float *parts = (float *)(sp + sbytes);
    int np = 1;
    VX_TRY(vxq_gemm(c, w, s, m, dp<float>(out), n, &np, parts, parts_floats));
    if (np > 1) VX_TRY(vxq_reduce_parts(c, parts, np, m, n, dp<float>(out), n));
    return VX_OK;
}
int vx_matmul_q4_0(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) { return matmul_quant(c, VX_T_Q4_0, a, b, out, m, n, k); }
int vx_matmul_q4_k(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) { return matmul_quant(c, VX_T_Q4_K, a, b, out, m, n, k); }
int vx_matmul_q6_k(vx_ctx *c, vx_dptr a, vx_dptr b, vx_dptr out, int m, int n, int k) { return matmul_quant(c, VX_T_Q6_K, a, b, out, m, n, k); }

int vx_set_tc_min_rows(int rows) { if (rows >= 1000) { g_q4k_tc_floor = rows - 1000; return VX_OK; } g_tc_min_rows = rows; return VX_OK; }   // (1000 + r: the Q4_K floor, for timing comparisons)
int vx_set_repack_cache(vx_ctx *c, int enable) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    c->repack_cache = enable != 0;
    if (!enable) vx_repack_invalidate(c, nullptr, ~(size_t)0 >> 1);
    return VX_OK;
}
int vx_set_dependent_launch(int mode) { g_vx_pdl = mode < 0 ? 0 : mode > 2 ? 2 : mode; return VX_OK; }
int vx_set_gemm_terms(int terms) { if (terms == 1 || terms == 2) { g_gemm_terms = terms; return VX_OK; } return VX_E_BAD_ARG; }

}  // extern "C"
