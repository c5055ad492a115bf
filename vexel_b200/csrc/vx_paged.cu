// PagedKVOps (inference/backend/backend.go:415-466): scatter into the block pool and paged decode
// attention.  Semantics follow the reference's Metal shaders (backend/metal/metal_bridge_darwin.m:
// 8539-8755, 11074-11311): score = (q.k)*scale, max-subtracted softmax, out = sum w*v, GQA
// kvHead = qHead / (Hq/Hkv); plus the soft-cap and sliding-window variants the CPU branch applies
// (runtime/block.go:925-953, backend/cpu/cpu.go:705-767).
//
// The decode kernel is a ragged, split-K FlashDecoding pass: a work item is (query row, chunk of pages);
// a CTA of four warps handles one work item for one KV head, each warp streaming whole 16-token pages
// with 128-bit loads (a token's head slice is D*2 contiguous bytes), online softmax with warp shuffles,
// then a four-way merge in shared memory.  Rows cut into several chunks are finished by a merge kernel.
#include <algorithm>

#include "vx_paged.cuh"

// ------------------------------------------------------------------ scatter (ReshapePagedKV[F16])
template <typename T>
__global__ void reshape_paged_kernel(const float *__restrict__ src, T *__restrict__ pool, const int32_t *__restrict__ blk,
                                     const int32_t *__restrict__ off, int n_tokens, int hs, int block_size, int is_v) {
    long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
    if (idx >= (long)n_tokens * hs) return;
    int t = (int)(idx / hs), e = (int)(idx % hs);
    size_t part = (size_t)block_size * hs;
    size_t dst = (size_t)blk[t] * 2 * part + (is_v ? part : 0) + (size_t)off[t] * hs + e;
    if (sizeof(T) == 2) reinterpret_cast<__half *>(pool)[dst] = __float2half_rn(src[idx]);   // (half)x, round-to-nearest-even
    else reinterpret_cast<float *>(pool)[dst] = src[idx];
}

// ------------------------------------------------------------------ generic paged attention
// Any block size / head dim <= 256 / pool type.  One CTA (256 threads) per (row, q head).
__global__ void paged_generic_kernel(VxAttnArgs a) {
    extern __shared__ float sm[];
    float *qs = sm, *ps = sm + a.head_dim;
    __shared__ float red[32];
    int h = blockIdx.x, row = blockIdx.y, D = a.head_dim;
    int kvh = h / (a.n_q_heads / a.n_kv_heads);
    int kv_start = a.row_kv_start ? a.row_kv_start[row] : 0, kv_len = a.row_kv_len[row];
    const int32_t *table = a.tables[a.row_slot[row]];
    size_t hs = (size_t)a.n_kv_heads * D, part = (size_t)a.block_size * hs;
    const float *qh = a.q + (size_t)row * a.q_row_stride + (size_t)h * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qh[d];
    __syncthreads();
    const __half *ph = (const __half *)a.pool; const float *pf = (const float *)a.pool;
    float m_run = -INFINITY, l_run = 0.f, acc = 0.f;
    for (int t0 = kv_start; t0 < kv_len; t0 += 256) {
        int pos = t0 + threadIdx.x;
        float s = -INFINITY;
        if (pos < kv_len) {
            size_t base = (size_t)table[pos / a.block_size] * 2 * part + (size_t)(pos % a.block_size) * hs + (size_t)kvh * D;
            float dot = 0.f;
            for (int d = 0; d < D; d++) dot = fmaf(qs[d], a.pool_is_f16 ? __half2float(ph[base + d]) : pf[base + d], dot);
            s = dot * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        }
        float m_new = fmaxf(m_run, block_max(s, red));
        float p = pos < kv_len ? __expf(s - m_new) : 0.f;
        float corr = __expf(m_run - m_new);
        float psum = block_sum(p, red);
        ps[threadIdx.x] = p;
        __syncthreads();
        l_run = l_run * corr + psum;
        acc *= corr;
        if (threadIdx.x < D) {
            int cnt = min(256, kv_len - t0);
            for (int i = 0; i < cnt; i++) {
                int pp = t0 + i;
                size_t base = (size_t)table[pp / a.block_size] * 2 * part + part + (size_t)(pp % a.block_size) * hs + (size_t)kvh * D + threadIdx.x;
                acc = fmaf(ps[i], a.pool_is_f16 ? __half2float(ph[base]) : pf[base], acc);
            }
        }
        m_run = m_new;
        __syncthreads();
    }
    if (threadIdx.x < D) a.out[(size_t)row * a.out_row_stride + (size_t)h * D + threadIdx.x] = l_run > 0.f ? acc / l_run : 0.f;
}

// ------------------------------------------------------------------ split-K FlashDecoding kernel (f16 pool, 16-token pages)
// one atomic per warp: non-negative floats order like their bit patterns (a NaN or infinity becomes a huge bound, and the
// row scale falls back to 1 exactly as the row-wide maximum would make it)
__device__ __forceinline__ void vx_raise_row_bound(unsigned int *slot, float v) {
    v = warp_max(v);
    if ((threadIdx.x & 31) == 0 && v > 0.f) atomicMax(slot, __float_as_uint(v));
}
constexpr int ATT_WARPS = 4;
constexpr int ATT_BS = 16;

__device__ __forceinline__ void unpack8(const uint4 &u, float (&f)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// Five CTAs per SM (96 registers, a two-word spill) instead of the four that 115 registers allow: 3 % more bandwidth.  Six
// (80 registers) spills enough to give that back; eight is 25 % slower.  Folding the chunk merge and the output split into
// this kernel (arrival tickets, the last CTA of a row finishes it) was measured too: the fence and the ticket every CTA then
// pays cost more (+9 us per launch) than the separate 10 us merge kernel.
template <int D, int G>
__global__ void __launch_bounds__(ATT_WARPS * 32, 5)
paged_flash_kernel(VxAttnArgs a) {
    vx_pdl_wait();
    vx_pdl_trigger();
    constexpr int LPT = D / 8;            // lanes per token
    constexpr int TPW = 32 / LPT;         // tokens per warp-wide load
    constexpr int NI = ATT_BS / TPW;      // loads per page
    __shared__ float sm_m[ATT_WARPS][G], sm_l[ATT_WARPS][G];
    __shared__ __align__(16) float sm_acc[ATT_WARPS][G][D];

    const int wi = blockIdx.x;
    if (wi >= *a.n_work_dev) return;
    const int4 item = a.work[wi];
    const int row = item.x, first_page = item.y, n_pages = item.z;
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tg = lane / LPT, dl = lane % LPT;
    const int kv_start = a.row_kv_start ? a.row_kv_start[row] : 0, kv_len = a.row_kv_len[row];
    const int32_t *table = a.tables[a.row_slot[row]];
    const size_t hs = (size_t)a.n_kv_heads * D;
    const __half *pool = (const __half *)a.pool;

    float qf[G][8];
#pragma unroll
    for (int gi = 0; gi < G; gi++) {
        const float *qp = a.q + (size_t)row * a.q_row_stride + (size_t)(kvh * G + gi) * D + dl * 8;
        float4 q0 = *reinterpret_cast<const float4 *>(qp), q1 = *reinterpret_cast<const float4 *>(qp + 4);
        qf[gi][0] = q0.x; qf[gi][1] = q0.y; qf[gi][2] = q0.z; qf[gi][3] = q0.w;
        qf[gi][4] = q1.x; qf[gi][5] = q1.y; qf[gi][6] = q1.z; qf[gi][7] = q1.w;
    }
    float m_run[G], l_run[G], acc[G][8];
#pragma unroll
    for (int gi = 0; gi < G; gi++) {
        m_run[gi] = -INFINITY; l_run[gi] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; e++) acc[gi][e] = 0.f;
    }

    int page = first_page + warp;
    int blk_next = page < first_page + n_pages ? table[page] : 0;
    for (; page < first_page + n_pages; page += ATT_WARPS) {
        const int blk = blk_next;
        if (page + ATT_WARPS < first_page + n_pages) blk_next = table[page + ATT_WARPS];
        const __half *kbase = pool + (size_t)blk * 2 * ATT_BS * hs + (size_t)kvh * D + dl * 8;
        uint4 kr[NI], vr[NI];
#pragma unroll
        for (int i = 0; i < NI; i++) {
            const __half *kp = kbase + (size_t)(i * TPW + tg) * hs;
            kr[i] = *reinterpret_cast<const uint4 *>(kp);
            vr[i] = *reinterpret_cast<const uint4 *>(kp + ATT_BS * hs);
        }
        float s[NI][G];
        float pmax[G];
#pragma unroll
        for (int gi = 0; gi < G; gi++) pmax[gi] = -INFINITY;
#pragma unroll
        for (int i = 0; i < NI; i++) {
            float kf[8];
            unpack8(kr[i], kf);
            const int pos = page * ATT_BS + i * TPW + tg;
            const bool valid = pos >= kv_start && pos < kv_len;
#pragma unroll
            for (int gi = 0; gi < G; gi++) {
                float d = 0.f;
#pragma unroll
                for (int e = 0; e < 8; e++) d = fmaf(qf[gi][e], kf[e], d);
#pragma unroll
                for (int o = 1; o < LPT; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                d *= a.scale;
                if (a.softcap > 0.f) d = a.softcap * tanhf(d / a.softcap);
                s[i][gi] = valid ? d : -INFINITY;
                pmax[gi] = fmaxf(pmax[gi], s[i][gi]);
            }
        }
#pragma unroll
        for (int gi = 0; gi < G; gi++) {
#pragma unroll
            for (int o = LPT; o < 32; o <<= 1) pmax[gi] = fmaxf(pmax[gi], __shfl_xor_sync(0xffffffffu, pmax[gi], o));
            const float m_new = fmaxf(m_run[gi], pmax[gi]);
            if (m_new == -INFINITY) continue;      // page entirely outside the window (uniform across the warp)
            const float corr = __expf(m_run[gi] - m_new);
            l_run[gi] *= corr;
#pragma unroll
            for (int e = 0; e < 8; e++) acc[gi][e] *= corr;
            m_run[gi] = m_new;
        }
#pragma unroll
        for (int i = 0; i < NI; i++) {
            float vf[8];
            unpack8(vr[i], vf);
#pragma unroll
            for (int gi = 0; gi < G; gi++) {
                // masked positions have s = -inf -> p = 0; the pool holds only finite fp16 values
                const float p = (s[i][gi] == -INFINITY) ? 0.f : __expf(s[i][gi] - m_run[gi]);
                l_run[gi] += p;
#pragma unroll
                for (int e = 0; e < 8; e++) acc[gi][e] = fmaf(p, vf[e], acc[gi][e]);
            }
        }
    }

    // combine the token groups of the warp, then the warps of the CTA
#pragma unroll
    for (int gi = 0; gi < G; gi++) {
#pragma unroll
        for (int o = LPT; o < 32; o <<= 1) {
            l_run[gi] += __shfl_xor_sync(0xffffffffu, l_run[gi], o);
#pragma unroll
            for (int e = 0; e < 8; e++) acc[gi][e] += __shfl_xor_sync(0xffffffffu, acc[gi][e], o);
        }
        if (tg == 0) {
            if (dl == 0) { sm_m[warp][gi] = m_run[gi]; sm_l[warp][gi] = l_run[gi]; }
            float4 *dst = reinterpret_cast<float4 *>(&sm_acc[warp][gi][dl * 8]);
            dst[0] = make_float4(acc[gi][0], acc[gi][1], acc[gi][2], acc[gi][3]);
            dst[1] = make_float4(acc[gi][4], acc[gi][5], acc[gi][6], acc[gi][7]);
        }
    }
    __syncthreads();
    const bool single = (a.row_work_start[row + 1] - a.row_work_start[row]) == 1;
    float bound = 0.f;
    for (int idx = threadIdx.x; idx < G * D; idx += ATT_WARPS * 32) {
        const int gi = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) M = fmaxf(M, sm_m[w][gi]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; w++) {
            const float f = sm_m[w][gi] == -INFINITY ? 0.f : __expf(sm_m[w][gi] - M);
            L = fmaf(sm_l[w][gi], f, L); O = fmaf(sm_acc[w][gi][d], f, O);
        }
        const int h = kvh * G + gi;
        const float o = L > 0.f ? O / L : 0.f;
        bound = fmaxf(bound, fabsf(o));
        if (single) {
            a.out[(size_t)row * a.out_row_stride + (size_t)h * D + d] = o;
        } else {
            float *part = a.partials + ((size_t)wi * a.n_q_heads + h) * (D + 2);
            part[d] = O;
            if (d == 0) { part[D] = M; part[D + 1] = L; }
        }
    }
    if (a.row_bound) vx_raise_row_bound(a.row_bound + row, bound);
}

// ------------------------------------------------------------------ grouped-query variant on the tensor cores
// With G query heads per KV head the dot products above cost G times the CUDA-core work per KV byte (at G = 8 more than
// the FMA pipes can deliver at HBM speed) and a warp-shuffle reduction per head.  Here a warp turns one 16-token page into
// two small matrix products on mma.sync.m16n8k16 with the 16 tokens as the M dimension and the group's heads as N = 8:
//   S^T[16 tokens x 8 heads] = K[16 x D] . Q^T[D x 8]          K from shared memory (ldmatrix), Q^T in registers
//   O^T[D x 8 heads]        += V^T[D x 16 tokens] . P^T[16 x 8]  V^T via ldmatrix.trans, P^T from S^T by four shuffles
// K and V pages are staged through a per-warp double buffer with cp.async (16-byte chunks, XOR-swizzled rows so that
// ldmatrix is conflict-free).  q and p are carried as exact fp16 hi + lo pairs (two MMAs each), K and V are fp16 already,
// accumulation is float32: the result matches the float32 reference to rounding, like the CUDA-core kernel.
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(uint32_t saddr, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(saddr), "l"(g));
}
__device__ __forceinline__ uint32_t pack_hi_lo(float x, float y, uint32_t *lo) {     // exact split of two floats into fp16 hi, lo pairs
    const __half hx = __float2half_rn(x), hy = __float2half_rn(y);
    const __half2 h = __halves2half2(hx, hy);
    const __half2 l = __floats2half2_rn(x - __half2float(hx), y - __half2float(hy));
    *lo = *reinterpret_cast<const uint32_t *>(&l);
    return *reinterpret_cast<const uint32_t *>(&h);
}

template <int D, int G, int NW>
__global__ void __launch_bounds__(NW * 32)
paged_flash_mma_kernel(VxAttnArgs a) {
    constexpr int KS = D / 16;                    // K=16 steps of the score product = 16-row tiles of the output product
    constexpr int ROW_B = D * 2;                  // bytes of one token's head slice
    constexpr int TILE_B = ATT_BS * ROW_B;        // one K (or V) page tile
    constexpr int STAGE_B = 2 * TILE_B;           // K tile then V tile
    constexpr int CPL = STAGE_B / 16 / 32;        // 16-byte chunks per lane and page
    extern __shared__ __align__(128) unsigned char att_smem[];
    vx_pdl_wait();
    vx_pdl_trigger();

    const int wi = blockIdx.x;
    if (wi >= *a.n_work_dev) return;
    const int4 item = a.work[wi];
    const int row = item.x, first_page = item.y, n_pages = item.z;
    const int kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int kv_start = a.row_kv_start ? a.row_kv_start[row] : 0, kv_len = a.row_kv_len[row];
    const int32_t *table = a.tables[a.row_slot[row]];
    const size_t hs = (size_t)a.n_kv_heads * D;
    const __half *pool = (const __half *)a.pool;
    const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(att_smem) + warp * 2 * STAGE_B;

    // Q^T fragments: lane (g, c) holds head g (zero beyond the group), d = 16 ks + 2c, +1 and + 8, +9, as hi and lo halves
    uint32_t qh[KS][2], ql[KS][2];
    {
        const float *qp = a.q + (size_t)row * a.q_row_stride + (size_t)(kvh * G + (g < G ? g : 0)) * D;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            float2 v0 = make_float2(0.f, 0.f), v1 = v0;
            if (g < G) { v0 = *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * c); v1 = *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * c + 8); }
            qh[ks][0] = pack_hi_lo(v0.x, v0.y, &ql[ks][0]);
            qh[ks][1] = pack_hi_lo(v1.x, v1.y, &ql[ks][1]);
        }
    }
    float acc[KS][4];
#pragma unroll
    for (int i = 0; i < KS; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};     // heads 2c, 2c+1; l over this lane's tokens only

    // cp.async plan of one page: chunk (t, cc) of the K and of the V tile, t = tl + RPI * jj.  Everything but the block base
    // is fixed per lane: global offset g_off + jj * g_step (+ the V tile), shared offset from t and the swizzled chunk.
    constexpr int CPR = D / 8;                    // 16-byte chunks per token row
    constexpr int RPI = 32 / CPR;                 // token rows covered by one warp-wide copy
    static_assert(CPL == 2 * (ATT_BS / RPI), "copy plan");
    const int tl = lane / CPR, cc = lane % CPR;
    const size_t g_off = (size_t)kvh * D + (size_t)tl * hs + cc * 8, g_step = (size_t)RPI * hs, g_v = (size_t)ATT_BS * hs;
    auto issue = [&](int page, int stage) {       // stages the K and V tiles of one page (all lanes)
        const int blk = table[page];
        const __half *kb = pool + (size_t)blk * 2 * ATT_BS * hs + g_off;
        const uint32_t sb = stage0 + stage * STAGE_B;
#pragma unroll
        for (int jj = 0; jj < ATT_BS / RPI; jj++) {
            const int t = tl + RPI * jj;
            const uint32_t so = sb + t * ROW_B + ((cc ^ (t & 7)) << 4);
            cp_async_16(so, kb + jj * g_step);
            cp_async_16(so + TILE_B, kb + jj * g_step + g_v);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    const int last_page = first_page + n_pages;
    int page = first_page + warp, stage = 0;
    if (page < last_page) issue(page, 0);
    for (; page < last_page; page += NW, stage ^= 1) {
        if (page + NW < last_page) { issue(page + NW, stage ^ 1); asm volatile("cp.async.wait_group 1;\n" ::); }
        else asm volatile("cp.async.wait_group 0;\n" ::);
        __syncwarp();
        const uint32_t kb_s = stage0 + stage * STAGE_B, vb_s = kb_s + TILE_B;

        // scores, transposed: rows = tokens g and g + 8, columns = heads 2c and 2c + 1
        float st[4] = {0.f, 0.f, 0.f, 0.f};
        {
            float st2[4] = {0.f, 0.f, 0.f, 0.f};                               // two accumulation chains halve the MMA latency chain
            const int mj = lane >> 3, r = (lane & 7) + 8 * (mj & 1);           // ldmatrix row address of this lane
            const uint32_t krow = kb_s + r * ROW_B;
            const int sw = r & 7, co = mj >> 1;
#pragma unroll
            for (int ks = 0; ks < KS; ks += 2) {
                uint32_t ka[4], kc[4];
                ldsm_x4(ka, krow + (((2 * ks + co) ^ sw) << 4));
                ldsm_x4(kc, krow + (((2 * ks + 2 + co) ^ sw) << 4));
                mma_16816(st, ka, qh[ks][0], qh[ks][1]);
                mma_16816(st2, kc, qh[ks + 1][0], qh[ks + 1][1]);
                mma_16816(st, ka, ql[ks][0], ql[ks][1]);
                mma_16816(st2, kc, ql[ks + 1][0], ql[ks + 1][1]);
            }
#pragma unroll
            for (int i = 0; i < 4; i++) st[i] += st2[i];
        }
        const int pos0 = page * ATT_BS + g, pos1 = pos0 + 8;
        const bool ok0 = pos0 >= kv_start && pos0 < kv_len, ok1 = pos1 >= kv_start && pos1 < kv_len;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float v = st[i] * a.scale;
            if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
            st[i] = ((i < 2) ? ok0 : ok1) ? v : -INFINITY;
        }
        float p[4];
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            float mx = fmaxf(st[hh], st[2 + hh]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[hh], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;            // page fully outside the window: p = 0, no rescale
            const float corr = __expf(m_run[hh] - m_use);                    // exp(-inf) = 0 on the first page
            p[hh] = st[hh] == -INFINITY ? 0.f : __expf(st[hh] - m_use);
            p[2 + hh] = st[2 + hh] == -INFINITY ? 0.f : __expf(st[2 + hh] - m_use);
            l_run[hh] = l_run[hh] * corr + p[hh] + p[2 + hh];
#pragma unroll
            for (int i = 0; i < KS; i++) { acc[i][hh] *= corr; acc[i][2 + hh] *= corr; }
            m_run[hh] = m_new;
        }
        // P^T as the B operand: lane (g, c) needs head g at tokens 2c, 2c+1 (b0) and 2c+8, 2c+9 (b1); in the score layout
        // token t, head h sits in lane (t & 7, h >> 1), register 2 (t >> 3) + (h & 1)
        uint32_t xl0, xl1;
        const uint32_t xh0 = pack_hi_lo(p[0], p[2], &xl0), xh1 = pack_hi_lo(p[1], p[3], &xl1);   // {token g, token g+8} of head 2c / 2c+1
        const int srcA = (2 * c) * 4 + (g >> 1), srcB = (2 * c + 1) * 4 + (g >> 1);
        const bool odd = g & 1;
        uint32_t ah0 = __shfl_sync(0xffffffffu, xh0, srcA), ah1 = __shfl_sync(0xffffffffu, xh1, srcA);
        uint32_t bh0 = __shfl_sync(0xffffffffu, xh0, srcB), bh1 = __shfl_sync(0xffffffffu, xh1, srcB);
        uint32_t al0 = __shfl_sync(0xffffffffu, xl0, srcA), al1 = __shfl_sync(0xffffffffu, xl1, srcA);
        uint32_t bl0 = __shfl_sync(0xffffffffu, xl0, srcB), bl1 = __shfl_sync(0xffffffffu, xl1, srcB);
        const uint32_t ya_h = odd ? ah1 : ah0, yb_h = odd ? bh1 : bh0, ya_l = odd ? al1 : al0, yb_l = odd ? bl1 : bl0;
        const uint32_t ph0 = __byte_perm(ya_h, yb_h, 0x5410), ph1 = __byte_perm(ya_h, yb_h, 0x7632);
        const uint32_t pl0 = __byte_perm(ya_l, yb_l, 0x5410), pl1 = __byte_perm(ya_l, yb_l, 0x7632);
        {
            const int mj = lane >> 3, t = (lane & 7) + 8 * (mj >> 1);          // token row read by this lane
#pragma unroll
            for (int mt = 0; mt < KS; mt++) {
                uint32_t va[4];
                ldsm_x4_t(va, vb_s + t * ROW_B + (((2 * mt + (mj & 1)) ^ (t & 7)) << 4));
                mma_16816(acc[mt], va, ph0, ph1);
                mma_16816(acc[mt], va, pl0, pl1);
            }
        }
        __syncwarp();                              // every lane is done with this stage before it is refilled
    }

    // this warp's partial result to shared memory (reusing the staging area), then the same 4-way merge as above
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
    }
    __syncthreads();
    float *sm_acc = reinterpret_cast<float *>(att_smem);                      // [warp][G][D]
    float *sm_m = sm_acc + NW * G * D, *sm_l = sm_m + NW * G;    // [warp][G]
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int h = 2 * c + hh;
        if (h < G) {
            if (g == 0) { sm_m[warp * G + h] = m_run[hh]; sm_l[warp * G + h] = l_run[hh]; }
#pragma unroll
            for (int mt = 0; mt < KS; mt++) {
                sm_acc[(warp * G + h) * D + 16 * mt + g] = acc[mt][hh];
                sm_acc[(warp * G + h) * D + 16 * mt + g + 8] = acc[mt][2 + hh];
            }
        }
    }
    __syncthreads();
    const bool single = (a.row_work_start[row + 1] - a.row_work_start[row]) == 1;
    float bound = 0.f;
    for (int idx = threadIdx.x; idx < G * D; idx += NW * 32) {
        const int gi = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, sm_m[w * G + gi]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float f = sm_m[w * G + gi] == -INFINITY ? 0.f : __expf(sm_m[w * G + gi] - M);
            L = fmaf(sm_l[w * G + gi], f, L); O = fmaf(sm_acc[(w * G + gi) * D + d], f, O);
        }
        const int h = kvh * G + gi;
        const float o = L > 0.f ? O / L : 0.f;
        bound = fmaxf(bound, fabsf(o));
        if (single) {
            a.out[(size_t)row * a.out_row_stride + (size_t)h * D + d] = o;
        } else {
            float *part = a.partials + ((size_t)wi * a.n_q_heads + h) * (D + 2);
            part[d] = O;
            if (d == 0) { part[D] = M; part[D + 1] = L; }
        }
    }
    if (a.row_bound) vx_raise_row_bound(a.row_bound + row, bound);
}

// rows cut into more than one chunk: out = sum_c O_c e^{m_c-M} / sum_c l_c e^{m_c-M}
__global__ void paged_merge_kernel(VxAttnArgs a) {
    const int row = blockIdx.y, h = blockIdx.x, D = a.head_dim;
    const int w0 = a.row_work_start[row], n = a.row_work_start[row + 1] - w0;
    if (n <= 1) return;
    float M = -INFINITY;
    for (int c = 0; c < n; c++) M = fmaxf(M, a.partials[((size_t)(w0 + c) * a.n_q_heads + h) * (D + 2) + D]);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.f, O = 0.f;
        for (int c = 0; c < n; c++) {
            const float *part = a.partials + ((size_t)(w0 + c) * a.n_q_heads + h) * (D + 2);
            const float f = part[D] == -INFINITY ? 0.f : __expf(part[D] - M);
            L = fmaf(part[D + 1], f, L); O = fmaf(part[d], f, O);
        }
        a.out[(size_t)row * a.out_row_stride + (size_t)h * D + d] = L > 0.f ? O / L : 0.f;
    }
}

static int g_attn_mma = 1;     // grouped-query shapes use the tensor-core kernel (0 = the CUDA-core kernel, for comparison)

// ------------------------------------------------------------------ multi-row (chunked prefill) attention over the paged cache
// A prompt chunk that does not start at position 0 attends over pages that earlier chunks wrote (runtime/decode.go:1033-1060
// walks the prompt token by token through the same cache).  Running it through the decode kernels re-reads the whole cache
// once per query row; here a CTA owns 64 consecutive rows of one sequence and one query head (a warp 16 rows), walks the
// pages once in tiles of 64 tokens staged in shared memory, and does both products on mma.sync.m16n8k16 with the query
// rows as M:   S[16 x 64] = Q . K^T   (K via ldmatrix),   O[16 x D] += P . V   (V via ldmatrix.trans, P straight from the
// score accumulators).  q and p are exact fp16 hi + lo pairs, accumulation is float32; masks are per row
// (kv_start <= t < kv_len), so causal order, sliding windows and ragged tails need no special cases.
constexpr int PF_ROWS = 64;           // query rows per CTA
constexpr int PF_TOK = 64;            // KV tokens per tile (four pages)

template <int D>
__global__ void __launch_bounds__(128)
paged_prefill_mma_kernel(VxAttnArgs a, int row0, int n_rows) {
    constexpr int KS = D / 16, ND = D / 8, ROW_B = D * 2, TILE_B = PF_TOK * ROW_B, STAGE_B = 2 * TILE_B;
    constexpr int CPR = D / 8;                                // 16-byte chunks per token row
    extern __shared__ __align__(128) unsigned char pf_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int h = blockIdx.y, kvh = h / (a.n_q_heads / a.n_kv_heads);
    const int rt0 = row0 + blockIdx.x * PF_ROWS, rt1 = min(row0 + n_rows, rt0 + PF_ROWS);      // this CTA's rows
    const int rA = rt0 + warp * 16 + g, rB = rA + 8;                                            // this lane's two rows
    const bool vA = rA < rt1, vB = rB < rt1;
    const int32_t *table = a.tables[a.row_slot[rt0]];
    const size_t hs = (size_t)a.n_kv_heads * D;
    const __half *pool = (const __half *)a.pool;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(pf_smem);

    // the tile's token range: from the smallest window start to the largest length among its rows (rows are in position order)
    const int t_begin = (a.row_kv_start ? a.row_kv_start[rt0] : 0) / ATT_BS * ATT_BS;
    const int t_end = a.row_kv_len[rt1 - 1];
    const int lenA = vA ? a.row_kv_len[rA] : 0, lenB = vB ? a.row_kv_len[rB] : 0;
    const int stA = (vA && a.row_kv_start) ? a.row_kv_start[rA] : 0, stB = (vB && a.row_kv_start) ? a.row_kv_start[rB] : 0;

    uint32_t qh[KS][4], ql[KS][4];
    {
        const float *qa = a.q + (size_t)(vA ? rA : rt0) * a.q_row_stride + (size_t)h * D;
        const float *qb = a.q + (size_t)(vB ? rB : rt0) * a.q_row_stride + (size_t)h * D;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const float2 a0 = *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * c), a2 = *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * c + 8);
            const float2 b0 = *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * c), b2 = *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * c + 8);
            qh[ks][0] = pack_hi_lo(a0.x, a0.y, &ql[ks][0]); qh[ks][1] = pack_hi_lo(b0.x, b0.y, &ql[ks][1]);
            qh[ks][2] = pack_hi_lo(a2.x, a2.y, &ql[ks][2]); qh[ks][3] = pack_hi_lo(b2.x, b2.y, &ql[ks][3]);
        }
    }
    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;        // l over this lane's columns only

    auto issue = [&](int t0, int stage) {           // stages tokens t0 .. t0+63 (four pages) of K and V; all 128 threads
        const uint32_t sb = sbase + stage * STAGE_B;
#pragma unroll
        for (int j = 0; j < 2 * PF_TOK * CPR / 128; j++) {
            const int ci = threadIdx.x + 128 * j;
            const int isv = ci / (PF_TOK * CPR), r = ci % (PF_TOK * CPR), t = r / CPR, cc = r % CPR;
            const int tok = t0 + t;
            const uint32_t so = isv * TILE_B + t * ROW_B + ((cc ^ (t & 7)) << 4);
            if (tok < t_end) {
                const int blk = table[tok / ATT_BS];
                const __half *src = pool + (size_t)blk * 2 * ATT_BS * hs + (size_t)isv * ATT_BS * hs + (size_t)(tok % ATT_BS) * hs + (size_t)kvh * D + cc * 8;
                cp_async_16(sb + so, src);
            } else {
                // beyond the last attended token: zeros, so that a masked probability of 0 never meets stale bytes that read as NaN
                *reinterpret_cast<uint4 *>(pf_smem + stage * STAGE_B + so) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    int stage = 0;
    if (t_begin < t_end) issue(t_begin, 0);
    for (int t0 = t_begin; t0 < t_end; t0 += PF_TOK, stage ^= 1) {
        if (t0 + PF_TOK < t_end) { issue(t0 + PF_TOK, stage ^ 1); asm volatile("cp.async.wait_group 1;\n" ::); }
        else asm volatile("cp.async.wait_group 0;\n" ::);
        __syncthreads();
        const uint32_t kb_s = sbase + stage * STAGE_B, vb_s = kb_s + TILE_B;
        float st[PF_TOK / 8][4];
#pragma unroll
        for (int j = 0; j < PF_TOK / 8; j++) { st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f; }
        {
            const int mj = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
#pragma unroll
                for (int j = 0; j < PF_TOK / 8; j += 2) {        // two token tiles per ldmatrix.x4
                    const int t = 8 * (j + (mj >> 1)) + (lane & 7);
                    uint32_t kf[4];
                    ldsm_x4(kf, kb_s + t * ROW_B + (((2 * ks + (mj & 1)) ^ (t & 7)) << 4));
                    mma_16816(st[j], qh[ks], kf[0], kf[1]); mma_16816(st[j], ql[ks], kf[0], kf[1]);
                    mma_16816(st[j + 1], qh[ks], kf[2], kf[3]); mma_16816(st[j + 1], ql[ks], kf[2], kf[3]);
                }
        }
        // scale, soft-cap, masks; running maxima per row (this lane: columns 8j + 2c, +1 of rows A and B)
        float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
        for (int j = 0; j < PF_TOK / 8; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int tok = t0 + 8 * j + 2 * c + e;
                float va = st[j][e] * a.scale, vb = st[j][2 + e] * a.scale;
                if (a.softcap > 0.f) { va = a.softcap * tanhf(va / a.softcap); vb = a.softcap * tanhf(vb / a.softcap); }
                va = (tok >= stA && tok < lenA) ? va : -INFINITY;
                vb = (tok >= stB && tok < lenB) ? vb : -INFINITY;
                st[j][e] = va; st[j][2 + e] = vb;
                mxA = fmaxf(mxA, va); mxB = fmaxf(mxB, vb);
            }
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
        const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
        const float uA = nA == -INFINITY ? 0.f : nA, uB = nB == -INFINITY ? 0.f : nB;
        const float cA = __expf(mA - uA), cB = __expf(mB - uB);
        mA = nA; mB = nB; lA *= cA; lB *= cB;
#pragma unroll
        for (int i = 0; i < ND; i++) { acc[i][0] *= cA; acc[i][1] *= cA; acc[i][2] *= cB; acc[i][3] *= cB; }
        // P as the A operand of the second product, K=16 tokens per step: registers of score tiles 2kt and 2kt+1
#pragma unroll
        for (int kt = 0; kt < PF_TOK / 16; kt++) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int j = 2 * kt + half;
                const float p0 = st[j][0] == -INFINITY ? 0.f : __expf(st[j][0] - uA), p1 = st[j][1] == -INFINITY ? 0.f : __expf(st[j][1] - uA);
                const float p2 = st[j][2] == -INFINITY ? 0.f : __expf(st[j][2] - uB), p3 = st[j][3] == -INFINITY ? 0.f : __expf(st[j][3] - uB);
                lA += p0 + p1; lB += p2 + p3;
                ph[2 * half] = pack_hi_lo(p0, p1, &pl[2 * half]);
                ph[2 * half + 1] = pack_hi_lo(p2, p3, &pl[2 * half + 1]);
            }
            const int mj = lane >> 3, t = 16 * kt + 8 * (mj & 1) + (lane & 7);
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {             // two 8-wide d tiles per ldmatrix.x4.trans
                uint32_t vf[4];
                ldsm_x4_t(vf, vb_s + t * ROW_B + (((nd + (mj >> 1)) ^ (t & 7)) << 4));
                mma_16816(acc[nd], ph, vf[0], vf[1]); mma_16816(acc[nd], pl, vf[0], vf[1]);
                mma_16816(acc[nd + 1], ph, vf[2], vf[3]); mma_16816(acc[nd + 1], pl, vf[2], vf[3]);
            }
        }
        __syncthreads();                             // the stage is refilled two iterations later by all threads
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    const float iA = lA > 0.f ? 1.0f / lA : 0.f, iB = lB > 0.f ? 1.0f / lB : 0.f;
#pragma unroll
    for (int nd = 0; nd < ND; nd++) {
        if (vA) *reinterpret_cast<float2 *>(a.out + (size_t)rA * a.out_row_stride + (size_t)h * D + 8 * nd + 2 * c) = make_float2(acc[nd][0] * iA, acc[nd][1] * iA);
        if (vB) *reinterpret_cast<float2 *>(a.out + (size_t)rB * a.out_row_stride + (size_t)h * D + 8 * nd + 2 * c) = make_float2(acc[nd][2] * iB, acc[nd][3] * iB);
    }
}

// The first chunk of a prompt attends causally over its own freshly projected float32 K and V (runtime/block.go:891-895),
// not over the fp16 cache.  Same tiling as above with the tiles built from the float32 rows: K and V are split into exact
// fp16 hi + lo pairs on their way into shared memory and both products take three terms (hi*hi, lo*hi, hi*lo; the dropped
// lo*lo term is 2^-22 relative), so the result matches the float32 arithmetic to rounding.
template <int D>
__global__ void __launch_bounds__(128)
prefill_f32_mma_kernel(const float *__restrict__ q, int q_ld, const float *__restrict__ k, const float *__restrict__ v, long kv_ld,
                       float *__restrict__ out, int out_ld, int n_rows, int n_q_heads, int n_kv_heads, float scale, float softcap) {
    constexpr int KS = D / 16, ND = D / 8, ROW_B = D * 2, TILE_B = PF_TOK * ROW_B;
    constexpr int CPR = D / 8;
    extern __shared__ __align__(128) unsigned char pf_smem[];           // [K_hi | K_lo | V_hi | V_lo], one 64-token tile each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int h = blockIdx.y, kvh = h / (n_q_heads / n_kv_heads);
    const int rt0 = blockIdx.x * PF_ROWS, rt1 = min(n_rows, rt0 + PF_ROWS);
    const int rA = rt0 + warp * 16 + g, rB = rA + 8;
    const bool vA = rA < rt1, vB = rB < rt1;
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(pf_smem);
    const int t_end = rt1;                                                // causal: the last row sees tokens 0 .. rt1-1
    const int lenA = vA ? rA + 1 : 0, lenB = vB ? rB + 1 : 0;

    uint32_t qh[KS][4], ql[KS][4];
    {
        const float *qa = q + (size_t)(vA ? rA : rt0) * q_ld + (size_t)h * D, *qb = q + (size_t)(vB ? rB : rt0) * q_ld + (size_t)h * D;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const float2 a0 = *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * c), a2 = *reinterpret_cast<const float2 *>(qa + 16 * ks + 2 * c + 8);
            const float2 b0 = *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * c), b2 = *reinterpret_cast<const float2 *>(qb + 16 * ks + 2 * c + 8);
            qh[ks][0] = pack_hi_lo(a0.x, a0.y, &ql[ks][0]); qh[ks][1] = pack_hi_lo(b0.x, b0.y, &ql[ks][1]);
            qh[ks][2] = pack_hi_lo(a2.x, a2.y, &ql[ks][2]); qh[ks][3] = pack_hi_lo(b2.x, b2.y, &ql[ks][3]);
        }
    }
    float acc[ND][4];
#pragma unroll
    for (int i = 0; i < ND; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;

    for (int t0 = 0; t0 < t_end; t0 += PF_TOK) {
        // float32 rows -> fp16 hi / lo tiles (16-byte chunks of 8 dims, XOR-swizzled like the paged tiles)
        for (int ci = threadIdx.x; ci < 2 * PF_TOK * CPR; ci += 128) {
            const int isv = ci / (PF_TOK * CPR), r = ci % (PF_TOK * CPR), t = r / CPR, cc = r % CPR;
            const int tok = t0 + t;
            uint4 hi4 = make_uint4(0, 0, 0, 0), lo4 = hi4;
            if (tok < t_end) {
                const float *src = (isv ? v : k) + (size_t)tok * kv_ld + (size_t)kvh * D + cc * 8;
                const float4 x0 = *reinterpret_cast<const float4 *>(src), x1 = *reinterpret_cast<const float4 *>(src + 4);
                hi4.x = pack_hi_lo(x0.x, x0.y, &lo4.x); hi4.y = pack_hi_lo(x0.z, x0.w, &lo4.y);
                hi4.z = pack_hi_lo(x1.x, x1.y, &lo4.z); hi4.w = pack_hi_lo(x1.z, x1.w, &lo4.w);
            }
            const uint32_t so = isv * 2 * TILE_B + t * ROW_B + ((cc ^ (t & 7)) << 4);
            *reinterpret_cast<uint4 *>(pf_smem + so) = hi4;
            *reinterpret_cast<uint4 *>(pf_smem + so + TILE_B) = lo4;
        }
        __syncthreads();
        const uint32_t kh_s = sbase, kl_s = sbase + TILE_B, vh_s = sbase + 2 * TILE_B, vl_s = sbase + 3 * TILE_B;
        float st[PF_TOK / 8][4];
#pragma unroll
        for (int j = 0; j < PF_TOK / 8; j++) { st[j][0] = st[j][1] = st[j][2] = st[j][3] = 0.f; }
        {
            const int mj = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < KS; ks++)
#pragma unroll
                for (int j = 0; j < PF_TOK / 8; j += 2) {
                    const int t = 8 * (j + (mj >> 1)) + (lane & 7);
                    const uint32_t off = t * ROW_B + (((2 * ks + (mj & 1)) ^ (t & 7)) << 4);
                    uint32_t kf[4], kg[4];
                    ldsm_x4(kf, kh_s + off); ldsm_x4(kg, kl_s + off);
                    mma_16816(st[j], qh[ks], kf[0], kf[1]); mma_16816(st[j], ql[ks], kf[0], kf[1]); mma_16816(st[j], qh[ks], kg[0], kg[1]);
                    mma_16816(st[j + 1], qh[ks], kf[2], kf[3]); mma_16816(st[j + 1], ql[ks], kf[2], kf[3]); mma_16816(st[j + 1], qh[ks], kg[2], kg[3]);
                }
        }
        float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
        for (int j = 0; j < PF_TOK / 8; j++)
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const int tok = t0 + 8 * j + 2 * c + e;
                float va = st[j][e] * scale, vb = st[j][2 + e] * scale;
                if (softcap > 0.f) { va = softcap * tanhf(va / softcap); vb = softcap * tanhf(vb / softcap); }
                va = tok < lenA ? va : -INFINITY; vb = tok < lenB ? vb : -INFINITY;
                st[j][e] = va; st[j][2 + e] = vb;
                mxA = fmaxf(mxA, va); mxB = fmaxf(mxB, vb);
            }
        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1)); mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1)); mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
        const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
        const float uA = nA == -INFINITY ? 0.f : nA, uB = nB == -INFINITY ? 0.f : nB;
        const float cA = __expf(mA - uA), cB = __expf(mB - uB);
        mA = nA; mB = nB; lA *= cA; lB *= cB;
#pragma unroll
        for (int i = 0; i < ND; i++) { acc[i][0] *= cA; acc[i][1] *= cA; acc[i][2] *= cB; acc[i][3] *= cB; }
#pragma unroll
        for (int kt = 0; kt < PF_TOK / 16; kt++) {
            uint32_t ph[4], pl[4];
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int j = 2 * kt + half;
                const float p0 = st[j][0] == -INFINITY ? 0.f : __expf(st[j][0] - uA), p1 = st[j][1] == -INFINITY ? 0.f : __expf(st[j][1] - uA);
                const float p2 = st[j][2] == -INFINITY ? 0.f : __expf(st[j][2] - uB), p3 = st[j][3] == -INFINITY ? 0.f : __expf(st[j][3] - uB);
                lA += p0 + p1; lB += p2 + p3;
                ph[2 * half] = pack_hi_lo(p0, p1, &pl[2 * half]);
                ph[2 * half + 1] = pack_hi_lo(p2, p3, &pl[2 * half + 1]);
            }
            const int mj = lane >> 3, t = 16 * kt + 8 * (mj & 1) + (lane & 7);
#pragma unroll
            for (int nd = 0; nd < ND; nd += 2) {
                const uint32_t off = t * ROW_B + (((nd + (mj >> 1)) ^ (t & 7)) << 4);
                uint32_t vf[4], vg[4];
                ldsm_x4_t(vf, vh_s + off); ldsm_x4_t(vg, vl_s + off);
                mma_16816(acc[nd], ph, vf[0], vf[1]); mma_16816(acc[nd], pl, vf[0], vf[1]); mma_16816(acc[nd], ph, vg[0], vg[1]);
                mma_16816(acc[nd + 1], ph, vf[2], vf[3]); mma_16816(acc[nd + 1], pl, vf[2], vf[3]); mma_16816(acc[nd + 1], ph, vg[2], vg[3]);
            }
        }
        __syncthreads();
    }
    lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    const float iA = lA > 0.f ? 1.0f / lA : 0.f, iB = lB > 0.f ? 1.0f / lB : 0.f;
#pragma unroll
    for (int nd = 0; nd < ND; nd++) {
        if (vA) *reinterpret_cast<float2 *>(out + (size_t)rA * out_ld + (size_t)h * D + 8 * nd + 2 * c) = make_float2(acc[nd][0] * iA, acc[nd][1] * iA);
        if (vB) *reinterpret_cast<float2 *>(out + (size_t)rB * out_ld + (size_t)h * D + 8 * nd + 2 * c) = make_float2(acc[nd][2] * iB, acc[nd][3] * iB);
    }
}

// causal attention of n_rows query rows over their own float32 K / V rows (row stride kv_ld floats, kv head h at h * D);
// VX_E_UNSUPPORTED when the shape has no such kernel
int vxp_prefill_f32(vx_ctx *c, const float *q, int q_ld, const float *k, const float *v, long kv_ld, float *out, int out_ld, int n_rows,
                    int hq, int hkv, int d, float scale, float softcap) {
    if (!((d == 64 || d == 128) && n_rows >= 16 && q_ld % 4 == 0 && kv_ld % 4 == 0 && out_ld % 2 == 0 && hkv > 0 && hq % hkv == 0)) return VX_E_UNSUPPORTED;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) != 0) return VX_E_UNSUPPORTED;
    dim3 grid(ceil_div(n_rows, PF_ROWS), hq);
    const int smem = 4 * PF_TOK * d * 2;
    if (d == 64) {
        static VxPerDevice attr;
        VX_CUDA(c, attr.max_dynamic_smem(c, prefill_f32_mma_kernel<64>, smem));
        prefill_f32_mma_kernel<64><<<grid, 128, smem, c->stream>>>(q, q_ld, k, v, kv_ld, out, out_ld, n_rows, hq, hkv, scale, softcap);
    } else {
        static VxPerDevice attr;
        VX_CUDA(c, attr.max_dynamic_smem(c, prefill_f32_mma_kernel<128>, smem));
        prefill_f32_mma_kernel<128><<<grid, 128, smem, c->stream>>>(q, q_ld, k, v, kv_ld, out, out_ld, n_rows, hq, hkv, scale, softcap);
    }
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// rows [row0, row0 + n_rows) belong to one sequence, in position order; f16 pool, 16-token pages, head_dim 64 or 128
int vxp_prefill_rows(vx_ctx *c, const VxAttnArgs &a, int row0, int n_rows) {
    const int D = a.head_dim;
    if (!(a.pool_is_f16 && a.block_size == ATT_BS && (D == 64 || D == 128) && a.q_row_stride % 2 == 0 && a.out_row_stride % 2 == 0 && n_rows > 0))
        return VX_E_UNSUPPORTED;
    dim3 grid(ceil_div(n_rows, PF_ROWS), a.n_q_heads);
    const int smem = 2 * 2 * PF_TOK * D * 2;
    if (D == 64) {
        static VxPerDevice attr;
        VX_CUDA(c, attr.max_dynamic_smem(c, paged_prefill_mma_kernel<64>, smem));
        paged_prefill_mma_kernel<64><<<grid, 128, smem, c->stream>>>(a, row0, n_rows);
    } else {
        static VxPerDevice attr;
        VX_CUDA(c, attr.max_dynamic_smem(c, paged_prefill_mma_kernel<128>, smem));
        paged_prefill_mma_kernel<128><<<grid, 128, smem, c->stream>>>(a, row0, n_rows);
    }
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// Merge of the split-K chunks fused with the fp16 hi/lo split that feeds the output projection: one CTA per query row.
// Phase 1, one thread per head: the chunk maxima and weights e^{m_c - M} / L into shared memory.  Phase 2, four consecutive
// head dimensions per thread: the weighted sum of the chunk outputs with independent loads (rows written directly by a
// single-chunk CTA are read back instead), then the row maximum, the power-of-two scale and the split store.  Replaces
// paged_merge_kernel + split_rows_kernel; nothing but the projection reads the attention output on that path.
template <int NC>
__global__ void __launch_bounds__(VX_ROW_THREADS) paged_merge_split_kernel(VxAttnArgs a, VxSplit s, int cols, int n_max) {
    extern __shared__ float fw[];                  // [n_q_heads][n_max] normalised chunk weights, then [n_q_heads][n_max] chunk sums
    __shared__ float red[32];
    vx_pdl_wait();             // (chained launch: the attention kernel before this one has completed)
    vx_pdl_trigger();          // the projection that follows may become resident and fetch its first weights now
    const int row = blockIdx.x, D = a.head_dim, Hq = a.n_q_heads;
    const int w0 = a.row_work_start[row], n = a.row_work_start[row + 1] - w0;
    if (n > 1) {
        // chunk maxima and sums of all heads in one coalesced sweep, then one thread per head turns them into weights
        float *ms = fw, *ls = fw + Hq * n_max;
        for (int i = threadIdx.x; i < Hq * n; i += VX_ROW_THREADS) {
            const int c = i / Hq, h = i % Hq;
            const float *p0 = a.partials + ((size_t)(w0 + c) * Hq + h) * (D + 2) + D;
            ms[h * n_max + c] = p0[0]; ls[h * n_max + c] = p0[1];
        }
        __syncthreads();
        for (int h = threadIdx.x; h < Hq; h += VX_ROW_THREADS) {
            float M = -INFINITY;
            for (int c = 0; c < n; c++) M = fmaxf(M, ms[h * n_max + c]);
            float L = 0.f;
            for (int c = 0; c < n; c++) {
                const float mc = ms[h * n_max + c];
                const float f = mc == -INFINITY ? 0.f : __expf(mc - M);
                ms[h * n_max + c] = f;
                L = fmaf(ls[h * n_max + c], f, L);
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            for (int c = 0; c < n; c++) fw[h * n_max + c] = ms[h * n_max + c] * inv;
        }
        __syncthreads();
    }
    float4 v[NC];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int k0 = (j * VX_ROW_THREADS + threadIdx.x) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k0 < cols) {
            if (n > 1) {
                const int h = k0 / D, d = k0 % D;
                const float *pp = a.partials + ((size_t)w0 * Hq + h) * (D + 2) + d;
                const size_t cs = (size_t)Hq * (D + 2);
                const float *f = fw + h * n_max;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int c = 0; c < n; c++) {
                    const float2 x0 = *reinterpret_cast<const float2 *>(pp + c * cs), x1 = *reinterpret_cast<const float2 *>(pp + c * cs + 2);
                    const float fc = f[c];
                    acc.x = fmaf(x0.x, fc, acc.x); acc.y = fmaf(x0.y, fc, acc.y); acc.z = fmaf(x1.x, fc, acc.z); acc.w = fmaf(x1.y, fc, acc.w);
                }
                v[j] = acc;
            } else {
                v[j] = *reinterpret_cast<const float4 *>(a.out + (size_t)row * a.out_row_stride + k0);
            }
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
    }
    amax = block_max(amax, red);
    float sc, inv;
    vx_row_scale(amax, sc, inv);
    if (threadIdx.x == 0) s.scale[row] = sc;
    __half *hi = s.hi + (size_t)row * s.k_pad, *lo = s.lo + (size_t)row * s.k_pad;
    float *bs = s.bsum + (size_t)row * (s.k_pad / 32);
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int k0 = (j * VX_ROW_THREADS + threadIdx.x) * 4;
        if (k0 < s.k_pad) {
            const float t[4] = {v[j].x * inv, v[j].y * inv, v[j].z * inv, v[j].w * inv};
            vx_split_store4(t, hi, lo, bs, k0);
        }
    }
}

// The same merge + split with the row scale taken from a.row_bound instead of a row-wide maximum: nothing ties the CTAs of
// a row together any more, so a row is spread over cols / 1024 CTAs of 256 threads (four consecutive head dimensions per
// thread, whole heads per CTA), four times as many SMs work on the launch and every CTA's chain of dependent loads is a
// quarter as wide.  The bound is at least the row's largest magnitude and rarely more than a small factor above it: the
// fp16 pair keeps 22 - log2(factor) significant bits.
constexpr int MS_THREADS = 256, MS_COLS = MS_THREADS * 4;
__global__ void __launch_bounds__(MS_THREADS) paged_merge_split_heads_kernel(VxAttnArgs a, VxSplit s, int n_max) {
    extern __shared__ float fw[];                  // [heads of this CTA][n_max] normalised chunk weights, then the chunk sums
    vx_pdl_wait();             // (chained launch: the attention kernel before this one has completed)
    vx_pdl_trigger();          // the projection that follows may become resident and fetch its first weights now
    const int row = blockIdx.x, D = a.head_dim, Hq = a.n_q_heads;
    const int col0 = blockIdx.y * MS_COLS, h0 = col0 / D, nh = MS_COLS / D;
    const int w0 = a.row_work_start[row], n = a.row_work_start[row + 1] - w0;
    float sc, inv;
    vx_row_scale(__uint_as_float(a.row_bound[row]), sc, inv);
    if (blockIdx.y == 0 && threadIdx.x == 0) s.scale[row] = sc;
    if (n > 1) {
        float *ms = fw, *ls = fw + nh * n_max;
        for (int i = threadIdx.x; i < nh * n; i += MS_THREADS) {
            const int c = i / nh, h = i % nh;
            const float *p0 = a.partials + ((size_t)(w0 + c) * Hq + h0 + h) * (D + 2) + D;
            ms[h * n_max + c] = p0[0]; ls[h * n_max + c] = p0[1];
        }
        __syncthreads();
        for (int h = threadIdx.x; h < nh; h += MS_THREADS) {
            float M = -INFINITY;
            for (int c = 0; c < n; c++) M = fmaxf(M, ms[h * n_max + c]);
            float L = 0.f;
            for (int c = 0; c < n; c++) {
                const float mc = ms[h * n_max + c];
                const float f = mc == -INFINITY ? 0.f : __expf(mc - M);
                ms[h * n_max + c] = f;
                L = fmaf(ls[h * n_max + c], f, L);
            }
            const float il = L > 0.f ? 1.0f / L : 0.f;
            for (int c = 0; c < n; c++) fw[h * n_max + c] = ms[h * n_max + c] * il;
        }
        __syncthreads();
    }
    const int k0 = col0 + threadIdx.x * 4;
    float4 v;
    if (n > 1) {
        const int h = k0 / D, d = k0 % D;
        const float *pp = a.partials + ((size_t)w0 * Hq + h) * (D + 2) + d;
        const size_t cs = (size_t)Hq * (D + 2);
        const float *f = fw + (h - h0) * n_max;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int c = 0; c < n; c++) {
            const float2 x0 = *reinterpret_cast<const float2 *>(pp + c * cs), x1 = *reinterpret_cast<const float2 *>(pp + c * cs + 2);
            const float fc = f[c];
            acc.x = fmaf(x0.x, fc, acc.x); acc.y = fmaf(x0.y, fc, acc.y); acc.z = fmaf(x1.x, fc, acc.z); acc.w = fmaf(x1.y, fc, acc.w);
        }
        v = acc;
    } else {
        v = *reinterpret_cast<const float4 *>(a.out + (size_t)row * a.out_row_stride + k0);
    }
    const float t[4] = {v.x * inv, v.y * inv, v.z * inv, v.w * inv};
    vx_split_store4(t, s.hi + (size_t)row * s.k_pad, s.lo + (size_t)row * s.k_pad, s.bsum + (size_t)row * (s.k_pad / 32), k0);
}

template <int D, int G>
static int flash_launch_mma(vx_ctx *c, const VxAttnArgs &a, dim3 grid) {
    // head_dim 256 doubles the staging buffers and the register file per warp: two warps per CTA keep three CTAs on an SM
    constexpr int NW = D == 256 ? 2 : ATT_WARPS;
    constexpr int SMEM = NW * 2 * 2 * ATT_BS * D * 2;      // per warp: two stages of a K and a V page tile
    static_assert(SMEM >= (int)((NW * G * D + 2 * NW * G) * sizeof(float)), "merge buffers fit in the staging area");
    static VxPerDevice attr;
    if (attr.max_dynamic_smem(c, paged_flash_mma_kernel<D, G, NW>, SMEM) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (vx_launch_chain(paged_flash_mma_kernel<D, G, NW>, grid, dim3(NW * 32), (size_t)SMEM, c->stream, a) != cudaSuccess) return VX_E_CUDA;
    return 0;
}

template <int D>
static int flash_launch_g(vx_ctx *c, const VxAttnArgs &a, int G) {
    dim3 grid(a.n_work, a.n_kv_heads);
    if (g_attn_mma && G > 1) {
        switch (G) {
        case 2: return flash_launch_mma<D, 2>(c, a, grid);
        case 4: return flash_launch_mma<D, 4>(c, a, grid);
        case 8: return flash_launch_mma<D, 8>(c, a, grid);
        default: return -1;
        }
    }
    switch (G) {
    case 1: if (vx_launch_chain(paged_flash_kernel<D, 1>, grid, dim3(ATT_WARPS * 32), 0, c->stream, a) != cudaSuccess) return VX_E_CUDA; break;
    case 2: if (vx_launch_chain(paged_flash_kernel<D, 2>, grid, dim3(ATT_WARPS * 32), 0, c->stream, a) != cudaSuccess) return VX_E_CUDA; break;
    case 4: if (vx_launch_chain(paged_flash_kernel<D, 4>, grid, dim3(ATT_WARPS * 32), 0, c->stream, a) != cudaSuccess) return VX_E_CUDA; break;
    case 8: if (vx_launch_chain(paged_flash_kernel<D, 8>, grid, dim3(ATT_WARPS * 32), 0, c->stream, a) != cudaSuccess) return VX_E_CUDA; break;
    default: return -1;
    }
    return 0;
}

int vxp_attention(vx_ctx *c, const VxAttnArgs &a) { return vxp_attention_split(c, a, nullptr, 0, nullptr); }

// The same, optionally followed by the fp16 split of the attention output (split != nullptr): when the split-K merge and the
// split can share one kernel, *fused is set and `split` holds the rows; otherwise the caller runs the split itself.
// n_max_chunks bounds the chunks of one row.
int vxp_attention_split(vx_ctx *c, const VxAttnArgs &a, const VxSplit *split, int n_max_chunks, bool *fused) {
    if (fused) *fused = false;
    if (a.rows <= 0) return VX_OK;
    if (a.n_q_heads <= 0 || a.n_kv_heads <= 0 || a.n_q_heads % a.n_kv_heads != 0)
        return vx_fail(c, VX_E_BAD_ARG, "paged attention: %d q heads over %d kv heads", a.n_q_heads, a.n_kv_heads);
    if (a.head_dim <= 0 || a.head_dim > 256) return vx_fail(c, VX_E_BAD_ARG, "paged attention: head_dim %d (max 256)", a.head_dim);
    const int G = a.n_q_heads / a.n_kv_heads, D = a.head_dim;
    bool fast = a.pool_is_f16 && a.block_size == ATT_BS && (D == 64 || D == 128 || D == 256) &&
                (G == 1 || G == 2 || G == 4 || G == 8) && a.work != nullptr && a.n_work > 0 && (a.q_row_stride % 4 == 0);
    if (fast) {
        int rc = D == 64 ? flash_launch_g<64>(c, a, G) : D == 128 ? flash_launch_g<128>(c, a, G) : flash_launch_g<256>(c, a, G);
        if (rc == 0) {
            VX_LAUNCH_CHECK(c);
            const int cols = a.n_q_heads * D;
            const size_t fw_bytes = 2 * (size_t)a.n_q_heads * max(n_max_chunks, 1) * sizeof(float);
            if (split && fused && a.row_bound && n_max_chunks > 0 && cols % MS_COLS == 0 && split->k_pad == cols && MS_COLS % D == 0 &&
                a.out_row_stride % 4 == 0 && 2 * (size_t)(MS_COLS / D) * n_max_chunks * sizeof(float) <= 40 * 1024) {
                const size_t bytes = 2 * (size_t)(MS_COLS / D) * n_max_chunks * sizeof(float);
                if (vx_launch_chain(paged_merge_split_heads_kernel, dim3(a.rows, cols / MS_COLS), dim3(MS_THREADS), bytes, c->stream, a, *split, n_max_chunks) != cudaSuccess) return vx_fail(c, VX_E_CUDA, "merge launch");
                VX_LAUNCH_CHECK(c);
                *fused = true;
                return VX_OK;
            }
            if (split && fused && n_max_chunks > 0 && fw_bytes <= 40 * 1024 && split->k_pad <= 8 * VX_ROW_THREADS * 4 && a.out_row_stride % 4 == 0) {
                const int nc = ceil_div(split->k_pad, VX_ROW_THREADS * 4);
                switch (nc) {
#define VX_MS_CASE(N) case N: if (vx_launch_chain(paged_merge_split_kernel<N>, dim3(a.rows), dim3(VX_ROW_THREADS), fw_bytes, c->stream, a, *split, cols, n_max_chunks) != cudaSuccess) return vx_fail(c, VX_E_CUDA, "merge launch"); break;
                    VX_MS_CASE(1) VX_MS_CASE(2) VX_MS_CASE(3) VX_MS_CASE(4) VX_MS_CASE(5) VX_MS_CASE(6) VX_MS_CASE(7) VX_MS_CASE(8)
#undef VX_MS_CASE
                }
                VX_LAUNCH_CHECK(c);
                *fused = true;
                return VX_OK;
            }
            dim3 mg(a.n_q_heads, a.rows);
            paged_merge_kernel<<<mg, min(D, 256), 0, c->stream>>>(a);
            VX_LAUNCH_CHECK(c);
            return VX_OK;
        }
    }
    dim3 grid(a.n_q_heads, a.rows);
    size_t smem = (size_t)(D + 256) * sizeof(float);
    paged_generic_kernel<<<grid, 256, smem, c->stream>>>(a);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

// ------------------------------------------------------------------ interface-level entry points
__global__ void iface_build_work_kernel(int rows, const int32_t *kv_start, const int32_t *kv_len, int block_size, int chunk_pages,
                                        int4 *work, int32_t *row_work_start, int32_t *n_work, int max_work) {
    __shared__ int tmp[33];
    __shared__ int ovf;
    if (threadIdx.x == 0) ovf = 0;
    __syncthreads();
    int n = vx_build_work(rows, kv_start, kv_len, nullptr, block_size, chunk_pages, work, row_work_start, max_work, &ovf, tmp);
    if (threadIdx.x == 0) *n_work = n;
}

// Lays out in the context scratch: tables[], row_slot[], kv_start[], kv_len[], row_work_start[], n_work, work[], partials.
// kv_len_dev != 0: per-row lengths already on the device (multi-query verify); else kv_len_host is uploaded.
static int paged_iface(vx_ctx *c, vx_dptr q, vx_dptr pool, int pool_is_f16, const vx_dptr *tables, const int *row_slot,
                       const int *kv_start_host, const int *kv_len_host, vx_dptr kv_len_dev, int max_kv_len, vx_dptr out,
                       int rows, int n_tables, int block_size, int hq, int hkv, int d, float scale, float softcap) {
    VX_REQUIRE(c, q && pool && out, "nil device pointer");
    VX_REQUIRE(c, rows > 0 && block_size > 0 && hq > 0 && hkv > 0 && d > 0 && d <= 256 && hq % hkv == 0, "bad dimensions");
    int max_pages = ceil_div(max_kv_len, block_size);
    int chunk_pages = max(4, ceil_div(max_pages * rows * hkv, 4 * c->sm_count));
    int max_work = rows * ceil_div(max_pages, chunk_pages) + rows;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    size_t o_tab = take(sizeof(void *) * n_tables), o_slot = take(4 * rows), o_ks = take(4 * rows), o_kl = take(4 * rows),
           o_rws = take(4 * (rows + 1)), o_nw = take(4), o_work = take(sizeof(int4) * max_work),
           o_part = take((size_t)max_work * hq * (d + 2) * 4);
    void *base;
    VX_TRY(vx_scratch(c, off, &base));
    char *p = (char *)base;
    std::vector<int32_t> ks(rows, 0);
    if (kv_start_host) for (int i = 0; i < rows; i++) ks[i] = kv_start_host[i];
    VX_CUDA(c, cudaMemcpyAsync(p + o_tab, tables, sizeof(vx_dptr) * n_tables, cudaMemcpyHostToDevice, c->stream));
    VX_CUDA(c, cudaMemcpyAsync(p + o_slot, row_slot, 4 * rows, cudaMemcpyHostToDevice, c->stream));
    VX_CUDA(c, cudaMemcpyAsync(p + o_ks, ks.data(), 4 * rows, cudaMemcpyHostToDevice, c->stream));
    const int32_t *kl_dev;
    if (kv_len_dev) kl_dev = dp<int32_t>(kv_len_dev);
    else { VX_CUDA(c, cudaMemcpyAsync(p + o_kl, kv_len_host, 4 * rows, cudaMemcpyHostToDevice, c->stream)); kl_dev = (const int32_t *)(p + o_kl); }
    VX_CUDA(c, cudaStreamSynchronize(c->stream));   // host staging arrays go out of scope
    iface_build_work_kernel<<<1, 256, 0, c->stream>>>(rows, (const int32_t *)(p + o_ks), kl_dev, block_size, chunk_pages,
                                                      (int4 *)(p + o_work), (int32_t *)(p + o_rws), (int32_t *)(p + o_nw), max_work);
    VX_LAUNCH_CHECK(c);
    VxAttnArgs a{};
    a.q = dp<float>(q); a.q_row_stride = hq * d; a.pool = dp<void>(pool); a.pool_is_f16 = pool_is_f16;
    a.tables = (const int32_t *const *)(p + o_tab); a.row_slot = (const int32_t *)(p + o_slot);
    a.row_kv_start = (const int32_t *)(p + o_ks); a.row_kv_len = kl_dev;
    a.work = (const int4 *)(p + o_work); a.n_work_dev = (const int32_t *)(p + o_nw); a.n_work = max_work;
    a.row_work_start = (const int32_t *)(p + o_rws); a.partials = (float *)(p + o_part);
    a.out = dp<float>(out); a.out_row_stride = hq * d;
    a.rows = rows; a.n_q_heads = hq; a.n_kv_heads = hkv; a.head_dim = d; a.block_size = block_size;
    a.scale = scale; a.softcap = softcap;
    return vxp_attention(c, a);
}

// ------------------------------------------------------------------ decode attention without any allocation
// Some callers must not allocate device memory when they attend: a serving process that has handed every free byte of
// HBM to its KV pool, a host thread inside a latency-critical section, or an embedder whose allocator is not reentrant.
// For them the split-K scratch of the paged decode (block-table pointer, row descriptors, work list, partial results)
// lives in this fixed array.  Every GPU that loads the library holds these 4 MiB until the process exits.
constexpr size_t VX_NOALLOC_SCRATCH_BYTES = 4u << 20;
constexpr int VX_NOALLOC_MAX_WORK = 1024;
static __device__ __align__(256) unsigned char g_noalloc_scratch[VX_NOALLOC_SCRATCH_BYTES];
// The array's name is a host-side stand-in in host code, not a device address: the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static std::atomic<void *> g_noalloc_dev_ptr[64];     // zero-initialised; contexts on different threads may race to fill an entry with the same value

struct NoAllocLayout { size_t tab, slot, ks, kl, rws, nw, work, part; };
static NoAllocLayout noalloc_layout() {
    NoAllocLayout L;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += (bytes + 255) & ~(size_t)255; return o; };
    L.tab = take(sizeof(void *)); L.slot = take(4); L.ks = take(4); L.kl = take(4); L.rws = take(8); L.nw = take(4);
    L.work = take(sizeof(int4) * VX_NOALLOC_MAX_WORK); L.part = off;
    return L;
}
// fills the single-row descriptors from kernel arguments (no host-to-device copy) and builds the work list
__global__ void noalloc_setup_kernel(unsigned char *scratch, NoAllocLayout L, const int32_t *table, int kv_len, int block_size, int chunk_pages) {
    __shared__ int tmp[33];
    __shared__ int ovf;
    if (threadIdx.x == 0) {
        ovf = 0;
        *reinterpret_cast<const int32_t **>(scratch + L.tab) = table;
        *reinterpret_cast<int32_t *>(scratch + L.slot) = 0;
        *reinterpret_cast<int32_t *>(scratch + L.ks) = 0;
        *reinterpret_cast<int32_t *>(scratch + L.kl) = kv_len;
    }
    __syncthreads();
    int n = vx_build_work(1, reinterpret_cast<const int32_t *>(scratch + L.ks), reinterpret_cast<const int32_t *>(scratch + L.kl), nullptr, block_size,
                          chunk_pages, reinterpret_cast<int4 *>(scratch + L.work), reinterpret_cast<int32_t *>(scratch + L.rws),
                          VX_NOALLOC_MAX_WORK, &ovf, tmp);
    if (threadIdx.x == 0) *reinterpret_cast<int32_t *>(scratch + L.nw) = n;
}

template <typename T>
static int reshape_launch(vx_ctx *c, vx_dptr src, vx_dptr pool, vx_dptr pt, vx_dptr bo, int n_tokens, int hkv, int d, int bs, int is_v) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (n_tokens <= 0) return VX_OK;
    VX_REQUIRE(c, src && pool && pt && bo && hkv > 0 && d > 0 && bs > 0, "bad arguments");
    long total = (long)n_tokens * hkv * d;
    reshape_paged_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, c->stream>>>(dp<float>(src), dp<T>(pool), dp<int32_t>(pt),
                                                                                   dp<int32_t>(bo), n_tokens, hkv * d, bs, is_v);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

extern "C" {

int vx_reshape_paged_kv(vx_ctx *c, vx_dptr src, vx_dptr pool, vx_dptr pt, vx_dptr bo, int n_tokens, int hkv, int d, int bs, int is_v) {
    return reshape_launch<float>(c, src, pool, pt, bo, n_tokens, hkv, d, bs, is_v);
}
int vx_reshape_paged_kv_f16(vx_ctx *c, vx_dptr src, vx_dptr pool, vx_dptr pt, vx_dptr bo, int n_tokens, int hkv, int d, int bs, int is_v) {
    return reshape_launch<__half>(c, src, pool, pt, bo, n_tokens, hkv, d, bs, is_v);
}

// kvLen = (numBlocks-1)*blockSize + tokensInLastBlock (backend/metal/metal_bridge_darwin.m:11092-11100)
static int decode_one(vx_ctx *c, vx_dptr q, vx_dptr pool, int f16, vx_dptr table, vx_dptr out, int n_blocks, int bs, int hq,
                      int hkv, int d, float scale, int til) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, n_blocks > 0 && til > 0 && til <= bs && table, "bad block table arguments");
    int kv_len = (n_blocks - 1) * bs + til, slot = 0;
    return paged_iface(c, q, pool, f16, &table, &slot, nullptr, &kv_len, 0, kv_len, out, 1, 1, bs, hq, hkv, d, scale, 0.f);
}
int vx_sdpa_paged_decode(vx_ctx *c, vx_dptr q, vx_dptr pool, vx_dptr table, vx_dptr out, int n_blocks, int bs, int hq, int hkv,
                         int d, float scale, int til) {
    return decode_one(c, q, pool, 0, table, out, n_blocks, bs, hq, hkv, d, scale, til);
}
int vx_sdpa_paged_decode_f16(vx_ctx *c, vx_dptr q, vx_dptr pool, vx_dptr table, vx_dptr out, int n_blocks, int bs, int hq, int hkv,
                             int d, float scale, int til) {
    return decode_one(c, q, pool, 1, table, out, n_blocks, bs, hq, hkv, d, scale, til);
}

int vx_sdpa_paged_decode_ex(vx_ctx *c, vx_dptr q, vx_dptr pool, vx_dptr table, vx_dptr out, int kv_start, int kv_len, int bs,
                            int hq, int hkv, int d, float scale, float softcap, int f16) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, table && kv_start >= 0 && kv_len > kv_start, "empty attention range");
    int slot = 0;
    return paged_iface(c, q, pool, f16, &table, &slot, &kv_start, &kv_len, 0, kv_len, out, 1, 1, bs, hq, hkv, d, scale, softcap);
}

// every sequence has its own table pointer and length; queries and outputs are packed [batch][Hq*D]
int vx_sdpa_paged_decode_batched(vx_ctx *c, vx_dptr q, vx_dptr pool, const vx_dptr *tables, vx_dptr out, int batch,
                                 int max_blocks, int bs, int hq, int hkv, int d, float scale, const int *seq_lens, int f16) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, batch > 0 && tables && seq_lens && max_blocks > 0, "bad arguments");
    std::vector<int> slot(batch);
    int mx = 0;
    for (int i = 0; i < batch; i++) {
        slot[i] = i;
        VX_REQUIRE(c, tables[i] != 0 && seq_lens[i] > 0 && seq_lens[i] <= max_blocks * bs, "sequence length outside its block table");
        mx = max(mx, seq_lens[i]);
    }
    return paged_iface(c, q, pool, f16, tables, slot.data(), nullptr, seq_lens, 0, mx, out, batch, batch, bs, hq, hkv, d, scale, 0.f);
}

// query i attends positions [0, kvLens[i]) (backend/metal/metal_bridge_darwin.m:11205-11311); kvLens is a device buffer
int vx_sdpa_paged_decode_multiquery(vx_ctx *c, vx_dptr q, vx_dptr pool, vx_dptr table, vx_dptr out, vx_dptr kv_lens,
                                    int n_blocks, int bs, int hq, int hkv, int d, float scale, int query_len, int f16) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, table && kv_lens && n_blocks > 0 && query_len > 0, "bad arguments");
    std::vector<int> slot(query_len, 0);
    return paged_iface(c, q, pool, f16, &table, slot.data(), nullptr, nullptr, kv_lens, n_blocks * bs, out, query_len, 1, bs, hq, hkv, d,
                       scale, 0.f);
}


// Same result as vx_sdpa_paged_decode_f16, but the call allocates nothing: no cudaMalloc / cudaFree, no growth of the
// context scratch, no host heap.  Limits: head_dim <= 256, n_q_heads * (head_dim + 2) * 4 bytes per split-K chunk must fit
// the 4 MiB array (the number of chunks shrinks to fit; at worst one chunk per row), n_blocks <= 65536; anything larger is
// refused with VX_E_BAD_ARG (so is a block size above 16384, which keeps kv_len inside an int).  The first call on a device
// looks up the array's address (cudaGetSymbolAddress) and may make the driver load this library's kernels for that device,
// which can allocate inside the driver: make one warm-up call per device outside the section that must not allocate, and
// before starting a stream capture.  All calls share the one array, which keeps the previous call's contents
// (nothing in it needs to start at zero: every field is written before it is read), so two calls that overlap on the GPU
// -- different streams or contexts of one process -- race.
int vx_sdpa_paged_decode_f16_noalloc(vx_ctx *c, vx_dptr q, vx_dptr pool, vx_dptr table, vx_dptr out, int n_blocks, int bs, int hq,
                                     int hkv, int d, float scale, int til) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, q && pool && out && table, "nil device pointer");
    VX_REQUIRE(c, n_blocks > 0 && n_blocks <= 65536 && bs > 0 && bs <= 16384 && til > 0 && til <= bs,
               "bad block table arguments (n_blocks <= 65536, block size <= 16384)");
    VX_REQUIRE(c, hq > 0 && hkv > 0 && hq % hkv == 0 && d > 0 && d <= 256, "bad head configuration (head_dim <= 256)");
    VX_REQUIRE(c, c->device >= 0 && c->device < 64, "device index out of range");
    void *sym = g_noalloc_dev_ptr[c->device].load(std::memory_order_acquire);
    if (!sym) {     // once per device, with that device current (VxGuard made it so)
        cudaError_t e = cudaGetSymbolAddress(&sym, g_noalloc_scratch);
        if (e != cudaSuccess || !sym) return vx_cuda_fail(c, e, "cudaGetSymbolAddress(no-alloc scratch)");
        g_noalloc_dev_ptr[c->device].store(sym, std::memory_order_release);
    }
    unsigned char *sp = static_cast<unsigned char *>(sym);
    const NoAllocLayout L = noalloc_layout();
    const size_t per_chunk = (size_t)hq * (d + 2) * sizeof(float);
    if (L.part + per_chunk > VX_NOALLOC_SCRATCH_BYTES)
        return vx_fail(c, VX_E_BAD_ARG, "vx_sdpa_paged_decode_f16_noalloc: %d heads x head_dim %d exceed the %zu-byte scratch", hq, d, VX_NOALLOC_SCRATCH_BYTES);
    const int kv_len = (n_blocks - 1) * bs + til;
    int max_chunks = (int)std::min<size_t>((VX_NOALLOC_SCRATCH_BYTES - L.part) / per_chunk, (size_t)VX_NOALLOC_MAX_WORK);
    int chunk_pages = max(4, ceil_div(n_blocks * hkv, 4 * c->sm_count));
    if (ceil_div(n_blocks, chunk_pages) > max_chunks) chunk_pages = ceil_div(n_blocks, max_chunks);
    noalloc_setup_kernel<<<1, 32, 0, c->stream>>>(sp, L, dp<int32_t>(table), kv_len, bs, chunk_pages);
    VX_LAUNCH_CHECK(c);
    VxAttnArgs a{};
    a.q = dp<float>(q); a.q_row_stride = hq * d; a.pool = dp<void>(pool); a.pool_is_f16 = 1;
    a.tables = reinterpret_cast<const int32_t *const *>(sp + L.tab); a.row_slot = reinterpret_cast<const int32_t *>(sp + L.slot);
    a.row_kv_start = reinterpret_cast<const int32_t *>(sp + L.ks); a.row_kv_len = reinterpret_cast<const int32_t *>(sp + L.kl);
    a.work = reinterpret_cast<const int4 *>(sp + L.work); a.n_work_dev = reinterpret_cast<const int32_t *>(sp + L.nw);
    a.n_work = ceil_div(n_blocks, chunk_pages); a.row_work_start = reinterpret_cast<const int32_t *>(sp + L.rws);
    a.partials = reinterpret_cast<float *>(sp + L.part);
    a.out = dp<float>(out); a.out_row_stride = hq * d;
    a.rows = 1; a.n_q_heads = hq; a.n_kv_heads = hkv; a.head_dim = d; a.block_size = bs; a.scale = scale; a.softcap = 0.f;
    return vxp_attention(c, a);
}

}  // extern "C"
