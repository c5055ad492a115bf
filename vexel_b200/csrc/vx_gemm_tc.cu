// Q4_0 projection on the 5th-generation tensor cores (tcgen05 + TMEM) for batches of 17..64 rows per tile.
//
// Shape ("swap-AB"): D[128 weight rows x 64 batch rows] += A[128 x 64k] * B[64 x 64k]^T per pipeline stage, accumulator in
// TMEM (128 lanes x 64 fp32 columns), one CTA per 128-row weight tile and split-K slice.
//   * A is produced on the fly: 8 producer warps copy the packed nibbles of the stage into shared memory (cp.async),
//     expand them to fp16 and write two K-major, 128-byte-swizzled operand tiles A_hi and A_lo with
//         w = d*(q-8) = A_hi + A_lo exactly      (A_hi = fp16 product, A_lo = fp16 FMA residual).
//   * B is the activation split x = s*(x_hi + x_lo) (vx_common.cuh), copied by cp.async into the same swizzled layout.
//   * One elected thread issues tcgen05.mma for A_hi*x_hi + A_lo*x_hi + A_hi*x_lo (the dropped A_lo*x_lo is 2^-22 relative),
//     and tcgen05.commit hands the stage back to the producers.
//   * Warps 0-3 read the accumulator with tcgen05.ld, scale by the row's power of two and store.
// Every wait on an mbarrier is bounded: on timeout the kernel raises an error flag, skips to the end, frees its TMEM and
// returns, so a protocol bug cannot hang the GPU.
#include "vx_common.cuh"

namespace {

constexpr int TC_ROWS = 128;          // weight rows per CTA (MMA M)
constexpr int TC_MT = 64;             // batch rows per CTA (MMA N)
constexpr int TC_BK = 64;             // k per stage = one 128-byte swizzle row of fp16
constexpr int TC_STAGES = 4;
constexpr int TC_RAW_STAGES = 4;        // > PREFETCH + 1: a slot is rewritten only after a producer barrier follows its last read
constexpr int TC_PREFETCH = 2;        // stages of cp.async in flight
constexpr int TC_PRODUCERS = 256;
constexpr int TC_THREADS = TC_PRODUCERS + 32;
constexpr int A_TILE = TC_ROWS * 128;         // bytes of one fp16 operand tile (128 rows x 128 B)
constexpr int X_TILE = TC_MT * 128;
constexpr int STAGE_BYTES = 2 * A_TILE + 2 * X_TILE;       // A_hi, A_lo, X_hi, X_lo
constexpr int RAW_BYTES = TC_ROWS * 32;                    // packed nibbles of one stage
constexpr int SMEM_BYTES = TC_STAGES * STAGE_BYTES + TC_RAW_STAGES * RAW_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
constexpr long long WAIT_CLOCKS = 400000000LL;             // ~0.2 s at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false on timeout or when another thread of the CTA has already given up
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CLOCKS) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                           // leading-dimension byte offset (unused with 128B swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride between 8-row core-matrix groups
    d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                           // SWIZZLE_128B
    return d;
}
// instruction descriptor: D=f32, A=B=f16, both K-major, N=64, M=128
constexpr uint32_t UMMA_IDESC = (1u << 4) | ((uint32_t)(TC_MT >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(UMMA_IDESC), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// (v & 0x000F000F) holds two nibbles -> half2 {q0-8, q1-8}
__device__ __forceinline__ __half2 nib2(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;
    return __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1032.f, 1032.f));
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }

// grid: (ceil(N/128), split_k, ceil(M/64)); out layout [split][M][ld_out]
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_q4_0_tc_kernel(const uint4 *__restrict__ qs, const __half *__restrict__ sc, const __half *__restrict__ xh,
                    const __half *__restrict__ xl, const float *__restrict__ xscale, float *__restrict__ out, int M, int N,
                    int k_groups, int kb_per_split, int x_ld, int ld_out, size_t part_stride, int *__restrict__ err_flag) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;            // operand tiles need 1024-byte alignment
    const uint32_t raw_base = base + TC_STAGES * STAGE_BYTES;
    const uint32_t bar_base = raw_base + TC_RAW_STAGES * RAW_BYTES;         // full[S], empty[S], accum
    unsigned char *gen_base = smem_raw + (base - smem_u32(smem_raw));
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (TC_STAGES + s); };
    const uint32_t accum_bar = bar_base + 8u * (2 * TC_STAGES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = blockIdx.x * TC_ROWS, m0 = blockIdx.z * TC_MT;
    const int n_kb_total = k_groups * 2;
    const int kb_begin = blockIdx.y * kb_per_split;
    const int n_kb = min(n_kb_total, kb_begin + kb_per_split) - kb_begin;

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < TC_STAGES; s++) { mbar_init(full_bar(s), TC_PRODUCERS); mbar_init(empty_bar(s), 1); }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {   // the MMA warp owns the TMEM allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TC_MT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;

    if (warp < 8) {
        // ------------------------------------------------------------------ producers
        const int row = tid & 127, h = tid >> 7;                 // operand row and which word pair {2h, 2h+1}
        const int grow = min(r0 + row, N - 1);
        const __half2 *scp = reinterpret_cast<const __half2 *>(sc + (size_t)grow * k_groups * 4);

        auto issue_loads = [&](int kb) {      // packed nibbles -> raw ring, activations -> stage
            const int gkb = kb_begin + kb, j = gkb >> 1, sub = gkb & 1, st = kb % TC_STAGES, rs = kb % TC_RAW_STAGES;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                int i = tid + TC_PRODUCERS * u, rr = i >> 2, c = i & 3;
                int gr = min(r0 + rr, N - 1);
                const unsigned char *src = reinterpret_cast<const unsigned char *>(qs + ((size_t)gr * k_groups + j) * 4 + c) + sub * 8;
                cp_async8(raw_base + rs * RAW_BYTES + rr * 32 + c * 8, src);
            }
            const uint32_t xs = base + st * STAGE_BYTES + 2 * A_TILE;
#pragma unroll
            for (int u = 0; u < 4; u++) {
                int i = tid + TC_PRODUCERS * u;                  // 0..1023: term, row, chunk
                int term = i >> 9, rr = (i >> 3) & 63, ch = i & 7;
                int m = min(m0 + rr, M - 1);
                const __half *src = (term ? xl : xh) + (size_t)m * x_ld + (size_t)gkb * TC_BK + ch * 8;
                cp_async16(xs + term * X_TILE + (rr >> 3) * 1024 + (rr & 7) * 128 + ((ch ^ (rr & 7)) << 4), src);
            }
        };

        bool ok = true;
        // prologue: loads for the first TC_PREFETCH stages (their buffers are fresh)
#pragma unroll
        for (int p = 0; p < TC_PREFETCH; p++) {
            if (p < n_kb) issue_loads(p);
            cp_commit();
        }
        __half2 d_cur = n_kb > 0 ? scp[kb_begin] : __floats2half2_rn(0.f, 0.f);
        for (int kb = 0; kb < n_kb && ok; kb++) {
            const int st = kb % TC_STAGES, rs = kb % TC_RAW_STAGES;
            // issue the loads of stage kb+PREFETCH once the tensor core has released its buffer
            const int nk = kb + TC_PREFETCH;
            if (nk < n_kb) {
                if (nk >= TC_STAGES) ok = mbar_wait(empty_bar(nk % TC_STAGES), ((nk / TC_STAGES) - 1) & 1, abort_flag);
                if (ok) issue_loads(nk);
            }
            cp_commit();
            const __half2 d_next = (kb + 1 < n_kb) ? scp[kb_begin + kb + 1] : d_cur;
            // the buffer of stage kb was released before its loads were issued (PREFETCH iterations ago)
            cp_wait<TC_PREFETCH>();          // this thread's copies for stage kb have landed
            // raw nibbles are read by other threads than the ones that copied them; the barrier also makes the decision to
            // give up uniform across the producers (a thread leaving alone would strand the others at the next barrier)
            {
                uint32_t give_up = (!ok || *abort_flag) ? 1u : 0u, any;
                asm volatile("{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.or.pred p, 1, %2, q;\nselp.u32 %0, 1, 0, p;\n}"
                             : "=r"(any) : "r"(give_up), "n"(TC_PRODUCERS) : "memory");
                if (any) { ok = false; break; }
            }
            const uint4 w = *reinterpret_cast<const uint4 *>(gen_base + TC_STAGES * STAGE_BYTES + rs * RAW_BYTES + row * 32 + h * 16);
            // w = { word 2h of block 0, word 2h of block 1, word 2h+1 of block 0, word 2h+1 of block 1 }
            const uint32_t wb[2][2] = {{w.x, w.z}, {w.y, w.w}};   // [block][word of the pair]
            unsigned char *a_hi = gen_base + st * STAGE_BYTES + (row >> 3) * 1024 + (row & 7) * 128;
            unsigned char *a_lo = a_hi + A_TILE;
#pragma unroll
            for (int b = 0; b < 2; b++) {
                const __half dd = b == 0 ? __low2half(d_cur) : __high2half(d_cur);
                const __half2 d2 = __half2half2(dd);
#pragma unroll
                for (int nib = 0; nib < 2; nib++) {
                    __half2 q[4];
                    q[0] = nib2(wb[b][0] >> (4 * nib)); q[1] = nib2(wb[b][0] >> (4 * nib + 8));
                    q[2] = nib2(wb[b][1] >> (4 * nib)); q[3] = nib2(wb[b][1] >> (4 * nib + 8));
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        __half2 ph = __hmul2(q[e], d2);
                        __half2 pl = __hfma2(q[e], d2, __hneg2(ph));
                        hi[e] = h2u(ph); lo[e] = h2u(pl);
                    }
                    const int chunk = 4 * b + 2 * nib + h;          // 16-byte chunk of the 128-byte row
                    const int off = (chunk ^ (row & 7)) << 4;
                    *reinterpret_cast<uint4 *>(a_hi + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    *reinterpret_cast<uint4 *>(a_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
            d_cur = d_next;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the tensor core
            mbar_arrive(full_bar(st));
        }
        cp_wait<0>();
    } else if (lane == 0) {
        // ------------------------------------------------------------------ MMA issue (one thread)
        bool ok = true;
        for (int kb = 0; kb < n_kb && ok; kb++) {
            const int st = kb % TC_STAGES;
            ok = mbar_wait(full_bar(st), (kb / TC_STAGES) & 1, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t sa = base + st * STAGE_BYTES;
            const uint64_t a_hi = umma_desc(sa), a_lo = umma_desc(sa + A_TILE);
            const uint64_t x_hi = umma_desc(sa + 2 * A_TILE), x_lo = umma_desc(sa + 2 * A_TILE + X_TILE);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; k++) {
                const uint64_t adv = (uint64_t)(k * 32 >> 4);     // 16 fp16 = 32 bytes along K inside the swizzle row
                umma_f16(tmem, a_hi + adv, x_hi + adv, (kb > 0 || k > 0) ? 1u : 0u);
                umma_f16(tmem, a_lo + adv, x_hi + adv, 1u);
                umma_f16(tmem, a_hi + adv, x_lo + adv, 1u);
            }
            umma_commit(empty_bar(st));       // arrives when the MMAs above have finished reading the stage
        }
        if (ok) umma_commit(accum_bar);
    }

    // ------------------------------------------------------------------ epilogue (warps 0-3: TMEM lanes 32*warp .. +31)
    __syncwarp();
    if (warp < 4) {
        bool ok = n_kb > 0 && mbar_wait(accum_bar, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            float *o = out + (size_t)blockIdx.y * part_stride;
            const int n = r0 + warp * 32 + lane;
#pragma unroll
            for (int cc = 0; cc < TC_MT; cc += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + cc;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
                    "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int m = m0 + cc + j;
                        if (m < M) o[(size_t)m * ld_out + n] = __uint_as_float(v[j]) * xscale[m];
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_MT) : "memory");
    }
    if (tid == 0 && s_abort) atomicExch(err_flag, VX_E_TIMEOUT);
}

}  // namespace

// same contract as vxq_gemm (vx_quant.cu); the context's device error word receives VX_E_TIMEOUT if a bounded wait gave up
int vxq_gemm_tc(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
                size_t parts_cap_floats) {
    int *err_flag = c->d_int_result + 8;
    if (w.type != VX_T_Q4_0) return vx_fail(c, VX_E_UNSUPPORTED, "tensor-core projection: weight type %d", w.type);
    if (x.k_pad != w.k_pad) return vx_fail(c, VX_E_BAD_ARG, "projection: activation row stride %d != weight k_pad %d", x.k_pad, w.k_pad);
    static bool attr_set = false;
    if (!attr_set) {
        VX_CUDA(c, cudaFuncSetAttribute(gemm_q4_0_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set = true;
    }
    const int k_groups = w.k_pad / 128, n_kb = k_groups * 2;
    const int tiles = ceil_div(w.n, TC_ROWS) * ceil_div(m, TC_MT);
    // split-K for whole waves of one CTA per SM
    int split = 1;
    if (parts) {
        const int slots = c->sm_count;
        double best = 0.0;
        for (int s = 1; s <= 8 && s <= max(1, n_kb / 8); s++) {
            if ((size_t)s * m * w.n > parts_cap_floats) break;
            int per = ceil_div(n_kb, s), s_eff = ceil_div(n_kb, per);
            long n_cta = (long)tiles * s_eff;
            double eff = (double)n_cta / (double)(ceil_div64(n_cta, slots) * slots) * ((double)n_kb / (double)(per * s_eff));
            if (eff > best + 0.03) { best = eff; split = s; }
        }
    }
    int per = ceil_div(n_kb, split);
    split = ceil_div(n_kb, per);
    float *dst = split > 1 ? parts : out;
    int ld = split > 1 ? w.n : ld_out;
    *n_parts_out = split;
    dim3 grid(ceil_div(w.n, TC_ROWS), split, ceil_div(m, TC_MT));
    gemm_q4_0_tc_kernel<<<grid, TC_THREADS, SMEM_BYTES, c->stream>>>((const uint4 *)w.qs, (const __half *)w.sc, x.hi, x.lo, x.scale, dst,
                                                                    m, w.n, k_groups, per, x.k_pad, ld, (size_t)m * w.n, err_flag);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}
