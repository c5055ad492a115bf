// Quantised projections (GGUF Q4_0, Q4_K, Q6_K) on the 5th-generation tensor cores (tcgen05 + TMEM) for batches above the
// measured crossover (17 rows).  Decode batches of up to 64 rows take the persistent kernel (vx_gemm_tcp.cu) when it is
// eligible; this kernel serves larger batches, odd group counts and the cases where no partial-sum buffer is passed.
//
// Shape ("swap-AB"): D[128 weight rows x batch] += A[128 x 64k] * B[batch x 64k]^T per pipeline stage, accumulator in tensor
// memory, one CTA per (128-row weight tile, split-K slice, 64-row batch tile).
//   warp 18    TMA producer: per stage the activation tiles x_hi and x_lo (64 rows x 128 B each, SWIZZLE_128B, stacked into
//              one 128-row operand) and, every second stage, the packed nibbles of a 128-weight group (128 rows x 64 B,
//              SWIZZLE_64B; Q6_K also the 32-byte rows of top bits).  Its program order keeps the nibble ring at most ~2.5
//              tiles ahead of the MMAs.
//   warps 0-15 dequantisers, two groups of eight warps on alternate stages: a thread reads the 32 weights of one block /
//              sub-block of its row from shared memory, expands them to an fp16 pair and stores the A operand straight
//              into TENSOR MEMORY (one 32-column tcgen05.st; lane = weight row, two fp16 per 32-bit column):
//              Q4_0  w = d (q - 8) = A_hi + A_lo exactly (fp16 product + FMA residual);
//              Q4_K  d1 (q - 8) with d1 = fl(d sc) carried as an fp16 pair, the constant 8 d1 - fl(dmin m) per sub-block is
//                    applied in the epilogue to the activations' 32-block sums;
//              Q6_K  d1 (q - 32), one d1 per 16 weights.
//              With A in shared memory every MMA re-read 4 KB of it and the kernel was bound by shared-memory traffic.
//   warps 16-17 one elected thread each issues, for its half of a stage's K=16 steps, A_hi x [x_hi; x_lo] (N=128) and
//              A_lo x x_hi (N=64) into its own accumulator; the dropped A_lo*x_lo term is 2^-22 relative.  One mbarrier per
//              stage says "ready" (activation bytes landed + eight dequantiser warps arrived); tcgen05.commit hands it back.
//   warps 0-15 epilogue: tcgen05.ld of the four accumulator parts, add in a fixed order, scale by the row's power of two, store.
// Measured dead ends, so that they are not tried again: four issuing threads taking turns per accumulator (slower: the cost
// sits in the number of tcgen05 instructions the SM dispatches per stage, not in one thread's latency); a separate
// producer thread for the nibbles running a full ring ahead (wrong sums on multi-tile batches); one CTA per SM walking the
// (row tile, slice, batch tile) items with its rings running across item boundaries (the loads of the next item overlap the
// epilogue, 1.5 % / 7 % faster than one CTA per item in the same code for Q4_0 / Q4_K, but the restructured kernel needed 96
// registers with spills instead of 64 and lost 3 % / 30 % against this one).
// Every TMA load targets this CTA only.  Every mbarrier wait is bounded: on timeout the kernel raises an error word, skips
// to the end, frees its tensor memory and returns, so a protocol bug cannot hang the GPU.
#include <map>
#include <mutex>
#include <tuple>

#include "vx_tc.cuh"

namespace {
using namespace vxtc;

constexpr int TC_MT = 64;             // batch rows per CTA (decode); batches above 64 rows use 128-row tiles (template parameter MT)
constexpr int TC_BK = 64;             // k per stage = one 128-byte swizzle row of fp16
constexpr int TC_ST = 4;              // pipeline stages: activation tiles in shared memory, weight operand in tensor memory
constexpr int TC_ISSUERS = 2;         // MMA-issuing threads (one per warp), each with its own accumulator
constexpr int TC_RAW = 4;             // ring of 128-weight nibble groups (each feeds two stages)
constexpr int TC_DEQ = 512;           // dequantiser threads: (row, block of the stage, word pair)
constexpr int TC_THREADS = TC_DEQ + 32 * (TC_ISSUERS + 2);   // + TMA producer + helper warp (block sums of the Q4_K correction)
constexpr int x_tile_bytes(int mt) { return mt * 128; }          // one fp16 activation tile (mt rows x 128 B)
constexpr int stage_bytes(int mt) { return 2 * x_tile_bytes(mt); }   // x_hi rows followed by x_lo rows: one 2*mt-row K-major operand
constexpr int issuers_of(int mt) { return mt == 64 ? 2 : 1; }    // a 128-row tile needs the whole accumulator space for one issuer
constexpr int RAW_BYTES = TC_ROWS * 64;       // packed nibbles of one 128-weight group
constexpr int RAWH_BYTES = TC_ROWS * 32;      // Q6_K only: the top two bits of the same group
// Q4_K: the per-sub-block constants (8 d1 - dmin m) and the activations' block sums become two small
// K-major fp16 operands (128-byte swizzled rows of 64 sub-blocks, hi and lo part each) so that the correction is a handful of
// MMAs at the end of the K loop instead of 1024 FMAs per epilogue thread
constexpr int CORR_U = 64;                                    // sub-blocks (K extent) of the correction operands
constexpr int CORR_A_BYTES = TC_ROWS * 128;                   // one part of the constants: 128 weight rows x 64 halfs
constexpr int corr_b_bytes(int mt) { return mt * 128; }       // one part of the block sums: mt batch rows x 64 halfs
constexpr int corr_bytes(int fmt, int mt) { return fmt == 1 ? 2 * CORR_A_BYTES + 2 * corr_b_bytes(mt) : 0; }
constexpr int rawh_bytes(int fmt) { return fmt == 2 ? RAWH_BYTES : 0; }   // only Q6_K stages a second tile per group
constexpr int smem_bytes(int fmt, int mt) {
    return TC_ST * stage_bytes(mt) + TC_RAW * (RAW_BYTES + rawh_bytes(fmt)) + corr_bytes(fmt, mt) + 1024 /*alignment*/ + 512 /*barriers*/ + 512 /*row scales*/;
}
static_assert(smem_bytes(1, 128) <= 232448 && smem_bytes(2, 128) <= 232448, "shared memory budget of the 128-row variants");
enum { TC_Q4_0 = 0, TC_Q4_K = 1, TC_Q6_K = 2 };
// what the block formats need beyond the nibble tiles: scales (Q4_0: half per block; K-quants: 8 bytes per 128-weight group),
// super-block scales (Q4_K: half2 {d, dmin}; Q6_K: half d), and the activations' per-32-block sums for the Q4_K minima
struct TcAux { const void *sc; const void *aux; const float *xbsum; int bsum_ld; };
// tensor memory columns: issuer j accumulates into [128j, 128j+128): cols 0-63 = A_hi*x_hi + A_lo*x_hi, cols 64-127 = A_hi*x_lo
// for its K=16 steps; weight stage s at TMEM_A + 64*s: [hi k0 k1 | lo k0 k1 | hi k2 k3 | lo k2 k3], 8 columns (two fp16 each)
// per K=16 step
constexpr int TMEM_A = TC_ISSUERS * 2 * TC_MT;    // = 256 for both tile heights: 2 issuers x 128 columns, or 1 issuer x 256
constexpr int TMEM_COLS = 512;                // 2 * 128 + 4 * 64
static_assert(TMEM_A + 64 * TC_ST <= TMEM_COLS, "tensor memory budget");
// Self-test of the give-up path: one CTA waits on an mbarrier that nothing ever arrives on, with a short limit, and must
// come back with the error word set instead of spinning.
__global__ void bounded_wait_selftest_kernel(long long limit_clocks, int *__restrict__ err_flag, int *__restrict__ reached_end) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int s_abort;
    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait_limit(smem_u32(&bar), 0, &s_abort, limit_clocks);     // every thread waits; the first to give up raises the flag
    __syncthreads();
    if (threadIdx.x == 0) {
        if (!ok || s_abort) atomicExch(err_flag, VX_E_TIMEOUT);
        *reached_end = 1;
    }
}
// grid: (ceil(N/128), split_k, ceil(M/64)); out layout [split][M][ld_out]; kb_per_split is even
template <int FMT, int MT>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_h, const __grid_constant__ CUtensorMap map_xh,
               const __grid_constant__ CUtensorMap map_xl, const TcAux aux, const float *__restrict__ xscale,
               float *__restrict__ out, int M, int N, int k_groups, int kb_per_split, int ld_out, size_t part_stride,
               int *__restrict__ err_flag) {
    constexpr int X_TILE = x_tile_bytes(MT), STAGE_BYTES = stage_bytes(MT), NISS = issuers_of(MT);
    const __half *sc = reinterpret_cast<const __half *>(aux.sc);
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;            // operand tiles need 1024-byte alignment
    const uint32_t raw_base = base + TC_ST * STAGE_BYTES;
    const uint32_t rawh_base = raw_base + TC_RAW * RAW_BYTES;
    constexpr bool CORR = corr_bytes(FMT, MT) > 0;
    constexpr int CORR_B_BYTES = corr_b_bytes(MT);
    const uint32_t corr_base = rawh_base + TC_RAW * rawh_bytes(FMT);     // [A_hi | A_lo | B_hi | B_lo], all 1024-byte aligned
    const uint32_t bar_base = corr_base + corr_bytes(FMT, MT);
    unsigned char *gen_base = smem_raw + (base - smem_u32(smem_raw));
    float *s_xscale = reinterpret_cast<float *>(gen_base + TC_ST * STAGE_BYTES + TC_RAW * (RAW_BYTES + rawh_bytes(FMT)) + corr_bytes(FMT, MT) + 512);
    unsigned char *corr_gen = gen_base + TC_ST * STAGE_BYTES + TC_RAW * (RAW_BYTES + rawh_bytes(FMT));
    auto xf_bar = [&](int s) { return bar_base + 8u * s; };                                 // activation tile landed
    auto af_bar = [&](int s) { return bar_base + 8u * (TC_ST + s); };                       // weight operand written
    auto e_bar = [&](int s) { return bar_base + 8u * (2 * TC_ST + s); };                    // stage consumed by every issuer's MMAs
    auto rawf_bar = [&](int s) { return bar_base + 8u * (3 * TC_ST + s); };                 // nibbles landed
    auto rawe_bar = [&](int s) { return bar_base + 8u * (3 * TC_ST + TC_RAW + s); };        // ... read by the dequantisers
    const uint32_t accum_bar = bar_base + 8u * (3 * TC_ST + 2 * TC_RAW);
    const uint32_t corr_bar = accum_bar + 8u;                                                // block sums of the correction staged

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r0 = blockIdx.x * TC_ROWS, m0 = blockIdx.z * MT;
    const int kb_begin = blockIdx.y * kb_per_split;
    const int n_kb = min(k_groups * 2, kb_begin + kb_per_split) - kb_begin;

    if (tid == 0) {
        s_abort = 0;
        // xf_bar(s): "stage s ready" = the activation tile has landed (one arrival carrying its byte count) and the eight warps
        // of the dequantiser group have written the weight operand: one probe per stage for the issuing threads
        for (int s = 0; s < TC_ST; s++) { mbar_init(xf_bar(s), 1 + TC_DEQ / 64); mbar_init(af_bar(s), 1); mbar_init(e_bar(s), NISS); }   // one arrival per warp:
        for (int s = 0; s < TC_RAW; s++) { mbar_init(rawf_bar(s), 1); mbar_init(rawe_bar(s), TC_DEQ / 32); }   // 512 arrivals on one word serialise
        mbar_init(accum_bar, NISS);
        mbar_init(corr_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // the tensor-core correction covers slices of up to CORR_U sub-blocks (32 stages); longer slices keep the epilogue loop
    const bool corr_mma = CORR && n_kb * 2 <= CORR_U;
    if (CORR) for (int i = tid; i < corr_bytes(FMT, MT) / 16; i += TC_THREADS) reinterpret_cast<uint4 *>(corr_gen)[i] = make_uint4(0, 0, 0, 0);
    if (CORR) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == TC_DEQ / 32) {   // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;
    // Up to here nothing depended on the kernel before this one in the stream, and neither do the weights: the first two
    // nibble tiles are requested before the wait for that kernel, whose tail then hides the set-up and the first DRAM latency.
    constexpr int RAW_EARLY = 2;
    if (warp == TC_DEQ / 32 + TC_ISSUERS && lane == 0) {
        for (int g = 0; g < RAW_EARLY && 2 * g < n_kb; g++) {
            mbar_arrive_expect_tx(rawf_bar(g), FMT == TC_Q6_K ? RAW_BYTES + RAWH_BYTES : RAW_BYTES);
            tma_load_2d(raw_base + g * RAW_BYTES, &map_w, ((kb_begin >> 1) + g) * 64, r0, rawf_bar(g));
            if (FMT == TC_Q6_K) tma_load_2d(rawh_base + g * RAWH_BYTES, &map_h, ((kb_begin >> 1) + g) * 32, r0, rawf_bar(g));
        }
    }
    vx_pdl_wait();
    if (tid < MT) s_xscale[tid] = m0 + tid < M ? xscale[m0 + tid] : 0.f;
    __syncthreads();

    if (warp < TC_DEQ / 32) {
        // ------------------------------------------------------------------ dequantisers
        // Two groups of eight warps take alternate stages, so the groups run out of phase and each scheduler always has
        // warps of both in flight.  Within a group, warp w owns the 32 operand rows (= tensor-memory lanes) of quadrant
        // w & 3 and the 32-weight block b of the stage: one thread turns one GGUF block of its row into 16 columns of
        // fp16 pairs, written with one 16-column store each for the hi and the lo part.
        const int grp = (warp >> 2) & 1, b = warp >> 3;
        const int row = (warp & 3) * 32 + lane;
        const int grow = min(r0 + row, N - 1);
        // nibble tile rows are 64 bytes with SWIZZLE_64B: 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3);
        // chunk c holds word c of the four nibble words of the 128-weight group
        const int rsw = (row >> 1) & 3;
        const uint32_t a_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + TMEM_A + 32 * b;
        if (FMT == TC_Q4_0) {
            // this thread's GGUF block is 2 * grp + b of the group: word index = block index
            const __half *scp = sc + (size_t)grow * k_groups * 4 + (size_t)kb_begin * 2 + b;
            int raw_off[4];
#pragma unroll
            for (int c = 0; c < 4; c++) raw_off[c] = row * 64 + ((c ^ rsw) << 4) + 4 * (2 * grp + b);
            __half d0 = grp < n_kb ? scp[2 * grp] : __float2half(0.f);
            for (int kb = grp; kb < n_kb; kb += 2) {
                const int as = kb % TC_ST, g = kb >> 1, slot = g % TC_RAW;
                const __half d1 = (kb + 2 < n_kb) ? scp[2 * (kb + 2)] : d0;        // scale of this group's next stage
                if (!mbar_wait(rawf_bar(slot), (g / TC_RAW) & 1, abort_flag)) break;
                const unsigned char *rp = gen_base + TC_ST * STAGE_BYTES + slot * RAW_BYTES;
                uint32_t w[4];
#pragma unroll
                for (int c = 0; c < 4; c++) w[c] = *reinterpret_cast<const uint32_t *>(rp + raw_off[c]);
                __syncwarp();
                if (lane == 0) mbar_arrive(rawe_bar(slot));
                if (kb >= TC_ST && !mbar_wait(e_bar(as), ((kb / TC_ST) - 1) & 1, abort_flag)) break;
                const __half2 dd = __half2half2(d0);
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int nib = 0; nib < 2; nib++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            // bytes e and e + 2 of word c: weights 16 nib + 4 c + {e, e + 2} of the block (the activation tiles
                            // carry the same order of k within every four), exact product d * (q - 8) as an fp16 pair
                            const __half2 q = nib2(w[c] >> (4 * nib + 8 * e));
                            const __half2 ph = __hmul2(q, dd);
                            const __half2 pl = __hfma2(q, dd, __hneg2(ph));
                            hi[8 * nib + 2 * c + e] = h2u(ph); lo[8 * nib + 2 * c + e] = h2u(pl);
                        }
                tmem_st32(a_lane + 64 * as, hi, lo);       // columns 32 b .. +15 the hi parts of K=16 steps 2b, 2b+1, .. +31 their lo parts
                d0 = d1;
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(xf_bar(as));
            }
        } else {
            // K-quants.  The stage of parity grp is 64-weight half grp of the 128-weight group; this thread expands its 32
            // weights 32 b .. 32 b + 31.  The float32 sub-block scale fl(d * sc) travels as an fp16 pair, so that
            // A_hi + A_lo = (d1_hi + d1_lo) * q to 2^-22: A_hi = fp16(q * d1_hi), A_lo = its FMA residual + q * d1_lo.
            //   Q4_K: sub-block u = 2 grp + b; words 2 grp and 2 grp + 1 of every chunk hold its positions 0-15 / 16-31 in the
            //         nibble b.  w = d1 q - dm is carried as d1 (q - 8) + (8 d1 - dm): the centred first term keeps the
            //         accumulator small (no cancellation against a large offset sum), the second is a constant per
            //         sub-block and is applied in the epilogue to the activations' block sums.
            //   Q6_K: word 2 grp + b of every chunk holds 16-weight sub-blocks 4 grp + 2 b (low nibbles) and + 1 (high nibbles);
            //         the top two bits come from the second tile (byte u of the chunk's 8, two bits per position).
            const uint2 *scq = reinterpret_cast<const uint2 *>(aux.sc) + (size_t)grow * k_groups + (kb_begin >> 1);
            const int g_abs0 = kb_begin >> 1;
            int raw_off[4], rawh_off[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                raw_off[c] = row * 64 + ((c ^ rsw) << 4) + (FMT == TC_Q4_K ? 8 * grp : 4 * (2 * grp + b));
                rawh_off[c] = row * 32 + c * 8 + 4 * grp + 2 * b;
            }
            auto sup = [&](int g) -> float2 {     // {d, dmin} (Q4_K) or {d, 0} (Q6_K) of the group's super-block
                if (FMT == TC_Q4_K) return __half22float2(reinterpret_cast<const __half2 *>(aux.aux)[(size_t)grow * (k_groups / 2) + ((g_abs0 + g) >> 1)]);
                return make_float2(__half2float(reinterpret_cast<const __half *>(aux.aux)[(size_t)grow * (k_groups / 2) + ((g_abs0 + g) >> 1)]), 0.f);
            };
            uint2 s8 = grp < n_kb ? scq[0] : make_uint2(0, 0);
            float2 dsup = grp < n_kb ? sup(0) : make_float2(0.f, 0.f);
            for (int kb = grp; kb < n_kb; kb += 2) {
                const int as = kb % TC_ST, g = kb >> 1, slot = g % TC_RAW;
                const uint2 s8n = (kb + 2 < n_kb) ? scq[g + 1] : s8;
                const float2 dsn = (kb + 2 < n_kb) ? sup(g + 1) : dsup;
                if (!mbar_wait(rawf_bar(slot), (g / TC_RAW) & 1, abort_flag)) break;
                const unsigned char *rp = gen_base + TC_ST * STAGE_BYTES + slot * RAW_BYTES;
                uint32_t w0[4], w1[4], hb[4];
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    if (FMT == TC_Q4_K) {
                        const uint2 t = *reinterpret_cast<const uint2 *>(rp + raw_off[c]);
                        w0[c] = t.x >> (4 * b); w1[c] = t.y >> (4 * b);           // positions 0-15 and 16-31, this sub-block's nibble
                        hb[c] = 0;
                    } else {
                        const uint32_t t = *reinterpret_cast<const uint32_t *>(rp + raw_off[c]);
                        w0[c] = t; w1[c] = t >> 4;                                 // sub-blocks 4 grp + 2 b and + 1
                        hb[c] = *reinterpret_cast<const unsigned short *>(gen_base + TC_ST * STAGE_BYTES + TC_RAW * RAW_BYTES + slot * RAWH_BYTES + rawh_off[c]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(rawe_bar(slot));
                if (kb >= TC_ST && !mbar_wait(e_bar(as), ((kb / TC_ST) - 1) & 1, abort_flag)) break;
                __half2 dh[2], dl[2];
                if (FMT == TC_Q4_K) {
                    const int u = 2 * grp + b;
                    const float d1 = __fmul_rn(dsup.x, (float)((s8.x >> (8 * u)) & 0xFF));                  // dequant.go:369-372
                    split_scale(d1, &dh[0], &dl[0]);
                    dh[1] = dh[0]; dl[1] = dl[0];
                    if (CORR && corr_mma) {
                        // constant of this sub-block, scaled by 2^10 to sit well inside the fp16 range (the block sums carry 2^-10)
                        const float ce = fmaf(8.f, d1, -__fmul_rn(dsup.y, (float)((s8.y >> (8 * u)) & 0xFF))) * 1024.f;
                        const __half ch = __float2half_rn(ce), cl = __float2half_rn(ce - __half2float(ch));
                        const int ul = 2 * kb + b;                                 // sub-block index within the slice = K position
                        const int off = row * 128 + (((ul >> 3) ^ (row & 7)) << 4) + (ul & 7) * 2;
                        *reinterpret_cast<__half *>(corr_gen + off) = ch;
                        *reinterpret_cast<__half *>(corr_gen + CORR_A_BYTES + off) = cl;
                    }
                } else {
                    const uint32_t sw = grp ? s8.y : s8.x;                        // int8 scales of sub-blocks 4 grp .. 4 grp + 3
                    split_scale(__fmul_rn(dsup.x, (float)(int)(signed char)((sw >> (16 * b)) & 0xFF)), &dh[0], &dl[0]);   // dequant.go:296-299
                    split_scale(__fmul_rn(dsup.x, (float)(int)(signed char)((sw >> (16 * b + 8)) & 0xFF)), &dh[1], &dl[1]);
                }
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int t = 0; t < 2; t++)
#pragma unroll
                    for (int c = 0; c < 4; c++)
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const uint32_t v = (t ? w1[c] : w0[c]) >> (8 * e);
                            __half2 q;
                            if (FMT == TC_Q4_K) q = nib2(v);          // q - 8: the offset 8 * d1 joins the minimum in the epilogue
                            else {
                                const uint32_t h8 = (hb[c] >> (8 * t)) & 0xFF;
                                q = q6h2(v, e ? (((h8 & 0x0C) << 2) | ((h8 & 0xC0) << 14)) : (((h8 & 0x03) << 4) | ((h8 & 0x30) << 16)));
                            }
                            const __half2 ph = __hmul2(q, dh[t]);
                            __half2 pl = __hfma2(q, dh[t], __hneg2(ph));
                            pl = __hfma2(q, dl[t], pl);
                            hi[8 * t + 2 * c + e] = h2u(ph); lo[8 * t + 2 * c + e] = h2u(pl);
                        }
                tmem_st32(a_lane + 64 * as, hi, lo);       // columns 32 b .. +15 the hi parts of K=16 steps 2b, 2b+1, .. +31 their lo parts
                s8 = s8n; dsup = dsn;
                if (CORR) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the constants are read by the MMA unit
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(xf_bar(as));
            }
        }
    } else if (warp == TC_DEQ / 32 + TC_ISSUERS) {
        // ------------------------------------------------------------------ TMA producer (one thread)
        if (lane == 0) {
            for (int kb = 0; kb < n_kb; kb++) {
                const int gkb = kb_begin + kb, xs = kb % TC_ST;
                if ((kb & 1) == 0 && (kb >> 1) >= RAW_EARLY) {
                    const int g = kb >> 1, slot = g % TC_RAW;
                    if (g >= TC_RAW && !mbar_wait(rawe_bar(slot), ((g / TC_RAW) - 1) & 1, abort_flag)) break;
                    mbar_arrive_expect_tx(rawf_bar(slot), FMT == TC_Q6_K ? RAW_BYTES + RAWH_BYTES : RAW_BYTES);
                    tma_load_2d(raw_base + slot * RAW_BYTES, &map_w, (gkb >> 1) * 64, r0, rawf_bar(slot));
                    if (FMT == TC_Q6_K) tma_load_2d(rawh_base + slot * RAWH_BYTES, &map_h, (gkb >> 1) * 32, r0, rawf_bar(slot));
                }
                if (kb >= TC_ST && !mbar_wait(e_bar(xs), ((kb / TC_ST) - 1) & 1, abort_flag)) break;
                mbar_arrive_expect_tx(xf_bar(xs), 2 * X_TILE);
                const uint32_t dst = base + xs * STAGE_BYTES;
                tma_load_2d(dst, &map_xh, gkb * TC_BK, m0, xf_bar(xs));
                tma_load_2d(dst + X_TILE, &map_xl, gkb * TC_BK, m0, xf_bar(xs));
            }
        }
    } else if (warp == TC_DEQ / 32 + TC_ISSUERS + 1) {
        // ------------------------------------------------------------------ helper warp: the activations' 32-block sums of this
        // slice as a K-major fp16 operand (hi and lo part, scaled by 2^-10), rows = batch rows, K = sub-blocks
        if (CORR && corr_mma) {
            const int U = n_kb * 2;
            for (int i = lane; i < MT * U; i += 32) {
                const int r = i / U, ul = i % U;
                const int m = min(m0 + r, M - 1);
                const float v = aux.xbsum[(size_t)m * aux.bsum_ld + (size_t)kb_begin * 2 + ul] * (1.0f / 1024.f);
                const __half vh = __float2half_rn(v), vl = __float2half_rn(v - __half2float(vh));
                const int off = r * 128 + (((ul >> 3) ^ (r & 7)) << 4) + (ul & 7) * 2;
                *reinterpret_cast<__half *>(corr_gen + 2 * CORR_A_BYTES + off) = vh;
                *reinterpret_cast<__half *>(corr_gen + 2 * CORR_A_BYTES + CORR_B_BYTES + off) = vl;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(corr_bar);
        }
    } else if (lane == 0 && warp < TC_DEQ / 32 + NISS) {
        // ------------------------------------------------------------------ MMA issue (one thread per issuer warp)
        // On a busy SM every tcgen05 instruction (mma or commit) costs its issuing thread ~80-100 cycles whatever its
        // shape, so the K=16 steps of a stage are shared between TC_ISSUERS threads on different schedulers, each with
        // its own accumulator (summed in the epilogue: the result stays deterministic), and a stage is released by a
        // single commit per issuer.  Per step: [A_hi] x [x_hi; x_lo] (N=128), then [A_lo] x [x_hi] (N=64).
        const int j = warp - TC_DEQ / 32;
        constexpr int KS = (TC_BK / 16) / NISS;                   // K=16 steps per issuer and stage
        uint64_t xdesc[TC_ST][KS];
#pragma unroll
        for (int s = 0; s < TC_ST; s++)
#pragma unroll
            for (int k = 0; k < KS; k++) xdesc[s][k] = umma_desc(base + s * STAGE_BYTES) + (uint64_t)(2 * (j * KS + k));   // +32 bytes of K per step
        const uint32_t acc = tmem + 2 * MT * j;
        bool ok = true;
        uint32_t first = 0u;
        for (int kb0 = 0; kb0 < n_kb && ok; kb0 += TC_ST) {
            const uint32_t par = (uint32_t)(kb0 / TC_ST) & 1u;
#pragma unroll
            for (int s = 0; s < TC_ST; s++) {
                if (kb0 + s >= n_kb) break;
                ok = mbar_wait(xf_bar(s), par, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // stage layout in tensor memory: [hi k0 k1 | lo k0 k1 | hi k2 k3 | lo k2 k3], 8 columns per K=16 step; issuer j owns steps 2j, 2j+1
                const uint32_t a_hi0 = tmem + TMEM_A + 64 * s + 32 * j * (KS / 2);
#pragma unroll
                for (int k = 0; k < KS; k++) {
                    const uint32_t a_hi = a_hi0 + 32 * (k >> 1) + 8 * (k & 1), a_lo = a_hi + 16;
                    umma_f16_ts(acc, a_hi, xdesc[s][k], umma_idesc(2 * MT), first);     // [x_hi; x_lo]: N = 2 MT
                    first = 1u;
                    umma_f16_ts(acc, a_lo, xdesc[s][k], umma_idesc(MT), 1u);            // x_hi only:   N = MT
                }
                umma_commit(e_bar(s));        // arrives when this issuer's MMAs have finished reading the stage
            }
        }
        if (CORR && corr_mma && ok && j == 0) {
            // every stage's "ready" barrier has been passed, so all constants are in place; wait for the block sums, then
            // acc[:, 0:MT] += C_hi B_hi + C_lo B_hi + C_hi B_lo over the slice's sub-blocks (K=16 per instruction)
            ok = mbar_wait(corr_bar, 0, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ah = umma_desc(corr_base), al = umma_desc(corr_base + CORR_A_BYTES);
                const uint64_t bh = umma_desc(corr_base + 2 * CORR_A_BYTES), bl = umma_desc(corr_base + 2 * CORR_A_BYTES + CORR_B_BYTES);
                const int steps = (n_kb * 2 + 15) / 16;
                for (int k = 0; k < steps; k++) {
                    umma_f16_ss(acc, ah + 2 * k, bh + 2 * k, umma_idesc(MT), 1u);
                    umma_f16_ss(acc, al + 2 * k, bh + 2 * k, umma_idesc(MT), 1u);
                    umma_f16_ss(acc, ah + 2 * k, bl + 2 * k, umma_idesc(MT), 1u);
                }
            }
        }
        if (ok) umma_commit(accum_bar);
    }

    // ------------------------------------------------------------------ epilogue: warp w reads lane quadrant w&3, columns 16*(w>>2)..
    __syncwarp();
    if (warp < TC_DEQ / 32) {
        bool ok = n_kb > 0 && mbar_wait(accum_bar, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            float *o = out + (size_t)blockIdx.y * part_stride;
            constexpr int CW = MT / 4;                                // batch columns per warp group
            const int n = r0 + (warp & 3) * 32 + lane, c0 = (warp >> 2) * CW;
            float sum[CW];
#pragma unroll
            for (int i = 0; i < CW; i++) sum[i] = 0.f;
#pragma unroll
            for (int part = 0; part < 2 * NISS; part++)               // issuer accumulators x {x_hi, x_lo} halves, fixed order
#pragma unroll
                for (int cb = 0; cb < CW / 16; cb++) {
                    uint32_t v[16];
                    VX_TMEM_LD16(v, tmem + ((uint32_t)((warp & 3) * 32) << 16) + part * MT + c0 + 16 * cb);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i++) sum[16 * cb + i] += __uint_as_float(v[i]);
                }
            if (FMT == TC_Q4_K && !corr_mma) {
                // plus sum over this slice's sub-blocks of (8 fl(d * sc_u) - fl(dmin * m_u)) * (sum of the activations of the sub-block)
                // (dequant.go:369-392: w = d1 * q - dm1)
                const int gn = min(n, N - 1);
                const uint2 *scq = reinterpret_cast<const uint2 *>(aux.sc) + (size_t)gn * k_groups + (kb_begin >> 1);
                const __half2 *supq = reinterpret_cast<const __half2 *>(aux.aux) + (size_t)gn * (k_groups / 2);
                for (int gi = 0; 2 * gi < n_kb; gi++) {
                    const int gabs = (kb_begin >> 1) + gi;
                    const uint2 sm8 = scq[gi];
                    const float2 dd = __half22float2(supq[gabs >> 1]);
                    float ce[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float d1 = __fmul_rn(dd.x, (float)((sm8.x >> (8 * u)) & 0xFF)), dm = __fmul_rn(dd.y, (float)((sm8.y >> (8 * u)) & 0xFF));
                        ce[u] = fmaf(8.f, d1, -dm);
                    }
#pragma unroll
                    for (int i = 0; i < CW; i++) {              // one 16-byte load brings the four sub-block sums of the group
                        const int m = min(m0 + c0 + i, M - 1);
                        const float4 bs = *reinterpret_cast<const float4 *>(aux.xbsum + (size_t)m * aux.bsum_ld + gabs * 4);
                        sum[i] = fmaf(ce[0], bs.x, fmaf(ce[1], bs.y, fmaf(ce[2], bs.z, fmaf(ce[3], bs.w, sum[i]))));
                    }
                }
            }
            if (n < N) {
#pragma unroll
                for (int i = 0; i < CW; i++) {
                    const int m = m0 + c0 + i;
                    if (m < M) o[(size_t)m * ld_out + n] = sum[i] * s_xscale[c0 + i];
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == TC_DEQ / 32) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (tid == 0 && s_abort) atomicExch(err_flag, VX_E_TIMEOUT);
}

}  // namespace

// Runs the self-test kernel with a wait limit of `limit_us` microseconds (clamped to [10, 100000]).  The kernel's status is
// reported by the next synchronising call (vx_sync returns VX_E_TIMEOUT), exactly as for the projection kernels; the
// context stays usable.  *reached_end tells that the kernel ran to its last line.
extern "C" int vx_selftest_bounded_wait(vx_ctx *c, int limit_us, int *reached_end) {
    if (!c || !reached_end) return VX_E_BAD_ARG;
    VxGuard g(c);
    limit_us = max(10, min(limit_us, 100000));
    int khz = 0;
    VX_CUDA(c, cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device));
    const long long limit_clocks = (long long)limit_us * (khz > 0 ? khz : 1500000) / 1000;
    int *d_flag = c->d_int_result + 9;
    VX_CUDA(c, cudaMemsetAsync(d_flag, 0, 4, c->stream));
    bounded_wait_selftest_kernel<<<1, 64, 0, c->stream>>>(limit_clocks, c->d_int_result + 8, d_flag);
    VX_LAUNCH_CHECK(c);
    VX_CUDA(c, cudaMemcpyAsync(c->h_int_result + 9, d_flag, 4, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    *reached_end = c->h_int_result[9];
    return VX_OK;
}

// same contract as vxq_gemm (vx_quant.cu); the context's device error word receives VX_E_TIMEOUT if a bounded wait gave up
int vxq_gemm_tc(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
                size_t parts_cap_floats) {
    if (vxq_gemm_tcp_eligible(w, m) && (w.type != VX_T_Q4_K || (parts && (size_t)2 * m * w.n <= parts_cap_floats)))   // (Q4_K needs a slot for its minima)
        return vxq_gemm_tcp(c, w, x, m, out, ld_out, n_parts_out, parts, parts_cap_floats);   // decode batches of Q4_0: the persistent kernel
    int *err_flag = c->d_int_result + 8;
    if (w.type != VX_T_Q4_0 && w.type != VX_T_Q4_K && w.type != VX_T_Q6_K) return vx_fail(c, VX_E_UNSUPPORTED, "tensor-core projection: weight type %d", w.type);
    if (x.k_pad != w.k_pad) return vx_fail(c, VX_E_BAD_ARG, "projection: activation row stride %d != weight k_pad %d", x.k_pad, w.k_pad);
    {
        static VxPerDevice a0, a1, a2, a3, a4, a5;
        VX_CUDA(c, a0.max_dynamic_smem(c, gemm_tc_kernel<TC_Q4_0, 64>, smem_bytes(TC_Q4_0, 64)));
        VX_CUDA(c, a1.max_dynamic_smem(c, gemm_tc_kernel<TC_Q4_K, 64>, smem_bytes(TC_Q4_K, 64)));
        VX_CUDA(c, a2.max_dynamic_smem(c, gemm_tc_kernel<TC_Q6_K, 64>, smem_bytes(TC_Q6_K, 64)));
        VX_CUDA(c, a3.max_dynamic_smem(c, gemm_tc_kernel<TC_Q4_0, 128>, smem_bytes(TC_Q4_0, 128)));
        VX_CUDA(c, a4.max_dynamic_smem(c, gemm_tc_kernel<TC_Q4_K, 128>, smem_bytes(TC_Q4_K, 128)));
        VX_CUDA(c, a5.max_dynamic_smem(c, gemm_tc_kernel<TC_Q6_K, 128>, smem_bytes(TC_Q6_K, 128)));
    }
    // batches above 64 rows (prefill chunks, verify) take 128-row tiles: the MMA count per stage stays the same, so each
    // dequantised weight tile and each tcgen05 instruction serves twice the rows
    const int mt = m > 64 ? 128 : 64;
    const int k_groups = w.k_pad / 128;
    const int tiles = ceil_div(w.n, TC_ROWS) * ceil_div(m, mt);
    // split-K (in whole 128-weight groups).  Cost model in units of one pipeline stage: a CTA pays its stages plus a fixed
    // set-up / drain / epilogue share (about eight stages' worth: the value was swept from 3 to 32 on three model shapes), CTAs run in waves of one per SM, and the
    // partial sums cost their write and read (mostly L2).  The cheapest split wins, the smaller one on near-ties.
    int split = 1;
    if (parts) {
        const int slots = c->sm_count;
        constexpr double OVERHEAD_STAGES = 8.0, PART_STAGES_PER_FLOAT = 2.2e-6;
        double best = 1e300;
        // Q4_K: slices of at most 16 groups (32 stages) keep the minima correction on the tensor cores
        const int s_min = w.type == VX_T_Q4_K ? min(8, ceil_div(k_groups, CORR_U / 4)) : 1;
        for (int s = 1; s <= 8 && s <= max(1, k_groups / 4); s++) {
            if ((size_t)s * m * w.n > parts_cap_floats) break;
            if (s < s_min && (size_t)s_min * m * w.n <= parts_cap_floats) continue;
            const int per = ceil_div(k_groups, s), s_eff = ceil_div(k_groups, per);
            const long n_cta = (long)tiles * s_eff;
            const double cost = (double)ceil_div64(n_cta, slots) * (2.0 * per + OVERHEAD_STAGES) +
                                (s_eff > 1 ? PART_STAGES_PER_FLOAT * s_eff * (double)m * w.n : 0.0);
            if (cost < best * 0.98) { best = cost; split = s; }
        }
    }
    int per = ceil_div(k_groups, split);
    split = ceil_div(k_groups, per);
    float *dst = split > 1 ? parts : out;
    int ld = split > 1 ? w.n : ld_out;
    *n_parts_out = split;
    // tensor maps: packed nibbles as bytes [n][k_groups*64], activations as fp16 [rows][k_pad].  A decode step launches the
    // same (weight, activation buffer, row count) combinations every time, so encoded maps are kept per combination instead
    // of paying four driver calls per launch.
    const uint64_t x_rows = (uint64_t)((m + 63) / 64) * 64;     // the split buffers are allocated in multiples of 64 rows
    struct MapKey {
        const void *qs, *hi, *xh, *xl; uint64_t rows; int n, kg, kp, mt;
        bool operator<(const MapKey &o) const {
            return std::tie(qs, hi, xh, xl, rows, n, kg, kp, mt) < std::tie(o.qs, o.hi, o.xh, o.xl, o.rows, o.n, o.kg, o.kp, o.mt);
        }
    };
    struct MapSet { CUtensorMap w, h, xh, xl; };
    static std::map<MapKey, MapSet> cache;
    static std::mutex cache_mu;
    const MapKey key{w.qs, w.type == VX_T_Q6_K ? w.hi : nullptr, x.hi, x.lo, x_rows, w.n, k_groups, x.k_pad, mt};
    MapSet ms;
    bool have = false;
    {
        std::lock_guard<std::mutex> lk(cache_mu);
        auto it = cache.find(key);
        if (it != cache.end()) { ms = it->second; have = true; }
    }
    CUtensorMap &map_w = ms.w, &map_h = ms.h, &map_xh = ms.xh, &map_xl = ms.xl;
    if (!have) {
    VX_TRY(make_map(c, &map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.qs, (uint64_t)k_groups * 64, (uint64_t)w.n, (uint64_t)k_groups * 64, 64,
                    TC_ROWS, CU_TENSOR_MAP_SWIZZLE_64B));
    VX_TRY(make_map(c, &map_xh, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x.hi, (uint64_t)x.k_pad, x_rows, (uint64_t)x.k_pad * 2, TC_BK, (uint32_t)mt,
                    CU_TENSOR_MAP_SWIZZLE_128B));
    VX_TRY(make_map(c, &map_xl, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x.lo, (uint64_t)x.k_pad, x_rows, (uint64_t)x.k_pad * 2, TC_BK, (uint32_t)mt,
                    CU_TENSOR_MAP_SWIZZLE_128B));
    // Q6_K: the top two bits of every weight as bytes [n][k_groups*32]; the other formats pass the nibble map again (unused)
    if (w.type == VX_T_Q6_K)
        VX_TRY(make_map(c, &map_h, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.hi, (uint64_t)k_groups * 32, (uint64_t)w.n, (uint64_t)k_groups * 32, 32,
                        TC_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE));
    else map_h = map_w;
        std::lock_guard<std::mutex> lk(cache_mu);
        if (cache.size() > 4096) cache.clear();     // buffers of destroyed models: start over rather than grow without bound
        cache[key] = ms;
    }
    dim3 grid(ceil_div(w.n, TC_ROWS), split, ceil_div(m, mt));
    const TcAux aux{w.sc, w.aux, x.bsum, x.k_pad / 32};
    const size_t pstride = (size_t)m * w.n;
    cudaError_t le = cudaSuccess;
#define VX_TC_LAUNCH(F, T) le = vx_launch_dependent(gemm_tc_kernel<F, T>, grid, dim3(TC_THREADS), (size_t)smem_bytes(F, T), c->stream, map_w, map_h, map_xh, map_xl, aux, (const float *)x.scale, dst, m, w.n, k_groups, per * 2, ld, pstride, err_flag)
    if (mt == 64) {
        if (w.type == VX_T_Q4_0) VX_TC_LAUNCH(TC_Q4_0, 64); else if (w.type == VX_T_Q4_K) VX_TC_LAUNCH(TC_Q4_K, 64); else VX_TC_LAUNCH(TC_Q6_K, 64);
    } else {
        if (w.type == VX_T_Q4_0) VX_TC_LAUNCH(TC_Q4_0, 128); else if (w.type == VX_T_Q4_K) VX_TC_LAUNCH(TC_Q4_K, 128); else VX_TC_LAUNCH(TC_Q6_K, 128);
    }
#undef VX_TC_LAUNCH
    if (le != cudaSuccess) return vx_cuda_fail(c, le, "projection launch");
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}
