// Q4_0, Q4_K and Q6_K projections for decode batches (17..64 rows) on tcgen05 + TMEM: the persistent form of the kernel
// in vx_gemm_tc.cu.  The text below describes the Q4_0 instance; the K-quant instances differ in the expansion step (the
// sub-block scale fl(d sc) carried as an fp16 pair, Q6_K with a second ring for its top-bit tiles, Q4_K with its minima
// term in a small kernel of its own that writes one more partial slot).
//
// What the one-CTA-per-tile kernel showed when its parts were switched off one at a time: nothing in it was saturated.  A
// CTA lived for 16-43 pipeline stages and spent a third of that filling its pipeline and draining its accumulator, a layer's
// projection needed two or three waves of such CTAs, and inside a stage the loads, the expansion of the weights, the
// tensor-memory stores and the MMAs ran one after the other (four stages in flight, tied to one ring).  Here:
//   * one CTA per SM walks (128-row weight tile, split-K slice) units; its rings keep running across unit boundaries, so the
//     pipeline is filled once per launch and the loads of the next unit are in flight while this one finishes;
//   * four epilogue warps take a finished unit out of the accumulators and hand them back as soon as it is in their
//     registers (a few hundred cycles per unit), then scale and store while the next unit's MMAs run;
//   * the rings are separate: activations eight stages deep, packed nibbles six 128-weight groups (twelve stages), block
//     scales as their own small tiles -- all fetched by TMA, so no dequantiser waits on a global load; two producer threads
//     (activations; weights), each a plain loop of one wait and one or two loads per item;
//   * four dequantiser groups of four warps, group g owning tensor-memory stage g: a thread expands both 32-weight blocks of
//     its row and stage, the first block before it waits for the stage to come free;
//   * two issuing warps on alternate stages, each with its own accumulator: the tensor pipe runs only while a thread is
//     issuing to it, so one warp's barrier probes and commit overlap the other's MMAs.
// Shape per stage as before ("swap-AB"): D[128 weight rows x 64 batch] += A[128 x 64k] * B^T, A = d (q - 8) as an exact fp16
// pair (A_hi + A_lo) in tensor memory, B = [x_hi; x_lo] stacked: A_hi x [x_hi; x_lo] (N = 128), then A_lo x x_hi (N = 64).
// Every TMA load targets this CTA only; every wait is bounded (a timeout raises the context's error word, the CTA drains
// what it has in flight, frees its tensor memory and returns).
#include <map>
#include <mutex>
#include <tuple>

#include "vx_tc.cuh"

namespace {
using namespace vxtc;

constexpr int P_MT = 64;                      // batch rows (MMA N / 2)
constexpr int P_BK = 64;                      // k per stage
constexpr int P_AST = 4;                      // weight-operand stages in tensor memory = dequantiser groups
constexpr int P_XST = 8;                      // activation stages in shared memory
constexpr int P_RAW = 6;                      // packed-nibble tiles (one 128-weight group = two stages each)
constexpr int P_SC = 4;                       // scale tiles (two groups = four stages each)
constexpr int P_X_TILE = P_MT * 128;          // one fp16 activation tile: 64 rows x 128 B
constexpr int P_STAGE_BYTES = 2 * P_X_TILE;   // x_hi rows, then x_lo rows
constexpr int P_RAW_BYTES = TC_ROWS * 64;
constexpr int P_SC_BYTES = TC_ROWS * 16;      // 128 rows x 8 scales
constexpr int P_RAWH_BYTES = TC_ROWS * 32;    // Q6_K only: the top two bits of a 128-weight group
enum { P_Q4_0 = 0, P_Q4_K = 1, P_Q6_K = 2 };
constexpr int P_DEQ_WARPS = 16, P_EPI_WARP0 = 16, P_ISSUE_WARP = 20, P_ISSUERS = 2, P_XPROD_WARP = 22, P_WPROD_WARP = 23;
constexpr int P_THREADS = 24 * 32;
constexpr int P_TMEM_ACC = 128;               // columns per accumulator (one per issuing warp): 0-63 = A_hi x_hi + A_lo x_hi, 64-127 = A_hi x_lo
constexpr int P_TMEM_A = P_ISSUERS * P_TMEM_ACC;      // weight stages start here, 64 columns each
constexpr int P_SMEM = P_XST * P_STAGE_BYTES + P_RAW * P_RAW_BYTES + P_SC * P_SC_BYTES + 1024 /*alignment*/ + 512 /*barriers*/ + 256 /*row scales*/;
constexpr int P_SMEM_Q6 = P_SMEM + P_RAW * P_RAWH_BYTES + 256;     // the high-bit tiles follow everything else
static_assert(P_TMEM_A + 64 * P_AST == 512, "tensor memory budget");
static_assert(P_SMEM_Q6 <= 232448, "shared memory budget");

#ifndef P_KNOCK
#define P_KNOCK 0      // timing experiments only (wrong results): 1 no weight expansion, 2 no operand stores, 4 no MMAs, 8 no activation loads, 16 no weight loads
#endif
// The units a CTA walks, in one of two modes.  Every role uses this iterator: divisions only when it is set up, additions
// from then on (a role is one thread's instruction stream, and an integer division costs it as much as a pipeline stage has
// to spare).
//   aligned: unit u = (row tile u / split, slice u % split) with slices of `per` groups; a CTA takes units blockIdx.x,
//            blockIdx.x + gridDim.x, ...
//   stream:  the stages of all tiles form one sequence (tile 0's K range, then tile 1's, ...) cut into gridDim.x equal runs
//            of whole quanta (a quantum = two 128-weight groups = four stages, the granularity of the scale tiles and of the
//            dequantiser groups); a CTA's run covers the tail of one tile, whole tiles, and the head of another.  Every CTA
//            then has the same number of stages (+- one quantum) whatever the tile count.  The CTAs that share a tile write
//            their partial sums to consecutive slots, in K order; the one that finishes a tile zero-fills the slots the tile
//            does not use, so that a consumer always sums `split` slots.
struct Unit { int r0, slice, g_begin, n_g; bool last; };
template <bool STREAM> struct UnitIter;
template <> struct UnitIter<false> {
    int tile, slice, d_tile, d_slice, split, per, k_groups;
    __device__ __forceinline__ UnitIter(int first, int stride, int split_, int per_, int k_groups_, int) : split(split_), per(per_), k_groups(k_groups_) {
        tile = first / split_; slice = first - tile * split_;
        d_tile = stride / split_; d_slice = stride - d_tile * split_;
    }
    __device__ __forceinline__ int count(int first, int stride, int n_units) const { return (n_units - first + stride - 1) / stride; }
    __device__ __forceinline__ Unit get() const {
        Unit U;
        U.slice = slice; U.r0 = tile * TC_ROWS; U.g_begin = slice * per; U.n_g = min(per, k_groups - U.g_begin); U.last = false;
        return U;
    }
    __device__ __forceinline__ void next() {
        tile += d_tile; slice += d_slice;
        if (slice >= split) { slice -= split; tile++; }
    }
};
template <> struct UnitIter<true> {
    int tile, slice, q, q_end, qt;                              // this CTA's quanta [q, q_end), quanta per tile
    __device__ __forceinline__ UnitIter(int first, int stride, int, int, int k_groups_, int stream_q) {
        qt = k_groups_ >> 1;
        q = (int)(((long long)first * stream_q) / stride); q_end = (int)(((long long)(first + 1) * stream_q) / stride);
        tile = q / qt;
        // slot of this CTA's first unit = how many CTAs before it touch the same tile: the first of them holds quantum tile * qt
        const int first_cta = (int)((((long long)tile * qt + 1) * stride + stream_q - 1) / stream_q) - 1;
        slice = first - first_cta;
    }
    __device__ __forceinline__ int count(int, int, int) const { return q_end > q ? (q_end - 1) / qt - q / qt + 1 : 0; }
    __device__ __forceinline__ Unit get() const {
        Unit U;
        const int off = q - tile * qt, n = min(q_end - q, qt - off);
        U.slice = slice; U.r0 = tile * TC_ROWS; U.g_begin = 2 * off; U.n_g = 2 * n; U.last = off + n == qt;
        return U;
    }
    __device__ __forceinline__ void next() { q = min(q_end, (tile + 1) * qt); tile++; slice = 0; }   // the next tile starts at its first quantum: this CTA is its first writer
};

#define VX_P_LD16(v, taddr) VX_TMEM_LD16(v, taddr)

// grid: one CTA per SM (or per unit when there are fewer); out layout [split][M][ld_out]; per and k_groups are even
template <bool STREAM, int FMT>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tcp_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s, const __grid_constant__ CUtensorMap map_x,
                const __grid_constant__ CUtensorMap map_h, const __half *__restrict__ sup,
                const float *__restrict__ xscale, float *__restrict__ out, int M, int N, int k_groups,
                int per, int split, int n_units, int stream_q, int ld_out, size_t part_stride, int *__restrict__ err_flag) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;            // operand tiles need 1024-byte alignment
    const uint32_t raw_base = base + P_XST * P_STAGE_BYTES;
    const uint32_t sc_base = raw_base + P_RAW * P_RAW_BYTES;
    const uint32_t bar_base = sc_base + P_SC * P_SC_BYTES;
    unsigned char *gen_base = smem_raw + (base - smem_u32(smem_raw));
    const unsigned char *raw_gen = gen_base + P_XST * P_STAGE_BYTES;
    const unsigned char *sc_gen = raw_gen + P_RAW * P_RAW_BYTES;
    float *s_xscale = reinterpret_cast<float *>(gen_base + P_XST * P_STAGE_BYTES + P_RAW * P_RAW_BYTES + P_SC * P_SC_BYTES + 512);
    const uint32_t rawh_base = bar_base + 1024;                              // (Q6_K) 16-byte aligned: every region before it is a multiple of 256 bytes
    const unsigned char *rawh_gen = gen_base + (rawh_base - base);
    auto xfull = [&](int s) { return bar_base + 8u * s; };                                  // activation stage landed
    auto done = [&](int s) { return bar_base + 8u * (P_XST + s); };                         // the MMAs of the stage in activation slot s have finished: the
                                                                                            // slot and the stage's weight operand in tensor memory are free
    auto rawfull = [&](int s) { return bar_base + 8u * (2 * P_XST + s); };                  // nibble tile landed
    auto rawempty = [&](int s) { return bar_base + 8u * (2 * P_XST + P_RAW + s); };         // ... read by both groups that use it
    auto scfull = [&](int s) { return bar_base + 8u * (2 * P_XST + 2 * P_RAW + s); };       // scale tile landed
    auto scempty = [&](int s) { return bar_base + 8u * (2 * P_XST + 2 * P_RAW + P_SC + s); };
    auto afull = [&](int s) { return bar_base + 8u * (2 * P_XST + 2 * P_RAW + 2 * P_SC + s); };                  // weight operand written
    const uint32_t accfull = bar_base + 8u * (2 * P_XST + 2 * P_RAW + 2 * P_SC + 2 * P_AST);       // a unit's MMAs are done (one commit per issuer)
    const uint32_t accempty = accfull + 8u;                                                         // ... and the accumulators are in registers

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);      // a broadcast value: the role branches below are warp-uniform
    const int n_my = UnitIter<STREAM>((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q).count((int)blockIdx.x, (int)gridDim.x, n_units);   // this CTA's units

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < P_XST; s++) { mbar_init(xfull(s), 1); mbar_init(done(s), 1); }
        for (int s = 0; s < P_RAW; s++) { mbar_init(rawfull(s), 1); mbar_init(rawempty(s), 8); }     // one arrival per warp of the two groups
        for (int s = 0; s < P_SC; s++) { mbar_init(scfull(s), 1); mbar_init(scempty(s), P_DEQ_WARPS); }
        for (int s = 0; s < P_AST; s++) mbar_init(afull(s), 4);
        mbar_init(accfull, P_ISSUERS); mbar_init(accempty, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == P_ISSUE_WARP) {   // the MMA warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int *abort_flag = &s_abort;

    if (warp < P_DEQ_WARPS) {
        // ------------------------------------------------------------------ dequantisers
        // Group fg = warp / 4 owns tensor-memory stage fg and expands the stages kb = fg (mod 4) of every unit (a unit has a
        // multiple of four stages, so this holds across units); within the group a warp owns the 32 operand rows (tensor-memory
        // lanes) of quadrant warp % 4.  Weights and scales do not depend on the kernel before this one, so this role never
        // waits for it.
        const int fg = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        // nibble tile rows are 64 bytes with SWIZZLE_64B: 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3); chunk c holds
        // word c of the four blocks of the 128-weight group; this thread's stage is blocks 2 (fg & 1) and + 1
        const int rsw = (row >> 1) & 3;
        int raw_off[4];
#pragma unroll
        for (int c = 0; c < 4; c++) raw_off[c] = row * 64 + ((c ^ rsw) << 4) + 8 * (fg & 1);
        // scale tile: row r holds the eight block scales of two groups; this thread's stage is group (fg >> 1) & 1 of the pair
        const int sc_off = row * 16 + (((fg >> 1) & 1) * 4 + (fg & 1) * 2) * 2;
        const uint32_t a_st = tmem + ((uint32_t)((warp & 3) * 32) << 16) + P_TMEM_A + 64 * fg;
        int it = 0, g_count = 0, t_count = 0;        // this group's iterations; nibble tiles and scale tiles before the current unit
        __half dsup_h = __float2half(0.f);          // (Q6_K) super-block scale of this thread's next stage
        const __half *sup_row = nullptr;
        __half2 dsup2 = __float2half2_rn(0.f);      // (Q4_K) {d, dmin} of this thread's next stage
        const __half2 *sup2_row = nullptr;
        bool ok = true;
        UnitIter<STREAM> uit((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q);
        for (int ui = 0; ui < n_my && ok; ui++, uit.next()) {
            const Unit U = uit.get();
            const int n_kb = 2 * U.n_g;
            if constexpr (FMT == P_Q6_K) {
                sup_row = sup + (size_t)min(U.r0 + row, N - 1) * (k_groups >> 1);
                if (fg < n_kb) dsup_h = __ldg(sup_row + ((U.g_begin + (fg >> 1)) >> 1));
            }
            if constexpr (FMT == P_Q4_K) {
                sup2_row = reinterpret_cast<const __half2 *>(sup) + (size_t)min(U.r0 + row, N - 1) * (k_groups >> 1);
                if (fg < n_kb) dsup2 = __ldg(sup2_row + ((U.g_begin + (fg >> 1)) >> 1));
            }
            for (int kb = fg; kb < n_kb; kb += P_AST, it++) {
                const int gi = g_count + (kb >> 1), ti = t_count + (kb >> 2);
                const int slot = gi % P_RAW, ss = ti % P_SC;
                if (!mbar_wait(scfull(ss), (uint32_t)(ti / P_SC) & 1u, abort_flag)) { ok = false; break; }
                if constexpr (FMT == P_Q4_K) {
                    // Q4_K (inference/pkg/gguf/dequant.go:342-396): the stage is 64-weight half `fg & 1` of the 128-weight group =
                    // sub-blocks 2 (fg & 1) + b; the same two words of every chunk hold positions 0-15 / 16-31 of both sub-blocks,
                    // b selects the nibble.  w = d1 q - dm1 is carried as d1 (q - 8) + (8 d1 - dm1): the centred term goes through
                    // the tensor cores with fl(d * sc) as an fp16 pair, the constant per sub-block meets the activations' block
                    // sums in a kernel of its own (q4k_minima_kernel), whose result is one more partial-sum slot.
                    const uint32_t scw = *reinterpret_cast<const uint32_t *>(sc_gen + ss * P_SC_BYTES + row * 16 + ((fg >> 1) & 1) * 8);
                    const float dsup = __low2float(dsup2);
                    {   // {d, dmin} of this group's next stage (one pair per 256 weights)
                        const int kbn = kb + P_AST < n_kb ? kb + P_AST : kb;
                        dsup2 = __ldg(sup2_row + ((U.g_begin + (kbn >> 1)) >> 1));
                    }
                    if (!mbar_wait(rawfull(slot), (uint32_t)(gi / P_RAW) & 1u, abort_flag)) { ok = false; break; }
                    const unsigned char *rp = raw_gen + slot * P_RAW_BYTES;
                    uint2 w[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) w[c] = *reinterpret_cast<const uint2 *>(rp + raw_off[c]);
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(scempty(ss)); mbar_arrive(rawempty(slot)); }
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int b = 0; b < 2; b++) {
                        __half2 dh, dl;
                        split_scale(__fmul_rn(dsup, (float)((scw >> (8 * (2 * (fg & 1) + b))) & 0xFF)), &dh, &dl);                 // dequant.go:369-372
#pragma unroll
                        for (int t = 0; t < 2; t++)
#pragma unroll
                            for (int c = 0; c < 4; c++)
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    const uint32_t word = t ? w[c].y : w[c].x;
                                    const __half2 q = nib2(word >> (4 * b + 8 * e));           // q - 8
                                    const __half2 ph = __hmul2(q, dh);
                                    __half2 pl = __hfma2(q, dh, __hneg2(ph));
                                    pl = __hfma2(q, dl, pl);
                                    hi[8 * t + 2 * c + e] = h2u(ph); lo[8 * t + 2 * c + e] = h2u(pl);
                                }
                        if (b == 0) {       // the first block is expanded before the stage is known to be free
                            if (it >= 1 && !mbar_wait(done((4 * (it - 1) + fg) & (P_XST - 1)), (uint32_t)((4 * (it - 1) + fg) / P_XST) & 1u, abort_flag)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        tmem_st32(a_st + 32 * b, hi, lo);
                    }
                    if (!ok) break;
                } else if constexpr (FMT == P_Q6_K) {
                    // Q6_K (inference/pkg/gguf/dequant.go:272-331): the stage is 64-weight half `fg & 1` of the 128-weight group; word
                    // 2 (fg & 1) + b of every chunk holds the 16-weight sub-blocks 4 (fg & 1) + 2 b (low nibbles) and + 1 (high
                    // nibbles), the top two bits come from the second tile; fl(d * sc) travels as an fp16 pair so that
                    // A_hi + A_lo = d1 (q - 32) to 2^-22.
                    const uint32_t sw = *reinterpret_cast<const uint32_t *>(sc_gen + ss * P_SC_BYTES + row * 16 + ((fg >> 1) & 1) * 8 + (fg & 1) * 4);
                    const float dsup = __half2float(dsup_h);
                    {   // the super-block scale of this group's next stage (two 128-weight groups further on: one scale per 256 weights)
                        const int kbn = kb + P_AST < n_kb ? kb + P_AST : kb;
                        dsup_h = __ldg(sup_row + ((U.g_begin + (kbn >> 1)) >> 1));
                    }
                    if (!mbar_wait(rawfull(slot), (uint32_t)(gi / P_RAW) & 1u, abort_flag)) { ok = false; break; }
                    const unsigned char *rp = raw_gen + slot * P_RAW_BYTES, *hp = rawh_gen + slot * P_RAWH_BYTES + row * 32 + 4 * (fg & 1);
                    uint2 w[4]; uint32_t hw[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) { w[c] = *reinterpret_cast<const uint2 *>(rp + raw_off[c]); hw[c] = *reinterpret_cast<const uint32_t *>(hp + 8 * c); }
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(scempty(ss)); mbar_arrive(rawempty(slot)); }
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int b = 0; b < 2; b++) {
                        __half2 dh[2], dl[2];
                        split_scale(__fmul_rn(dsup, (float)(int)(signed char)((sw >> (16 * b)) & 0xFF)), &dh[0], &dl[0]);        // dequant.go:296-299
                        split_scale(__fmul_rn(dsup, (float)(int)(signed char)((sw >> (16 * b + 8)) & 0xFF)), &dh[1], &dl[1]);
#pragma unroll
                        for (int t = 0; t < 2; t++)
#pragma unroll
                            for (int c = 0; c < 4; c++)
#pragma unroll
                                for (int e = 0; e < 2; e++) {
                                    const uint32_t word = b ? w[c].y : w[c].x;
                                    const uint32_t v = (t ? word >> 4 : word) >> (8 * e);
                                    // byte 2 b + t of hw[c]: bits [1:0], [3:2], [5:4], [7:6] are the top bits of positions 0..3.  One
                                    // multiply copies the two fields of a pair to bits 4-5 and 20-21 (and to places the mask drops):
                                    // pair (0, 2): x = h & 0x33, (x << 4 | x << 16);  pair (1, 3): y = h & 0xCC, (y << 2 | y << 14)
                                    const uint32_t h8 = hw[c] >> (16 * b + 8 * t);
                                    const uint32_t h6 = (e ? (h8 & 0xCCu) * 0x4004u : (h8 & 0x33u) * 0x10010u) & 0x00300030u;
                                    const __half2 q = q6h2(v, h6);
                                    const __half2 ph = __hmul2(q, dh[t]);
                                    __half2 pl = __hfma2(q, dh[t], __hneg2(ph));
                                    pl = __hfma2(q, dl[t], pl);
                                    hi[8 * t + 2 * c + e] = h2u(ph); lo[8 * t + 2 * c + e] = h2u(pl);
                                }
                        if (b == 0) {       // the first block is expanded before the stage is known to be free
                            if (it >= 1 && !mbar_wait(done((4 * (it - 1) + fg) & (P_XST - 1)), (uint32_t)((4 * (it - 1) + fg) / P_XST) & 1u, abort_flag)) { ok = false; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        tmem_st32(a_st + 32 * b, hi, lo);
                    }
                    if (!ok) break;
                } else {
                    const __half2 d2 = *reinterpret_cast<const __half2 *>(sc_gen + ss * P_SC_BYTES + sc_off);
                    if (!mbar_wait(rawfull(slot), (uint32_t)(gi / P_RAW) & 1u, abort_flag)) { ok = false; break; }
                    const unsigned char *rp = raw_gen + slot * P_RAW_BYTES;
                    uint2 w[4];
#pragma unroll
                    for (int c = 0; c < 4; c++) w[c] = *reinterpret_cast<const uint2 *>(rp + raw_off[c]);
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(scempty(ss)); mbar_arrive(rawempty(slot)); }
                    uint32_t hi[16], lo[16];
                    // bytes e and e + 2 of word c: weights 16 nib + 4 c + {e, e + 2} of the block (the activation tiles carry the same
                    // order of k within every four), exact product d * (q - 8) as an fp16 pair
#define VX_P_EXPAND(WORD, DD)                                                              \
    _Pragma("unroll") for (int nib = 0; nib < 2; nib++)                                    \
    _Pragma("unroll") for (int c = 0; c < 4; c++)                                          \
    _Pragma("unroll") for (int e = 0; e < 2; e++) {                                        \
            if (P_KNOCK & 1) { hi[8 * nib + 2 * c + e] = w[c].WORD; lo[8 * nib + 2 * c + e] = h2u(DD); } else {   \
            /* low nibbles: 0x6400 | q = 1024 + q, minus 1032; high nibbles in place: (1024 + 16 q) / 16 - 72, one exact FMA */ \
        const uint32_t wv = e ? w[c].WORD >> 8 : w[c].WORD;                                \
        const uint32_t hb = (wv & (nib ? 0x00F000F0u : 0x000F000Fu)) | 0x64006400u;        \
        const __half2 q = nib ? __hfma2(*reinterpret_cast<const __half2 *>(&hb), __half2half2(__ushort_as_half((unsigned short)0x2C00)), \
                                        __half2half2(__ushort_as_half((unsigned short)0xD480)))                                            \
                              : __hsub2(*reinterpret_cast<const __half2 *>(&hb), __half2half2(__ushort_as_half((unsigned short)0x6408))); \
            const __half2 ph = __hmul2(q, DD);                                                 \
            const __half2 pl = __hfma2(q, DD, __hneg2(ph));                                    \
            hi[8 * nib + 2 * c + e] = h2u(ph); lo[8 * nib + 2 * c + e] = h2u(pl); }            \
        }
                    const __half2 dd0 = __half2half2(__low2half(d2)), dd1 = __half2half2(__high2half(d2));
                    VX_P_EXPAND(x, dd0)                          // the first block is expanded before the stage is known to be free
                    // this group's previous stage, global index 4 (it - 1) + fg, sat in activation slot (4 (it - 1) + fg) % 8
                    if (it >= 1 && !mbar_wait(done((4 * (it - 1) + fg) & (P_XST - 1)), (uint32_t)((4 * (it - 1) + fg) / P_XST) & 1u, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (P_KNOCK & 2) asm volatile("" :: "r"(hi[0]), "r"(hi[15]), "r"(lo[3]), "r"(lo[12])); else
                    tmem_st32(a_st, hi, lo);                     // columns 0-15 hi, 16-31 lo of K=16 steps 0, 1; in flight while the second block is expanded
                    VX_P_EXPAND(y, dd1)
                    if (P_KNOCK & 2) asm volatile("" :: "r"(hi[0]), "r"(hi[15]), "r"(lo[3]), "r"(lo[12])); else
                    tmem_st32(a_st + 32, hi, lo);                // K=16 steps 2, 3
#undef VX_P_EXPAND
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(afull(fg));
            }
            g_count += U.n_g; t_count += U.n_g >> 1;
        }
    } else if (warp == P_XPROD_WARP) {
        // ------------------------------------------------------------------ activation producer (one thread): per stage one wait, one
        // expect_tx and ONE load -- x_hi and x_lo are the two planes of a 3-D tensor map, so both tiles arrive with one TMA
        // instruction.  (A single producer thread polling three streams, with a division per unit, took ~900 cycles per stage
        // and was what every other role waited for.)
        if (lane == 0) {
            vx_pdl_wait();                                   // the activations are the output of the kernel ahead of this one in the stream
            UnitIter<STREAM> uit((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q);
            int xc = 0;
            bool ok = true;
            for (int ui = 0; ui < n_my && ok; ui++, uit.next()) {
                const Unit U = uit.get();
                const int n_kb = 2 * U.n_g;
                int kcoord = U.g_begin * 2 * P_BK;
                for (int kb = 0; kb < n_kb; kb++, xc++, kcoord += P_BK) {
                    const int slot = xc & (P_XST - 1);
                    if (xc >= P_XST && !mbar_wait(done(slot), (uint32_t)(xc / P_XST - 1) & 1u, abort_flag)) { ok = false; break; }
                    if (P_KNOCK & 8) { mbar_arrive(xfull(slot)); continue; }
                    mbar_arrive_expect_tx(xfull(slot), P_STAGE_BYTES);
                    tma_load_3d(base + slot * P_STAGE_BYTES, &map_x, kcoord, 0, 0, xfull(slot));
                }
            }
        }
    } else if (warp == P_WPROD_WARP) {
        // ------------------------------------------------------------------ weight producer (one thread): nibble tiles (one per 128-weight
        // group) and scale tiles (one per two groups), in the order the dequantisers need them.  Weights do not depend on the
        // kernel ahead of this one, so this role never waits for it: the rings fill while that kernel finishes.
        if (lane == 0) {
            UnitIter<STREAM> uit((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q);
            int rc = 0, scn = 0;
            bool ok = true;
            for (int ui = 0; ui < n_my && ok; ui++, uit.next()) {
                const Unit U = uit.get();
                // row-major arrays: nibbles [n][k_groups * 64 B], scales [n][k_groups * 8 B]; a box is 128 rows x 64 (16) bytes
                int raw_col = U.g_begin * 64, sc_col = U.g_begin * 8;
                for (int g = 0; g < U.n_g; g++, rc++, raw_col += 64) {
                    if ((g & 1) == 0) {
                        const int ss = scn & (P_SC - 1);
                        if (scn >= P_SC && !mbar_wait(scempty(ss), (uint32_t)(scn / P_SC - 1) & 1u, abort_flag)) { ok = false; break; }
                        if (P_KNOCK & 16) mbar_arrive(scfull(ss)); else {
                        mbar_arrive_expect_tx(scfull(ss), P_SC_BYTES);
                        tma_load_2d(sc_base + ss * P_SC_BYTES, &map_s, sc_col, U.r0, scfull(ss)); }
                        scn++; sc_col += 16;
                    }
                    const int slot = rc % P_RAW;
                    if (rc >= P_RAW && !mbar_wait(rawempty(slot), (uint32_t)(rc / P_RAW - 1) & 1u, abort_flag)) { ok = false; break; }
                    if (P_KNOCK & 16) mbar_arrive(rawfull(slot)); else {
                    mbar_arrive_expect_tx(rawfull(slot), FMT == P_Q6_K ? P_RAW_BYTES + P_RAWH_BYTES : P_RAW_BYTES);
                    tma_load_2d(raw_base + slot * P_RAW_BYTES, &map_w, raw_col, U.r0, rawfull(slot));
                    if (FMT == P_Q6_K) tma_load_2d(rawh_base + slot * P_RAWH_BYTES, &map_h, raw_col >> 1, U.r0, rawfull(slot)); }
                }
            }
        }
    } else if (warp >= P_ISSUE_WARP && warp < P_ISSUE_WARP + P_ISSUERS) {
        // ------------------------------------------------------------------ MMA issue
        // A thread that issues tcgen05.mma is held until the tensor pipe takes the instruction, and the pipe queues next to
        // nothing: measured alone, the eight MMAs of a stage take the issuing thread 384 cycles, and every other instruction
        // it executes between stages (barrier probes ~45 cycles each, a commit ~50, a wait ~90) is added to the stage time
        // with the pipe idle.  So two warps on different schedulers take alternate stages, each into its own accumulator
        // (summed in a fixed order by the epilogue): while one runs its probes and its commit, the pipe works for the other.
        // The warp runs its loop converged and one elected lane issues, so addresses and descriptors stay warp-uniform.
        const int j = warp - P_ISSUE_WARP;
        int gs = 0;                                           // stages before the current unit (a multiple of four)
        bool ok = true;
        const bool leader = elect_one();
        const uint32_t acc = tmem + P_TMEM_ACC * j;
        UnitIter<STREAM> uit((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q);
        for (int ui = 0; ui < n_my && ok; ui++, uit.next()) {
            const Unit U = uit.get();
            const int n_kb = 2 * U.n_g;
            if (ui >= 1) {                                    // the epilogue must have read the previous unit out of the accumulators
                ok = __all_sync(0xffffffffu, mbar_wait(accempty, (uint32_t)(ui - 1) & 1u, abort_flag));
                if (!ok) break;
            }
            uint32_t first = 0u;
#pragma unroll 2
            for (int kb = j; kb < n_kb; kb += P_ISSUERS) {
                const int gsi = gs + kb;
                const int s = kb & (P_AST - 1), xs = gsi & (P_XST - 1);
                const uint32_t pa = (uint32_t)(gsi / P_AST) & 1u, px = (uint32_t)(gsi / P_XST) & 1u;
                const bool ra = mbar_try(afull(s), pa), rx = mbar_try(xfull(xs), px);     // probed back to back; the slow path is out of line
                if (!(ra && rx)) {
                    ok = mbar_wait(afull(s), pa, abort_flag) && mbar_wait(xfull(xs), px, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (leader) {
                    // stage layout in tensor memory: [hi k0 k1 | lo k0 k1 | hi k2 k3 | lo k2 k3], 8 columns per K=16 step
                    const uint32_t a0 = tmem + P_TMEM_A + 64 * s;
                    const uint64_t xd = umma_desc(base + xs * P_STAGE_BYTES);
#pragma unroll
                    for (int k = 0; k < P_BK / 16; k++) {
                        const uint32_t a_hi = a0 + 32 * (k >> 1) + 8 * (k & 1), a_lo = a_hi + 16;
                        if ((P_KNOCK & 4) && !(kb < 2 && k == 0)) continue;
                        umma_f16_ts(acc, a_hi, xd + (uint64_t)(2 * k), umma_idesc(2 * P_MT), k == 0 ? first : 1u);    // [x_hi; x_lo]: N = 128; +32 bytes of K per step
                        umma_f16_ts(acc, a_lo, xd + (uint64_t)(2 * k), umma_idesc(P_MT), 1u);                        // x_hi only:   N = 64
                    }
                    umma_commit(done(xs));                // one commit releases the activation slot and the weight stage
                    if (kb + P_ISSUERS >= n_kb) umma_commit(accfull);
                }
                first = 1u;
            }
            gs += n_kb;
        }
    } else if (warp >= P_EPI_WARP0 && warp < P_EPI_WARP0 + 4) {
        // ------------------------------------------------------------------ epilogue: warp w reads the 32 accumulator lanes of quadrant
        // w % 4 (one weight row per lane), adds the x_hi and x_lo halves, applies the batch rows' power-of-two scales and stores;
        // the accumulator is handed back as soon as it is in registers
        vx_pdl_wait();                                       // the scales are the previous kernel's output, and `out` may still be read by it
        const int q = warp & 3;
        for (int i = tid - P_EPI_WARP0 * 32; i < P_MT; i += 128) s_xscale[i] = i < M ? xscale[i] : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps only
        bool ok = true;
        UnitIter<STREAM> uit((int)blockIdx.x, (int)gridDim.x, split, per, k_groups, stream_q);
        for (int ui = 0; ui < n_my && ok; ui++, uit.next()) {
            const Unit U = uit.get();
            ok = mbar_wait(accfull, (uint32_t)ui & 1u, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t0 = tmem + ((uint32_t)(q * 32) << 16);
            float v[P_MT];
#pragma unroll
            for (int cb = 0; cb < P_MT / 16; cb++) {              // issuer 0's x_hi and x_lo halves, then issuer 1's: a fixed order
                uint32_t a[16], c2[16], a1[16], c3[16];
                VX_P_LD16(a, t0 + 16 * cb);
                VX_P_LD16(c2, t0 + P_MT + 16 * cb);
                VX_P_LD16(a1, t0 + P_TMEM_ACC + 16 * cb);
                VX_P_LD16(c3, t0 + P_TMEM_ACC + P_MT + 16 * cb);
                float sx[16];                                     // the batch rows' scales, applied here so that the stores below depend on nothing
#pragma unroll
                for (int i = 0; i < 4; i++) *reinterpret_cast<float4 *>(&sx[4 * i]) = *reinterpret_cast<const float4 *>(s_xscale + 16 * cb + 4 * i);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float t = ((__uint_as_float(a[i]) + __uint_as_float(c2[i])) + __uint_as_float(a1[i])) + __uint_as_float(c3[i]);
                    v[16 * cb + i] = t * sx[i];
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(accempty);
            const int n = U.r0 + q * 32 + lane;
            if (n < N) {
                float *o = out + (size_t)U.slice * part_stride + n;
                if (M == P_MT) {
#pragma unroll
                    for (int m = 0; m < P_MT; m++) { *o = v[m]; o += ld_out; }
                } else {
#pragma unroll
                    for (int m = 0; m < P_MT; m++) { if (m < M) *o = v[m]; o += ld_out; }
                }
                if (STREAM && U.last) {                       // stream mode: the tile is complete; the slots it does not use count as zero
                    for (int sl = U.slice + 1; sl < split; sl++) {
                        float *z = out + (size_t)sl * part_stride + n;
                        for (int m = 0; m < M; m++) { *z = 0.f; z += ld_out; }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == P_ISSUE_WARP) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
    if (tid == 0 && s_abort) atomicExch(err_flag, VX_E_TIMEOUT);
}

}  // namespace

// Q4_K minima: out[m][n] = s_m * sum_u (8 fl(d sc_u) - fl(dmin m_u)) * bsum[m][u] over all 32-weight sub-blocks u of row n
// (dequant.go:369-392: w = d1 q - dm1, and the projection kernel carries d1 (q - 8)).  A small GEMM (K = k / 32) on
// mma.sync.m16n8k16: the constants (times 2^8) and the block sums (times 2^-6, they reach 32 * 2048) are staged in shared
// memory as exact fp16 hi + lo pairs, weight rows are the M dimension (a warp owns 16 of them), batch rows the N dimension
// (eight tiles of 8), three MMAs per tile and K step (hi hi, lo hi, hi lo), float32 accumulation.  As float32 FMAs on
// 4 x 4 register tiles the same product took 30 us for the 28672-row gate/up matrix -- as long as two thirds of the
// projection it corrects.  Its result is written as one more partial-sum slot, which the consumer adds like the others.
constexpr int MN_U = 128;                 // sub-blocks staged per round
constexpr int MN_LD = MN_U + 8;           // row stride in halves: 68 words, so a fragment load touches 32 different banks
__device__ __forceinline__ void mn_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mn_split4(const float (&v)[4], __half *hi, __half *lo) {     // four values -> fp16 hi and lo parts, 8-byte stores
    __half h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) { h[i] = __float2half_rn(v[i]); l[i] = __float2half_rn(v[i] - __half2float(h[i])); }
    *reinterpret_cast<uint2 *>(hi) = make_uint2((uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16),
                                                (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
    *reinterpret_cast<uint2 *>(lo) = make_uint2((uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[1]) << 16),
                                                (uint32_t)__half_as_ushort(l[2]) | ((uint32_t)__half_as_ushort(l[3]) << 16));
}
template <int ROWS>
__global__ void __launch_bounds__(2 * ROWS) q4k_minima_kernel(const uint2 *__restrict__ sc, const __half2 *__restrict__ sup, const float *__restrict__ xbsum,
                                                              int bsum_ld, const float *__restrict__ xscale, float *__restrict__ out, int M, int N,
                                                              int k_groups, int ld_out) {
    extern __shared__ __align__(16) __half mn_smem[];
    __half *ceh = mn_smem, *cel = ceh + ROWS * MN_LD;                  // [weight row][sub-block]
    __half *bsh = cel + ROWS * MN_LD, *bsl = bsh + P_MT * MN_LD;       // [batch row][sub-block]
    vx_pdl_wait();
    vx_pdl_trigger();
    constexpr int NT = 2 * ROWS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * ROWS;
    float acc[8][4];                                        // tile t: weight rows 16 warp + {g, g + 8}, batch rows 8 t + {2c, 2c + 1}
#pragma unroll
    for (int t = 0; t < 8; t++) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f; }
    const int n_u = k_groups * 4;
    for (int u0 = 0; u0 < n_u; u0 += MN_U) {
        if (u0) __syncthreads();
        // Staging, eight items per thread at a time with all eight global loads issued before the first is used (as a plain
        // loop the rounds of dependent loads, ~1 us each, were most of the kernel's time).
        // constants: (weight row, group) items, groups fastest: 8-byte loads of a row's scale bytes side by side
        for (int base = 0; base < ROWS * (MN_U / 4); base += 8 * NT) {
            uint2 sm8[8]; __half2 dd2[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int i = base + j * NT + tid;
                const int gl = i % (MN_U / 4), r = i / (MN_U / 4), gq = min((u0 >> 2) + gl, k_groups - 1);
                const int gn = min(n0 + min(r, ROWS - 1), N - 1);
                sm8[j] = __ldg(sc + (size_t)gn * k_groups + gq);
                dd2[j] = __ldg(sup + (size_t)gn * (k_groups >> 1) + (gq >> 1));
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int i = base + j * NT + tid;
                if (i < ROWS * (MN_U / 4)) {
                    const int gl = i % (MN_U / 4), r = i / (MN_U / 4);
                    const bool live = (u0 >> 2) + gl < k_groups;
                    const float2 dd = __half22float2(dd2[j]);
                    float c4[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const float d1 = __fmul_rn(dd.x, (float)((sm8[j].x >> (8 * u)) & 0xFF)), dm = __fmul_rn(dd.y, (float)((sm8[j].y >> (8 * u)) & 0xFF));
                        c4[u] = live ? fmaf(8.f, d1, -dm) * 256.f : 0.f;
                    }
                    mn_split4(c4, ceh + r * MN_LD + 4 * gl, cel + r * MN_LD + 4 * gl);
                }
            }
        }
        // block sums: (batch row, group) items, groups fastest
        for (int base = 0; base < P_MT * (MN_U / 4); base += 8 * NT) {
            float4 v8[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int i = min(base + j * NT + tid, P_MT * (MN_U / 4) - 1);
                const int gl = i % (MN_U / 4), mrow = i / (MN_U / 4);
                v8[j] = __ldg(reinterpret_cast<const float4 *>(xbsum + (size_t)min(mrow, M - 1) * bsum_ld + min(u0 + 4 * gl, n_u - 4)));
            }
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int i = base + j * NT + tid;
                if (i < P_MT * (MN_U / 4)) {
                    const int gl = i % (MN_U / 4), mrow = i / (MN_U / 4);
                    const float f = u0 + 4 * gl < n_u ? 1.f / 64.f : 0.f;
                    const float b4[4] = {v8[j].x * f, v8[j].y * f, v8[j].z * f, v8[j].w * f};
                    mn_split4(b4, bsh + mrow * MN_LD + 4 * gl, bsl + mrow * MN_LD + 4 * gl);
                }
            }
        }
        __syncthreads();
        const int n_k = (min(MN_U, n_u - u0) + 15) / 16;         // (sub-blocks past the end were staged as zeros)
        const __half *ah = ceh + (16 * warp + g) * MN_LD + 2 * c, *al = cel + (16 * warp + g) * MN_LD + 2 * c;
        for (int k = 0; k < n_k; k++) {
            uint32_t fh[4], fl[4];
            fh[0] = *reinterpret_cast<const uint32_t *>(ah + 16 * k);                fl[0] = *reinterpret_cast<const uint32_t *>(al + 16 * k);
            fh[1] = *reinterpret_cast<const uint32_t *>(ah + 16 * k + 8 * MN_LD);    fl[1] = *reinterpret_cast<const uint32_t *>(al + 16 * k + 8 * MN_LD);
            fh[2] = *reinterpret_cast<const uint32_t *>(ah + 16 * k + 8);            fl[2] = *reinterpret_cast<const uint32_t *>(al + 16 * k + 8);
            fh[3] = *reinterpret_cast<const uint32_t *>(ah + 16 * k + 8 * MN_LD + 8); fl[3] = *reinterpret_cast<const uint32_t *>(al + 16 * k + 8 * MN_LD + 8);
#pragma unroll
            for (int t = 0; t < 8; t++) {
                const __half *bh = bsh + (8 * t + g) * MN_LD + 16 * k + 2 * c, *bl = bsl + (8 * t + g) * MN_LD + 16 * k + 2 * c;
                const uint32_t bh0 = *reinterpret_cast<const uint32_t *>(bh), bh1 = *reinterpret_cast<const uint32_t *>(bh + 8);
                const uint32_t bl0 = *reinterpret_cast<const uint32_t *>(bl), bl1 = *reinterpret_cast<const uint32_t *>(bl + 8);
                mn_mma(acc[t], fh, bh0, bh1);
                mn_mma(acc[t], fl, bh0, bh1);
                mn_mma(acc[t], fh, bl0, bl1);
            }
        }
    }
    // undo the two scalings (2^8 * 2^-6) and apply the batch rows' own scales
    const int na = n0 + 16 * warp + g, nb = na + 8;
#pragma unroll
    for (int t = 0; t < 8; t++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int m = 8 * t + 2 * c + e;
            if (m < M) {
                const float sxm = xscale[m] * 0.25f;
                if (na < N) out[(size_t)m * ld_out + na] = acc[t][e] * sxm;
                if (nb < N) out[(size_t)m * ld_out + nb] = acc[t][2 + e] * sxm;
            }
        }
}
template <int ROWS>
static cudaError_t minima_launch(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *slot, int k_groups) {
    const int bytes = 2 * (ROWS + P_MT) * MN_LD * (int)sizeof(__half);
    static VxPerDevice attr;
    cudaError_t e = attr.max_dynamic_smem(c, q4k_minima_kernel<ROWS>, bytes);
    if (e != cudaSuccess) return e;
    return vx_launch_chain(q4k_minima_kernel<ROWS>, dim3(ceil_div(w.n, ROWS)), dim3(2 * ROWS), (size_t)bytes, c->stream, (const uint2 *)w.sc,
                           (const __half2 *)w.aux, (const float *)x.bsum, x.k_pad / 32, (const float *)x.scale, slot, m, w.n, k_groups, w.n);
}

static int g_tcp = 1, g_tcp_stream = 1, g_tcp_q6 = 1;
// 0 = the one-CTA-per-tile kernel; 1 = persistent, aligned split-K only; 2 (default) = persistent, stream mode where it is cheaper
extern "C" int vx_set_persistent_projections(int mode) { g_tcp = mode != 0; g_tcp_stream = mode == 1 ? 0 : mode == 3 ? 2 : 1; g_tcp_q6 = mode != 4; return VX_OK; }   // (3: stream mode wherever it applies, for timing comparisons)

// Eligible: Q4_0, Q4_K or Q6_K, at most 64 batch rows, an even number of 128-weight groups per row (the scale tiles cover two
// groups; a Q6_K row is whole 256-weight super-blocks anyway).
bool vxq_gemm_tcp_eligible(const VxWeight &w, int m) {
    return g_tcp && (w.type == VX_T_Q4_0 || ((w.type == VX_T_Q6_K || w.type == VX_T_Q4_K) && g_tcp_q6)) && m <= P_MT && ((w.k_pad / 128) % 2) == 0;
}

// same contract as vxq_gemm (vx_quant.cu); the context's device error word receives VX_E_TIMEOUT if a bounded wait gave up
int vxq_gemm_tcp(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
                 size_t parts_cap_floats) {
    int *err_flag = c->d_int_result + 8;
    if (x.k_pad != w.k_pad) return vx_fail(c, VX_E_BAD_ARG, "projection: activation row stride %d != weight k_pad %d", x.k_pad, w.k_pad);
    {
        static VxPerDevice attr;
        VX_CUDA(c, attr.max_dynamic_smem(c, gemm_tcp_kernel<false, P_Q4_0>, P_SMEM));
        static VxPerDevice attr_s, attr6, attr6_s;
        VX_CUDA(c, attr_s.max_dynamic_smem(c, gemm_tcp_kernel<true, P_Q4_0>, P_SMEM));
        VX_CUDA(c, attr6.max_dynamic_smem(c, gemm_tcp_kernel<false, P_Q6_K>, P_SMEM_Q6));
        VX_CUDA(c, attr6_s.max_dynamic_smem(c, gemm_tcp_kernel<true, P_Q6_K>, P_SMEM_Q6));
        static VxPerDevice attr4, attr4_s;
        VX_CUDA(c, attr4.max_dynamic_smem(c, gemm_tcp_kernel<false, P_Q4_K>, P_SMEM));
        VX_CUDA(c, attr4_s.max_dynamic_smem(c, gemm_tcp_kernel<true, P_Q4_K>, P_SMEM));
    }
    const int k_groups = w.k_pad / 128;
    const int tiles = ceil_div(w.n, TC_ROWS);
    const int slots = c->sm_count;
    // Split-K in whole pairs of groups.  Cost in pipeline stages: the busiest CTA's stages, a little per unit it walks (the
    // accumulator hand-over), and the partial sums' write and read (mostly L2); the smaller split wins near-ties.
    int split = 1, per = k_groups;
    const int extra = w.type == VX_T_Q4_K ? 1 : 0;          // the minima slot
    if (parts) {
        constexpr double UNIT_STAGES = 2.5, PART_STAGES_PER_FLOAT = 2.2e-6;
        double best = 1e300;
        for (int s = 1; s <= 8 && 2 * s <= k_groups; s++) {
            if ((size_t)(s + extra) * m * w.n > parts_cap_floats) break;
            int p = ceil_div(k_groups, s);
            p += p & 1;
            const int s_eff = ceil_div(k_groups, p);
            const long units = (long)tiles * s_eff;
            const long per_cta = ceil_div64(units, std::min<long>(units, slots));
            const double cost = (double)per_cta * (2.0 * p + UNIT_STAGES) + (s_eff > 1 ? PART_STAGES_PER_FLOAT * s_eff * (double)m * w.n : 0.0);
            if (cost < best * 0.98) { best = cost; split = s_eff; per = p; }
        }
    }
    int n_units = tiles * split, stream_q = 0;
    if (parts && g_tcp_stream) {
        // Stream mode: all tiles' stages as one sequence cut into equal runs (see UnitIter).  Same cost terms, evaluated on the
        // busiest CTA; the slots are as many as the CTAs that can share one tile.
        constexpr double UNIT_STAGES = 2.5, PART_STAGES_PER_FLOAT = 2.2e-6;
        const int qt = k_groups / 2;
        const long Q = (long)tiles * qt;
        const long G = std::min<long>(Q, slots);
        int n_slots = 1;
        double worst = 0.0;
        auto cta_of = [&](long x) { return (int)(((x + 1) * G + Q - 1) / Q - 1); };
        for (int t = 0; t < tiles; t++) n_slots = std::max(n_slots, cta_of((long)(t + 1) * qt - 1) - cta_of((long)t * qt) + 1);
        for (long i = 0; i < G; i++) {
            const long q0 = i * Q / G, q1 = (i + 1) * Q / G;
            const long units = (q1 - 1) / qt - q0 / qt + 1;
            worst = std::max(worst, 4.0 * (double)(q1 - q0) + UNIT_STAGES * (double)units);
        }
        const double cost = worst + (n_slots > 1 ? PART_STAGES_PER_FLOAT * n_slots * (double)m * w.n : 0.0);
        // the aligned split's cost, in the same terms
        const long units_a = (long)tiles * split;
        const double cost_a = (double)ceil_div64(units_a, std::min<long>(units_a, slots)) * (2.0 * per + UNIT_STAGES) +
                              (split > 1 ? PART_STAGES_PER_FLOAT * split * (double)m * w.n : 0.0);
        // (an aligned launch without partial sums also spares its consumer a pass over them: it needs a clearer margin to lose)
        if (n_slots > 1 && (size_t)(n_slots + extra) * m * w.n <= parts_cap_floats && (g_tcp_stream == 2 ? split > 1 : cost < cost_a * (split > 1 ? 0.98 : 0.90))) {
            stream_q = (int)Q; split = n_slots; per = qt; n_units = (int)G;
        }
    }
    const bool to_slots = split > 1 || w.type == VX_T_Q4_K;   // Q4_K always writes slots: its minima come as one more
    float *dst = to_slots ? parts : out;
    const int ld = to_slots ? w.n : ld_out;
    *n_parts_out = split;
    // tensor maps, kept per (weight, activation buffer) combination: a decode step launches the same ones every time
    struct MapKey {
        const void *qs, *sc, *xh, *xl, *hi; int n, kg, kp;
        bool operator<(const MapKey &o) const { return std::tie(qs, sc, xh, xl, hi, n, kg, kp) < std::tie(o.qs, o.sc, o.xh, o.xl, o.hi, o.n, o.kg, o.kp); }
    };
    struct MapSet { CUtensorMap w, s, x, h; };
    static std::map<MapKey, MapSet> cache;
    static std::mutex cache_mu;
    const MapKey key{w.qs, w.sc, x.hi, x.lo, w.type == VX_T_Q6_K ? w.hi : nullptr, w.n, k_groups, x.k_pad};
    MapSet ms;
    bool have = false;
    {
        std::lock_guard<std::mutex> lk(cache_mu);
        auto it = cache.find(key);
        if (it != cache.end()) { ms = it->second; have = true; }
    }
    if (!have) {
        // packed nibbles as bytes [n][k_groups * 64]; block scales as bytes [n][k_groups * 8]
        VX_TRY(make_map(c, &ms.w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.qs, (uint64_t)k_groups * 64, (uint64_t)w.n, (uint64_t)k_groups * 64, 64, TC_ROWS,
                        CU_TENSOR_MAP_SWIZZLE_64B));
        VX_TRY(make_map(c, &ms.s, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.sc, (uint64_t)k_groups * 8, (uint64_t)w.n, (uint64_t)k_groups * 8, 16, TC_ROWS,
                        CU_TENSOR_MAP_SWIZZLE_NONE));
        // activations: plane 0 = x_hi, plane 1 = x_lo, each fp16 [64 rows][k_pad]; one box brings a stage's two tiles
        if ((const char *)x.lo <= (const char *)x.hi) return vx_fail(c, VX_E_BAD_ARG, "projection: the lo half of the activation split must follow the hi half");
        VX_TRY(make_map_3d(c, &ms.x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x.hi, (uint64_t)x.k_pad, (uint64_t)P_MT, 2, (uint64_t)x.k_pad * 2,
                           (uint64_t)((const char *)x.lo - (const char *)x.hi), P_BK, P_MT, 2, CU_TENSOR_MAP_SWIZZLE_128B));
        // Q6_K: the top two bits of every weight as bytes [n][k_groups * 32]; Q4_0 passes the nibble map again (unused)
        if (w.type == VX_T_Q6_K)
            VX_TRY(make_map(c, &ms.h, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w.hi, (uint64_t)k_groups * 32, (uint64_t)w.n, (uint64_t)k_groups * 32, 32,
                            TC_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE));
        else ms.h = ms.w;
        std::lock_guard<std::mutex> lk(cache_mu);
        if (cache.size() > 4096) cache.clear();     // buffers of destroyed models: start over rather than grow without bound
        cache[key] = ms;
    }
    const dim3 grid(std::min(n_units, slots));        // (stream mode: n_units is the number of runs = CTAs)
    cudaError_t le;
#define VX_TCP_LAUNCH(S, F, BYTES)                                                                                              \
    le = vx_launch_dependent(gemm_tcp_kernel<S, F>, grid, dim3(P_THREADS), (size_t)(BYTES), c->stream, ms.w, ms.s, ms.x, ms.h,  \
                             (const __half *)w.aux, (const float *)x.scale, dst, m, w.n, k_groups, per, split, n_units, stream_q, ld, \
                             (size_t)m * w.n, err_flag)
    if (w.type == VX_T_Q6_K) { if (stream_q > 0) VX_TCP_LAUNCH(true, P_Q6_K, P_SMEM_Q6); else VX_TCP_LAUNCH(false, P_Q6_K, P_SMEM_Q6); }
    else if (w.type == VX_T_Q4_K) { if (stream_q > 0) VX_TCP_LAUNCH(true, P_Q4_K, P_SMEM); else VX_TCP_LAUNCH(false, P_Q4_K, P_SMEM); }
    else { if (stream_q > 0) VX_TCP_LAUNCH(true, P_Q4_0, P_SMEM); else VX_TCP_LAUNCH(false, P_Q4_0, P_SMEM); }
#undef VX_TCP_LAUNCH
    if (le != cudaSuccess) return vx_cuda_fail(c, le, "projection launch");
    VX_LAUNCH_CHECK(c);
    if (w.type == VX_T_Q4_K) {     // the minima as one more slot behind the projection's own
        // 128-row CTAs when they fill the GPU, 64-row CTAs for the narrow matrices
        float *slot = parts + (size_t)split * m * w.n;
        le = w.n >= 128 * c->sm_count ? minima_launch<128>(c, w, x, m, slot, k_groups) : minima_launch<64>(c, w, x, m, slot, k_groups);
        if (le != cudaSuccess) return vx_cuda_fail(c, le, "minima launch");
        VX_LAUNCH_CHECK(c);
        *n_parts_out = split + 1;
    }
    return VX_OK;
}
