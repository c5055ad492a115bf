// Pieces shared by the tcgen05 projection kernels: bounded mbarrier waits, TMA loads into the own CTA, tensor-core
// descriptors and instructions, tensor-memory stores / loads, nibble expansion, and tensor-map encoding on the host.
#pragma once
#include <cuda.h>

#include "vx_common.cuh"

namespace vxtc {

constexpr int TC_ROWS = 128;          // weight rows per CTA tile (MMA M)

constexpr long long WAIT_CLOCKS = 400000000LL;             // ~0.2 s at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// waits in hardware for the phase to complete or for a short time limit, whichever comes first; a thread parked here
// takes no issue slots from the warps that share its scheduler (a test_wait spin loop does)
__device__ __forceinline__ bool mbar_try_park(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// bounded wait: false on timeout or when another thread of the CTA has already given up
__device__ __forceinline__ bool mbar_wait_limit(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit_clocks) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        if (mbar_try_park(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_clocks) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    return mbar_wait_limit(bar, parity, abort_flag, WAIT_CLOCKS);
}

// 2-D tiled TMA load into this CTA, completing on one of its mbarriers
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}

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
// instruction descriptors: D=f32, A=B=f16, both K-major, M=128, N = 128 (x_hi and x_lo stacked) or 64 (x_hi only)
constexpr uint32_t umma_idesc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24); }

// D[tmem_d] (+)= A[tmem_a] * B[smem desc]^T, the A operand read from tensor memory (8 columns of fp16 pairs per K=16)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// both operands from shared memory
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
                   "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&a)[16], const uint32_t (&b)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]), "r"(a[8]), "r"(a[9]),
                   "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(b[4]),
                   "r"(b[5]), "r"(b[6]), "r"(b[7]), "r"(b[8]), "r"(b[9]), "r"(b[10]), "r"(b[11]), "r"(b[12]), "r"(b[13]), "r"(b[14]), "r"(b[15])
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
#define VX_TMEM_LD16(v, taddr)                                                                                                    \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"      \
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),    \
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])                       \
                 : "r"(taddr))

// one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}
// (v & 0x000F000F) holds two nibbles -> half2 {q0-8, q1-8}
__device__ __forceinline__ __half2 nib2(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;
    return __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1032.f, 1032.f));
}
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
// unsigned variant -> half2 {q0, q1}
__device__ __forceinline__ __half2 nibu2(uint32_t v) {
    uint32_t h = (v & 0x000F000Fu) | 0x64006400u;
    return __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1024.f, 1024.f));
}
// low nibbles in v (bits 0-3, 16-19), the two top bits already placed at bits 4-5 and 20-21 -> half2 {q0 - 32, q1 - 32}
__device__ __forceinline__ __half2 q6h2(uint32_t v, uint32_t h6) {
    uint32_t h = (v & 0x000F000Fu) | h6 | 0x64006400u;
    return __hsub2(*reinterpret_cast<__half2 *>(&h), __floats2half2_rn(1056.f, 1056.f));
}
// a float32 scale as an fp16 pair (hi + lo carries 22 bits of it)
__device__ __forceinline__ void split_scale(float d, __half2 *hi, __half2 *lo) {
    const __half h = __float2half_rn(d);
    *hi = __half2half2(h); *lo = __half2half2(__float2half_rn(d - __half2float(h)));
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
// row-major 2-D tensor [rows][row_bytes] of `elem`-byte elements, box = box_cols x box_rows
inline int make_map(vx_ctx *c, CUtensorMap *map, CUtensorMapDataType dt, int elem, const void *base, uint64_t cols, uint64_t rows,
             uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return vx_fail(c, VX_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)base & 15) != 0 || (row_stride_bytes & 15) != 0) return vx_fail(c, VX_E_BAD_ARG, "tensor map: base and row stride must be 16-byte aligned");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    (void)elem;
    if (r != CUDA_SUCCESS) return vx_fail(c, VX_E_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return VX_OK;
}

// 3-D tensor [planes][rows][cols] of 2-byte elements (row and plane strides in bytes), box = box_cols x box_rows x box_planes
inline int make_map_3d(vx_ctx *c, CUtensorMap *map, CUtensorMapDataType dt, const void *base, uint64_t cols, uint64_t rows, uint64_t planes,
                       uint64_t row_stride_bytes, uint64_t plane_stride_bytes, uint32_t box_cols, uint32_t box_rows, uint32_t box_planes,
                       CUtensorMapSwizzle sw) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return vx_fail(c, VX_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if (((uintptr_t)base & 15) != 0 || (row_stride_bytes & 15) != 0 || (plane_stride_bytes & 15) != 0)
        return vx_fail(c, VX_E_BAD_ARG, "tensor map: base and strides must be 16-byte aligned");
    cuuint64_t dims[3] = {cols, rows, planes};
    cuuint64_t strides[2] = {row_stride_bytes, plane_stride_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, box_planes};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vx_fail(c, VX_E_CUDA, "cuTensorMapEncodeTiled (3-D) failed with %d", (int)r);
    return VX_OK;
}

}  // namespace vxtc
