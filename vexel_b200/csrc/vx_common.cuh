// Shared declarations of the CUDA backend: context, status handling, small device helpers.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "vexel_cuda.h"

struct vx_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    std::recursive_mutex mu;
    std::string err;
    // Alloc/ResetPool semantics of the reference's pooled backend (backend/metal/backend.go:490-566):
    // pooled buffers are handed out again after ResetPool, permanent ones never are.
    struct Buf { void *p; size_t bytes; bool in_use; };
    std::vector<Buf> pooled;
    std::unordered_map<void *, size_t> permanent;
    // scratch owned by the interface-level entry points
    void *scratch = nullptr; size_t scratch_bytes = 0;
    int *d_int_result = nullptr;      // device ints: [0] synchronous Argmax result, [8] sticky kernel error word
    int *h_int_result = nullptr;      // pinned
    int sm_count = 148;
    uint64_t launches = 0;
    void *tp = nullptr;               // tensor-parallel communicator of this context (vx_tp.cu), null for single-GPU use
    // Repacked copies of quantised weights that the interface-level MatMulQ* calls were given, keyed by the raw tensor's
    // address.  Only tensors inside a permanent allocation are kept (the reference uploads weights once into
    // AllocPermanent buffers, runtime/loader.go:507-708); an entry is dropped when the API writes into its raw bytes
    // (ToDevice, CopyBuffer, memset) or frees them.
    struct Repacked { int type, n, k; size_t raw_bytes; void *buf; };
    std::unordered_map<const void *, Repacked> repacked;
    bool repack_cache = true;
};
void vx_repack_invalidate(vx_ctx *c, const void *dst, size_t bytes);   // drops cached repacks whose raw bytes overlap [dst, dst + bytes)

struct VxGuard {
    vx_ctx *c;
    explicit VxGuard(vx_ctx *ctx) : c(ctx) { c->mu.lock(); cudaSetDevice(c->device); }
    ~VxGuard() { c->mu.unlock(); }
};

int vx_fail(vx_ctx *c, int code, const char *fmt, ...);
int vx_cuda_fail(vx_ctx *c, cudaError_t e, const char *what);
int vx_scratch(vx_ctx *c, size_t bytes, void **out);   // grows the interface-level scratch buffer

#define VX_CUDA(ctx, call)                                                        \
    do {                                                                          \
        cudaError_t e__ = (call);                                                 \
        if (e__ != cudaSuccess) return vx_cuda_fail((ctx), e__, #call);           \
    } while (0)
#define VX_LAUNCH_CHECK(ctx)                                                      \
    do {                                                                          \
        (ctx)->launches++;                                                        \
        cudaError_t e__ = cudaGetLastError();                                     \
        if (e__ != cudaSuccess) return vx_cuda_fail((ctx), e__, "kernel launch"); \
    } while (0)
#define VX_REQUIRE(ctx, cond, msg)                                                \
    do {                                                                          \
        if (!(cond)) return vx_fail((ctx), VX_E_BAD_ARG, "%s: %s", __func__, msg); \
    } while (0)
#define VX_TRY(expr)                                                              \
    do {                                                                          \
        int rc__ = (expr);                                                        \
        if (rc__ != VX_OK) return rc__;                                           \
    } while (0)

// cudaFuncSetAttribute changes the calling device's copy of a kernel only, and one process may drive a context per GPU:
// a call site keeps one of these (static) and asks it once per device, with that device current.
struct VxPerDevice {
    std::atomic<unsigned long long> mask{0};
    template <typename K> cudaError_t max_dynamic_smem(const vx_ctx *c, K kernel, int bytes) {
        const bool tracked = c->device >= 0 && c->device < 64;
        if (tracked && ((mask.load(std::memory_order_acquire) >> c->device) & 1ull)) return cudaSuccess;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e == cudaSuccess && tracked) mask.fetch_or(1ull << c->device, std::memory_order_release);
        return e;
    }
    // runs set() (any per-device kernel attribute calls) the first time this device comes by
    template <typename F> cudaError_t once(const vx_ctx *c, F set) {
        const bool tracked = c->device >= 0 && c->device < 64;
        if (tracked && ((mask.load(std::memory_order_acquire) >> c->device) & 1ull)) return cudaSuccess;
        cudaError_t e = set();
        if (e == cudaSuccess && tracked) mask.fetch_or(1ull << c->device, std::memory_order_release);
        return e;
    }
};

template <typename T> static inline T *dp(vx_dptr p) { return reinterpret_cast<T *>(static_cast<uintptr_t>(p)); }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device helpers -------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// block-wide reductions; `red` is >= 32 floats of shared memory; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float *red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float *red) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = lane < nw ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

// ---- programmatic dependent launch ------------------------------------------------------------
// A kernel launched through vx_launch_dependent may start while its predecessor in the stream is still running: its CTAs
// become resident as soon as every CTA of the predecessor has executed vx_pdl_trigger() (or exited).  Everything such a kernel
// does before vx_pdl_wait() must be independent of the predecessor (barrier set-up, weight prefetch); vx_pdl_wait() returns
// once the predecessor has completed and its writes are visible.  Both instructions are no-ops in a normal launch.
__device__ __forceinline__ void vx_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void vx_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
extern int g_vx_pdl;     // 0 = plain stream order for every launch
template <typename... KArgs, typename... Args>
static inline cudaError_t vx_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = g_vx_pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
// The other kernels of a layer (norms, RoPE + append, attention, merge, activation) chained the same way when the switch is
// at 2: each of them starts with vx_pdl_wait() followed by vx_pdl_trigger(), so its successor's launch is processed while it
// runs, but becomes resident only once its own predecessor has completed.  At 0 or 1 this is a plain launch.
template <typename... KArgs, typename... Args>
static inline cudaError_t vx_launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = g_vx_pdl >= 2 ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- shared between translation units ---------------------------------------------------------
// Activation rows prepared for the tensor-core projections: x = s * (hi + lo) with hi, lo fp16 and
// s a power of two per row; element k is stored at position perm4(k) so that one 8-byte load gives
// a thread its two B-fragment registers (see vx_quant.cu).
struct VxSplit {
    __half *hi; __half *lo; float *scale; float *bsum;   // bsum: per-32-block sums of x/s (K-quant minima)
    int k_pad;                                           // row stride in elements (multiple of 128)
};
__host__ __device__ __forceinline__ int vx_perm4(int k) {   // within each group of 4: order 0,2,1,3
    int r = k & 3;
    return (k & ~3) | ((r == 1) ? 2 : (r == 2) ? 1 : r);
}

// power-of-two row scale: max|x| = f * 2^e with f in [0.5, 1)  ->  s = 2^(e-11), so max|x/s| lies in [1024, 2048)
__device__ __forceinline__ void vx_row_scale(float amax, float &sc, float &inv) {
    sc = 1.0f; inv = 1.0f;
    if (amax > 0.f && amax < INFINITY) {
        int e; frexpf(amax, &e);
        e = max(-100, min(100, e - 11));
        sc = ldexpf(1.0f, e); inv = ldexpf(1.0f, -e);
    }
}
// splits four consecutive, already scaled activations starting at column k0 (a multiple of 4) into fp16 hi/lo, stores them
// in the 0,2,1,3 order and accumulates the 32-column block sum.  Must be reached by all 8 lanes that share a 32-block.
__device__ __forceinline__ void vx_split_store4(const float (&v)[4], __half *hi, __half *lo, float *bs, int k0) {
    __half h[4], l[4];
    float sum = (v[0] + v[1]) + (v[2] + v[3]);
#pragma unroll
    for (int i = 0; i < 4; i++) { h[i] = __float2half_rn(v[i]); l[i] = __float2half_rn(v[i] - __half2float(h[i])); }
    *reinterpret_cast<uint2 *>(hi + k0) = make_uint2((uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[2]) << 16),
                                                     (uint32_t)__half_as_ushort(h[1]) | ((uint32_t)__half_as_ushort(h[3]) << 16));
    *reinterpret_cast<uint2 *>(lo + k0) = make_uint2((uint32_t)__half_as_ushort(l[0]) | ((uint32_t)__half_as_ushort(l[2]) << 16),
                                                     (uint32_t)__half_as_ushort(l[1]) | ((uint32_t)__half_as_ushort(l[3]) << 16));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if ((threadIdx.x & 7) == 0) bs[k0 >> 5] = sum;
}
constexpr int VX_ROW_THREADS = 1024;   // row kernels: one CTA per row, thread t owns columns (c*1024 + t)*4 .. +3 of chunk c

// Repacked weight matrix for the MMA kernels (built by vx_model_finalize / the interface entry points).
struct VxWeight {
    int type = -1;          // VX_T_*
    int n = 0, k = 0, k_pad = 0;
    void *qs = nullptr;     // Q4_0: [n][k_pad/128][4 lanes][4 words]; F32: raw
    void *sc = nullptr;     // Q4_0: half [n][k_pad/32]
    void *aux = nullptr;    // K-quants: super-block scales (half2 {d, dmin} or half d) [n][k/256]
    void *hi = nullptr;     // Q6_K: top two bits [n][k_pad/128][4 lanes] uint2
    size_t bytes = 0;       // GGUF byte size (roofline accounting)
};
struct VxRepackLayout { size_t off[4]; size_t row_bytes[4]; size_t total; };   // arrays: qs, sc, aux, hi

// launchers implemented in vx_quant.cu
bool vxq_layout(int type, int n, int k, VxRepackLayout *L);
int vxq_repack_rows(vx_ctx *c, int type, const void *raw_dev, int n_rows, int k, void *base, const VxRepackLayout &L, int row0);
void vxq_weight_view(int type, int n, int k, void *base, const VxRepackLayout &L, VxWeight *w);
int vxq_gemm(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out,
             float *parts, size_t parts_cap_floats);
int vxq_gemm_tc(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
                size_t parts_cap_floats);
bool vxq_gemm_tcp_eligible(const VxWeight &w, int m);      // vx_gemm_tcp.cu: the persistent tcgen05 kernel covers this projection
int vxq_gemm_tcp(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
                 size_t parts_cap_floats);
// thin batches (1-8 rows) of Q4_0 weights: mma.sync kernel that streams the weights through registers (vx_gemv.cu)
bool vxq_gemv_eligible(const VxWeight &w, int m);
int vxq_gemv(vx_ctx *c, const VxWeight &w, const VxSplit &x, int m, float *out, int ld_out, int *n_parts_out, float *parts,
             size_t parts_cap_floats);
// tensor parallelism (vx_tp.cu)
int vxtp_world(vx_ctx *c);
int vxtp_rank(vx_ctx *c);
int vxtp_allreduce_sum(vx_ctx *c, float *buf, size_t n);
int vxtp_global_argmax(vx_ctx *c, const float *logits, long ld, const int32_t *local_idx, int rows, int local_vocab, void *scratch, int32_t *out_tok);
struct vx_model;
extern "C" vx_ctx *vx_model_ctx(vx_model *m);     // the context a model lives in (internal)
int vx_check_device_error(vx_ctx *c);   // after a stream synchronisation: reports and clears the sticky kernel error word
int vxq_split_rows(vx_ctx *c, const float *x, int rows, int cols, int ld, const VxSplit &s);
int vxq_reduce_parts(vx_ctx *c, const float *parts, int n_parts, int m, int n, float *out, int ld_out);
size_t vxq_split_bytes(int rows, int k, size_t *hi_off, size_t *lo_off, size_t *scale_off, size_t *bsum_off, int *k_pad);

// launchers implemented in vx_paged.cu
struct VxAttnArgs {
    const float *q; int q_row_stride;        // [rows][Hq*D] float32
    const void *pool; int pool_is_f16;
    const int32_t *const *tables;             // per sequence-slot block table base pointers (device array)
    const int32_t *row_slot;                  // [rows] -> index into tables
    const int32_t *row_kv_start;              // [rows] first attended position (nullptr = 0)
    const int32_t *row_kv_len;                // [rows]
    const int4 *work; const int32_t *n_work_dev; int n_work;   // (row, first_page, n_pages, chunk_index)
    const int32_t *row_work_start;            // [rows+1]
    float *partials;                          // [n_work][Hq][D+2]
    float *out; int out_row_stride;           // [rows][Hq*D]
    int rows, n_q_heads, n_kv_heads, head_dim, block_size;
    float scale, softcap;
    // optional, zeroed by the caller before the launch: the work-list kernels raise row_bound[row] (float bits, atomicMax) to
    // the largest |O| / L of any chunk and head of the row -- an upper bound of the row's largest output magnitude, since
    // the merged output is a convex combination of the chunks' normalised outputs.  With it the merge + split kernel knows
    // the row scale without a row-wide reduction and can spread a row over several CTAs.
    unsigned int *row_bound;
};
int vxp_attention(vx_ctx *c, const VxAttnArgs &a);
int vxp_prefill_f32(vx_ctx *c, const float *q, int q_ld, const float *k, const float *v, long kv_ld, float *out, int out_ld, int n_rows,
                    int hq, int hkv, int d, float scale, float softcap);
int vxp_prefill_rows(vx_ctx *c, const VxAttnArgs &a, int row0, int n_rows);   // VX_E_UNSUPPORTED when the shape has no such kernel
int vxp_attention_split(vx_ctx *c, const VxAttnArgs &a, const VxSplit *split, int n_max_chunks, bool *fused);
