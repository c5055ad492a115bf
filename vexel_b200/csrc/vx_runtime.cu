// Context lifecycle and memory entry points of the C ABI (include/vexel_cuda.h).
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "vx_common.cuh"

int vx_fail(vx_ctx *c, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (c) c->err = buf;
    return code;
}

int vx_cuda_fail(vx_ctx *c, cudaError_t e, const char *what) {
    return vx_fail(c, VX_E_CUDA, "CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
}

int vx_scratch(vx_ctx *c, size_t bytes, void **out) {
    if (bytes > c->scratch_bytes) {
        if (c->scratch) { cudaStreamSynchronize(c->stream); cudaFree(c->scratch); c->scratch = nullptr; c->scratch_bytes = 0; }
        size_t want = bytes + bytes / 4;
        cudaError_t e = cudaMalloc(&c->scratch, want);
        if (e != cudaSuccess) return vx_fail(c, VX_E_OOM, "scratch allocation of %zu bytes failed: %s", want, cudaGetErrorString(e));
        c->scratch_bytes = want;
    }
    *out = c->scratch;
    return VX_OK;
}

int vx_check_device_error(vx_ctx *c) {
    VX_CUDA(c, cudaMemcpyAsync(c->h_int_result + 8, c->d_int_result + 8, 4, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    int e = c->h_int_result[8];
    if (e != 0) {
        cudaMemsetAsync(c->d_int_result + 8, 0, 4, c->stream);
        return vx_fail(c, e, "a kernel reported status %d (%s)", e, e == VX_E_TIMEOUT ? "a bounded device-side wait gave up" : "device error");
    }
    return VX_OK;
}

void vx_repack_invalidate(vx_ctx *c, const void *dst, size_t bytes) {
    if (c->repacked.empty()) return;
    const char *lo = (const char *)dst, *hi = lo + bytes;
    for (auto it = c->repacked.begin(); it != c->repacked.end();) {
        const char *r0 = (const char *)it->first, *r1 = r0 + it->second.raw_bytes;
        if (r0 < hi && lo < r1) {
            cudaStreamSynchronize(c->stream);
            cudaFree(it->second.buf);
            it = c->repacked.erase(it);
        } else ++it;
    }
}

extern "C" {

int vx_init(int device, vx_ctx **out) {
    if (!out) return VX_E_BAD_ARG;
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n <= 0 || device < 0 || device >= n) return VX_E_CUDA;   // no CPU fallback
    if (cudaSetDevice(device) != cudaSuccess) return VX_E_CUDA;
    vx_ctx *c = new vx_ctx();
    c->device = device;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) { delete c; return VX_E_CUDA; }
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    if (cudaMalloc(&c->d_int_result, 64) != cudaSuccess || cudaMallocHost(&c->h_int_result, 64) != cudaSuccess ||
        cudaMemset(c->d_int_result, 0, 64) != cudaSuccess) {
        cudaStreamDestroy(c->stream); delete c; return VX_E_CUDA;
    }
    *out = c;
    return VX_OK;
}

int vx_destroy(vx_ctx *c) {
    if (!c) return VX_E_BAD_ARG;
    if (c->tp) vx_tp_shutdown(c);      // the NCCL communicator goes before the stream it runs on
    {
        VxGuard g(c);
        cudaStreamSynchronize(c->stream);
        for (auto &r : c->repacked) cudaFree(r.second.buf);
        for (auto &b : c->pooled) cudaFree(b.p);
        for (auto &kv : c->permanent) cudaFree(kv.first);
        if (c->scratch) cudaFree(c->scratch);
        cudaFree(c->d_int_result);
        cudaFreeHost(c->h_int_result);
        cudaStreamDestroy(c->stream);
    }
    delete c;
    return VX_OK;
}

const char *vx_last_error(vx_ctx *c) { return c ? c->err.c_str() : "null context"; }
int vx_device_index(vx_ctx *c) { return c ? c->device : -1; }

int vx_alloc(vx_ctx *c, size_t bytes, vx_dptr *out) {
    if (!c || !out) return VX_E_BAD_ARG;
    VxGuard g(c);
    *out = 0;
    if (bytes == 0) return VX_OK;   // Alloc(<=0) yields a nil DevicePtr (backend/cpu/cpu.go:42-45)
    // best-fit reuse of a free pooled buffer (at most 2x the request), as the pooled reference backend does
    int best = -1;
    for (size_t i = 0; i < c->pooled.size(); i++) {
        auto &b = c->pooled[i];
        if (!b.in_use && b.bytes >= bytes && b.bytes <= 2 * bytes && (best < 0 || b.bytes < c->pooled[best].bytes)) best = (int)i;
    }
    if (best >= 0) { c->pooled[best].in_use = true; *out = (vx_dptr)(uintptr_t)c->pooled[best].p; return VX_OK; }
    void *p = nullptr;
    size_t rounded = (bytes + 255) & ~(size_t)255;
    cudaError_t e = cudaMalloc(&p, rounded);
    if (e != cudaSuccess) { cudaGetLastError(); return vx_fail(c, VX_E_OOM, "cudaMalloc(%zu) failed: %s", rounded, cudaGetErrorString(e)); }
    c->pooled.push_back({p, rounded, true});
    *out = (vx_dptr)(uintptr_t)p;
    return VX_OK;
}

int vx_alloc_permanent(vx_ctx *c, size_t bytes, vx_dptr *out) {
    if (!c || !out) return VX_E_BAD_ARG;
    VxGuard g(c);
    *out = 0;
    if (bytes == 0) return VX_OK;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) { cudaGetLastError(); return vx_fail(c, VX_E_OOM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e)); }
    c->permanent[p] = bytes;
    *out = (vx_dptr)(uintptr_t)p;
    return VX_OK;
}

int vx_free(vx_ctx *c, vx_dptr p) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (p == 0) return VX_OK;
    void *vp = dp<void>(p);
    auto it = c->permanent.find(vp);
    if (it != c->permanent.end()) {
        VX_CUDA(c, cudaStreamSynchronize(c->stream));
        vx_repack_invalidate(c, vp, it->second);
        cudaFree(vp);
        c->permanent.erase(it);
        return VX_OK;
    }
    for (auto &b : c->pooled)
        if (b.p == vp) { b.in_use = false; return VX_OK; }   // returns to the pool, memory kept
    return vx_fail(c, VX_E_BAD_ARG, "vx_free: %p was not allocated by this context", vp);
}

int vx_reset_pool(vx_ctx *c) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    for (auto &b : c->pooled) b.in_use = false;
    return VX_OK;
}

int vx_h2d(vx_ctx *c, vx_dptr dst, const void *src, size_t bytes) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (bytes == 0 || dst == 0 || !src) return VX_OK;   // ToDevice ignores nil/empty (backend/cpu/cpu.go:57-63)
    vx_repack_invalidate(c, dp<void>(dst), bytes);
    VX_CUDA(c, cudaMemcpyAsync(dp<void>(dst), src, bytes, cudaMemcpyHostToDevice, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));   // the Go slice may be reused as soon as the call returns
    return VX_OK;
}

int vx_d2h(vx_ctx *c, void *dst, vx_dptr src, size_t bytes) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (bytes == 0 || src == 0 || !dst) return VX_OK;
    VX_CUDA(c, cudaMemcpyAsync(dst, dp<void>(src), bytes, cudaMemcpyDeviceToHost, c->stream));
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    return VX_OK;
}

int vx_d2d(vx_ctx *c, vx_dptr dst, vx_dptr src, size_t bytes) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (bytes == 0) return VX_OK;
    VX_REQUIRE(c, dst != 0 && src != 0, "nil device pointer");
    vx_repack_invalidate(c, dp<void>(dst), bytes);
    VX_CUDA(c, cudaMemcpyAsync(dp<void>(dst), dp<void>(src), bytes, cudaMemcpyDeviceToDevice, c->stream));
    return VX_OK;
}

int vx_memset(vx_ctx *c, vx_dptr dst, int byte, size_t bytes) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    if (bytes == 0) return VX_OK;
    VX_REQUIRE(c, dst != 0, "nil device pointer");
    vx_repack_invalidate(c, dp<void>(dst), bytes);
    VX_CUDA(c, cudaMemsetAsync(dp<void>(dst), byte, bytes, c->stream));
    return VX_OK;
}

int vx_sync(vx_ctx *c) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_CUDA(c, cudaStreamSynchronize(c->stream));
    return vx_check_device_error(c);
}

}  // extern "C"
