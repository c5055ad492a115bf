// Device-side helpers shared by the paged-attention launchers and the per-step packing kernel.
#pragma once
#include "vx_common.cuh"

// exclusive block-wide scan of one int per thread (blockDim.x <= 1024, multiple of 32).
// `tmp` is 33 ints of shared memory.  Returns the exclusive prefix; *total gets the block sum.
__device__ __forceinline__ int vx_block_excl_scan(int v, int *tmp, int *total) {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += t; }
    __syncthreads();
    if (lane == 31) tmp[w] = inc;
    __syncthreads();
    if (w == 0) {
        int x = lane < nw ? tmp[lane] : 0, xi = x;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, xi, o); if (lane >= o) xi += t; }
        tmp[lane] = xi - x;
        if (lane == 31) tmp[32] = xi;
    }
    __syncthreads();
    *total = tmp[32];
    return tmp[w] + inc - v;
}

// Split-K work list for paged attention.  Row r attends positions [kv_start[r], kv_len[r]); its pages
// first_page..last_page are cut into chunks of chunk_pages.  work[i] = (row, first page, page count,
// chunk index within the row); row_work_start[r] = index of the row's first chunk.  Must be called by
// every thread of the block.  Returns the number of work items (clamped to max_work, *overflow set).
// row_route (optional): rows with a non-zero entry are served by another attention kernel and get no work items.
__device__ __forceinline__ int vx_build_work(int rows, const int32_t *kv_start, const int32_t *kv_len, const int32_t *row_route, int block_size,
                                             int chunk_pages, int4 *work, int32_t *row_work_start, int max_work,
                                             int *overflow, int *scan_tmp) {
    int base = 0;
    for (int r0 = 0; r0 < rows; r0 += blockDim.x) {
        int r = r0 + threadIdx.x;
        int fp = 0, np = 0, nc = 0;
        if (r < rows) {
            int ks = kv_start ? kv_start[r] : 0, kl = kv_len[r];
            if (kl > ks && !(row_route && row_route[r] != 0)) {
                fp = ks / block_size;
                np = (kl - 1) / block_size - fp + 1;
                nc = (np + chunk_pages - 1) / chunk_pages;
            }
        }
        int total;
        int off = base + vx_block_excl_scan(nc, scan_tmp, &total);
        if (r < rows) {
            row_work_start[r] = min(off, max_work);
            for (int ci = 0; ci < nc; ci++) {
                int idx = off + ci;
                if (idx < max_work) work[idx] = make_int4(r, fp + ci * chunk_pages, min(chunk_pages, np - ci * chunk_pages), ci);
                else *overflow = 1;
            }
        }
        base += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) row_work_start[rows] = min(base, max_work);
    return min(base, max_work);
}
