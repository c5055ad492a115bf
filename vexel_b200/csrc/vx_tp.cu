// Tensor parallelism for models that do not fit (or should not sit on) one GPU: one process per GPU, every rank holds a
// slice of each projection matrix and of the KV pool, and the partial results of the two row-split projections of a
// layer (attention output, FFN down) are summed over the ranks with an NCCL all-reduce on the compute stream.
//
// The reference keeps whole Wq..W2 per block on its one device (inference/runtime/block.go:256-266); this is the
// Megatron-style split of that block: Wq/Wk/Wv and W1/W3 by output rows (heads, FFN columns -- no communication), Wo and W2
// by input columns (their outputs are partial sums over the ranks), the output head by vocabulary rows (each rank finds its
// local maximum, one small all-gather of (value, index) pairs picks the global first maximum).  Activations, norms, the
// embedding table, block tables and the packing kernel are replicated: every rank runs the same step on the same token ids.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2) so that the library has no link-time dependency on it; a process
// that never calls vx_tp_init never touches it.  NCCL's own collectives only: no peer-memory kernels here.
#include <dlfcn.h>
#include <nccl.h>

#include "vx_common.cuh"

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};
NcclApi *nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!api.handle) return;
#define VX_SYM(field, name) api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name))
        VX_SYM(GetUniqueId, "ncclGetUniqueId"); VX_SYM(CommInitRank, "ncclCommInitRank"); VX_SYM(CommDestroy, "ncclCommDestroy");
        VX_SYM(AllReduce, "ncclAllReduce"); VX_SYM(AllGather, "ncclAllGather"); VX_SYM(GetErrorString, "ncclGetErrorString");
#undef VX_SYM
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString;
    });
    return &api;
}

struct VxTp { ncclComm_t comm = nullptr; int rank = 0, world = 1; };
VxTp *tp_of(vx_ctx *c) { return static_cast<VxTp *>(c->tp); }

int nccl_fail(vx_ctx *c, ncclResult_t r, const char *what) {
    return vx_fail(c, VX_E_CUDA, "NCCL error %d (%s) at %s", (int)r, nccl_api()->GetErrorString ? nccl_api()->GetErrorString(r) : "?", what);
}

// per logits row: this rank's best (value, global index)
__global__ void tp_pack_best_kernel(const float *__restrict__ logits, long ld, const int32_t *__restrict__ local_idx, int rows, int idx_offset,
                                    float2 *__restrict__ out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const int i = local_idx[r];
    out[r] = make_float2(logits[(size_t)r * ld + i], __int_as_float(i + idx_offset));
}
// first maximum over the ranks' candidates (ranks hold ascending vocabulary ranges, so the lower rank wins a tie: sampler.go:79-90)
__global__ void tp_pick_best_kernel(const float2 *__restrict__ all, int rows, int world, int32_t *__restrict__ out_tok) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    float best = all[r].x; int idx = __float_as_int(all[r].y);
    for (int w = 1; w < world; w++) {
        const float2 v = all[(size_t)w * rows + r];
        if (v.x > best) { best = v.x; idx = __float_as_int(v.y); }
    }
    out_tok[r] = idx;
}

}  // namespace

int vxtp_world(vx_ctx *c) { return c->tp ? tp_of(c)->world : 1; }
int vxtp_rank(vx_ctx *c) { return c->tp ? tp_of(c)->rank : 0; }

// in-place sum over the ranks of n floats, on the context's stream
int vxtp_allreduce_sum(vx_ctx *c, float *buf, size_t n) {
    VxTp *t = tp_of(c);
    if (!t) return vx_fail(c, VX_E_BAD_ARG, "tensor parallelism was not initialised on this context");
    ncclResult_t r = nccl_api()->AllReduce(buf, buf, n, ncclFloat32, ncclSum, t->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(c, r, "ncclAllReduce");
    return VX_OK;
}

// global greedy tokens from the ranks' local argmax: scratch holds (1 + world) * rows float2
int vxtp_global_argmax(vx_ctx *c, const float *logits, long ld, const int32_t *local_idx, int rows, int local_vocab, void *scratch, int32_t *out_tok) {
    VxTp *t = tp_of(c);
    if (!t) return vx_fail(c, VX_E_BAD_ARG, "tensor parallelism was not initialised on this context");
    float2 *mine = static_cast<float2 *>(scratch), *all = mine + rows;
    tp_pack_best_kernel<<<ceil_div(rows, 128), 128, 0, c->stream>>>(logits, ld, local_idx, rows, t->rank * local_vocab, mine);
    VX_LAUNCH_CHECK(c);
    ncclResult_t r = nccl_api()->AllGather(mine, all, (size_t)rows * 2, ncclFloat32, t->comm, c->stream);
    if (r != ncclSuccess) return nccl_fail(c, r, "ncclAllGather");
    tp_pick_best_kernel<<<ceil_div(rows, 128), 128, 0, c->stream>>>(all, rows, t->world, out_tok);
    VX_LAUNCH_CHECK(c);
    return VX_OK;
}

extern "C" {

// ncclGetUniqueId: rank 0 makes the 128-byte id and hands it to the other ranks by whatever channel the host has
int vx_tp_unique_id(void *out, int cap) {
    if (!out || cap < NCCL_UNIQUE_ID_BYTES) return VX_E_BAD_ARG;
    NcclApi *api = nccl_api();
    if (!api->ok) return VX_E_UNSUPPORTED;
    ncclUniqueId id;
    if (api->GetUniqueId(&id) != ncclSuccess) return VX_E_CUDA;
    memcpy(out, &id, NCCL_UNIQUE_ID_BYTES);
    return VX_OK;
}

int vx_tp_init(vx_ctx *c, const void *unique_id, int rank, int world) {
    if (!c || !unique_id) return VX_E_BAD_ARG;
    VxGuard g(c);
    VX_REQUIRE(c, world >= 1 && rank >= 0 && rank < world, "rank outside [0, world)");
    VX_REQUIRE(c, c->tp == nullptr, "tensor parallelism is already initialised on this context");
    NcclApi *api = nccl_api();
    if (!api->ok) return vx_fail(c, VX_E_UNSUPPORTED, "libnccl.so.2 could not be loaded (or lacks a needed symbol)");
    ncclUniqueId id;
    memcpy(&id, unique_id, NCCL_UNIQUE_ID_BYTES);
    VxTp *t = new VxTp();
    t->rank = rank; t->world = world;
    ncclResult_t r = api->CommInitRank(&t->comm, world, id, rank);
    if (r != ncclSuccess) { delete t; return nccl_fail(c, r, "ncclCommInitRank"); }
    c->tp = t;
    return VX_OK;
}

int vx_tp_shutdown(vx_ctx *c) {
    if (!c) return VX_E_BAD_ARG;
    VxGuard g(c);
    VxTp *t = tp_of(c);
    if (!t) return VX_OK;
    cudaStreamSynchronize(c->stream);
    nccl_api()->CommDestroy(t->comm);
    delete t;
    c->tp = nullptr;
    return VX_OK;
}

}  // extern "C"
