// GGUF model files straight to the device: the parser of pkg/gguf/gguf.go (header, metadata, tensor table,
// aligned data section), the architecture switches of runtime/config.go:388-507 and the loader rules of
// runtime/loader.go:28-212 / 507-708 (which tensors stay in block format, which become float32, tied output head).
//
// The file is mapped read-only; tensor bytes go page cache -> pinned staging (two buffers, copy of one
// overlapping the PCIe transfer of the other) -> device, and quantised embeddings are expanded to float32
// on the device by the bit-exact dequantisation kernels instead of on the host.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdarg>
#include <map>
#include <string>

#include "vx_common.cuh"

namespace {

enum MetaType : uint32_t {   // gguf.go:21-35
    MT_U8 = 0, MT_I8 = 1, MT_U16 = 2, MT_I16 = 3, MT_U32 = 4, MT_I32 = 5, MT_F32 = 6, MT_BOOL = 7, MT_STR = 8, MT_ARR = 9,
    MT_U64 = 10, MT_I64 = 11, MT_F64 = 12
};

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0; int64_t i = 0; double f = 0; bool b = false;
    std::string s;
    uint32_t arr_type = 0; uint64_t arr_len = 0;
    // MetadataValue.AsUint32 / AsUint64 / AsFloat32 (gguf.go:161-206): other types read as zero
    uint32_t as_u32() const { return type == MT_U32 ? (uint32_t)u : type == MT_U64 ? (uint32_t)u : type == MT_I32 ? (uint32_t)i : 0u; }
    uint64_t as_u64() const { return (type == MT_U64 || type == MT_U32) ? u : 0ull; }
    float as_f32() const { return type == MT_F32 ? (float)f : type == MT_F64 ? (float)f : 0.f; }
};

struct TensorInfo { std::string name; int n_dims = 0; uint64_t ne[4] = {1, 1, 1, 1}; uint32_t type = 0; uint64_t offset = 0; uint64_t bytes = 0; };

// TensorType.BlockSize / BytesPerBlock (gguf.go:97-140) for the types this library can place on the device
bool type_geometry(uint32_t t, uint64_t *block, uint64_t *bpb) {
    switch (t) {
        case VX_T_F32: *block = 1; *bpb = 4; return true;
        case VX_T_F16: *block = 1; *bpb = 2; return true;
        case VX_T_Q4_0: *block = 32; *bpb = 18; return true;
        case VX_T_Q4_K: *block = 256; *bpb = 144; return true;
        case VX_T_Q6_K: *block = 256; *bpb = 210; return true;
        case 3: *block = 32; *bpb = 20; return true;      // Q4_1 .. BF16: sizes known so the table parses; not loadable
        case 6: *block = 32; *bpb = 22; return true;
        case 7: *block = 32; *bpb = 24; return true;
        case 8: *block = 32; *bpb = 34; return true;
        case 13: *block = 256; *bpb = 176; return true;
        case 30: *block = 1; *bpb = 2; return true;
        default: return false;
    }
}

}  // namespace

struct vx_gguf {
    int fd = -1; const uint8_t *base = nullptr; size_t size = 0;
    uint32_t version = 0; uint64_t data_offset = 0;
    std::map<std::string, MetaValue> meta;
    std::vector<TensorInfo> tensors;
    std::map<std::string, int> by_name;
    char err[512] = {0};
    int fail(const char *fmt, ...) {
        va_list ap; va_start(ap, fmt); vsnprintf(err, sizeof(err), fmt, ap); va_end(ap);
        return VX_E_BAD_ARG;
    }
    const MetaValue *get(const std::string &k) const { auto it = meta.find(k); return it == meta.end() ? nullptr : &it->second; }
    const TensorInfo *find(const std::string &name) const {
        auto it = by_name.find(name);
        return it == by_name.end() ? nullptr : &tensors[it->second];
    }
};

namespace {

struct Cursor {
    const uint8_t *p; size_t n, at = 0; bool ok = true;
    template <typename T> T rd() {
        T v{};
        if (!ok || at + sizeof(T) > n) { ok = false; return v; }
        memcpy(&v, p + at, sizeof(T)); at += sizeof(T);
        return v;
    }
    bool str(std::string *out) {                                        // readString (gguf.go:336-349): length capped at 65535
        uint64_t len = rd<uint64_t>();
        if (!ok || len > 65535 || at + len > n) { ok = false; return false; }
        if (out) out->assign((const char *)p + at, (size_t)len);
        at += (size_t)len;
        return true;
    }
    bool skip(uint64_t bytes) { if (!ok || bytes > n - at) { ok = false; return false; } at += (size_t)bytes; return true; }
};

bool read_scalar(Cursor &c, uint32_t t, MetaValue *v) {
    switch (t) {
        case MT_U8: v->u = c.rd<uint8_t>(); break;
        case MT_I8: v->i = c.rd<int8_t>(); break;
        case MT_U16: v->u = c.rd<uint16_t>(); break;
        case MT_I16: v->i = c.rd<int16_t>(); break;
        case MT_U32: v->u = c.rd<uint32_t>(); break;
        case MT_I32: v->i = c.rd<int32_t>(); break;
        case MT_U64: v->u = c.rd<uint64_t>(); break;
        case MT_I64: v->i = c.rd<int64_t>(); break;
        case MT_F32: v->f = c.rd<float>(); break;
        case MT_F64: v->f = c.rd<double>(); break;
        case MT_BOOL: v->b = c.rd<uint8_t>() != 0; break;
        case MT_STR: return c.str(&v->s);
        default: return false;
    }
    return c.ok;
}

size_t scalar_size(uint32_t t) {
    switch (t) {
        case MT_U8: case MT_I8: case MT_BOOL: return 1;
        case MT_U16: case MT_I16: return 2;
        case MT_U32: case MT_I32: case MT_F32: return 4;
        case MT_U64: case MT_I64: case MT_F64: return 8;
        default: return 0;
    }
}

int parse(vx_gguf *g) {
    Cursor c{g->base, g->size};
    uint32_t magic = c.rd<uint32_t>();
    if (!c.ok || magic != 0x46554747u) return g->fail("invalid magic: got 0x%08X, want 0x46554747", magic);   // gguf.go:13, 283-285
    g->version = c.rd<uint32_t>();
    if (!c.ok || g->version < 2 || g->version > 3) return g->fail("unsupported version: %u", g->version);       // gguf.go:291-293
    uint64_t n_tensors = c.rd<uint64_t>(), n_meta = c.rd<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_meta > (1u << 24)) return g->fail("implausible header counts");
    for (uint64_t i = 0; i < n_meta; i++) {
        std::string key;
        if (!c.str(&key)) return g->fail("failed to read metadata %llu: key", (unsigned long long)i);
        MetaValue v; v.type = c.rd<uint32_t>();
        if (v.type == MT_ARR) {
            v.arr_type = c.rd<uint32_t>(); v.arr_len = c.rd<uint64_t>();
            if (!c.ok) return g->fail("failed to read metadata %s", key.c_str());
            if (v.arr_type == MT_STR) { for (uint64_t j = 0; j < v.arr_len && c.ok; j++) c.str(nullptr); }
            else {
                size_t es = scalar_size(v.arr_type);
                if (es == 0) return g->fail("metadata %s: unsupported array element type %u", key.c_str(), v.arr_type);
                if (v.arr_len > g->size) return g->fail("metadata %s: array longer than the file", key.c_str());
                c.skip(v.arr_len * es);
            }
            if (!c.ok) return g->fail("failed to read metadata %s: truncated array", key.c_str());
        } else if (!read_scalar(c, v.type, &v)) {
            return g->fail("failed to read value for %s (type %u)", key.c_str(), v.type);
        }
        g->meta[key] = std::move(v);
    }
    g->tensors.resize((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {                           // readTensorInfo (gguf.go:463-501)
        TensorInfo &t = g->tensors[(size_t)i];
        if (!c.str(&t.name)) return g->fail("failed to read tensor info %llu: name", (unsigned long long)i);
        uint32_t nd = c.rd<uint32_t>();
        if (!c.ok || nd > 4) return g->fail("tensor %s: %u dimensions", t.name.c_str(), nd);
        t.n_dims = (int)nd;
        for (uint32_t d = 0; d < nd; d++) t.ne[d] = c.rd<uint64_t>();
        t.type = c.rd<uint32_t>(); t.offset = c.rd<uint64_t>();
        if (!c.ok) return g->fail("failed to read tensor info %llu", (unsigned long long)i);
        g->by_name[t.name] = (int)i;
    }
    uint64_t align = 32;                                                 // gguf.go:325-333
    if (const MetaValue *a = g->get("general.alignment")) align = a->as_u64();
    if (align == 0 || (align & (align - 1))) return g->fail("general.alignment = %llu is not a power of two", (unsigned long long)align);
    g->data_offset = ((uint64_t)c.at + align - 1) / align * align;
    for (TensorInfo &t : g->tensors) {                                   // ReadTensorData's size rule (gguf.go:596-603)
        uint64_t block, bpb, ne = 1;
        for (int d = 0; d < t.n_dims; d++) {
            if (t.ne[d] != 0 && ne > UINT64_MAX / t.ne[d]) return g->fail("tensor %s: element count overflows", t.name.c_str());
            ne *= t.ne[d];
        }
        if (t.n_dims == 0) ne = 0;
        if (!type_geometry(t.type, &block, &bpb)) { t.bytes = 0; continue; }   // unknown type: listed, not loadable
        t.bytes = (ne + block - 1) / block * bpb;
        if (g->data_offset + t.offset > g->size || t.bytes > g->size - g->data_offset - t.offset)
            return g->fail("tensor %s runs past the end of the file", t.name.c_str());
    }
    return VX_OK;
}

// host -> device through two pinned staging buffers: the memcpy out of the page cache overlaps the previous DMA
struct Stager {
    static constexpr size_t CHUNK = 32u << 20;
    void *pin[2] = {nullptr, nullptr}; cudaEvent_t done[2] = {nullptr, nullptr}; int cur = 0;
    ~Stager() { for (int i = 0; i < 2; i++) { if (pin[i]) cudaFreeHost(pin[i]); if (done[i]) cudaEventDestroy(done[i]); } }
    int init(vx_ctx *c) {
        for (int i = 0; i < 2; i++) {
            VX_CUDA(c, cudaMallocHost(&pin[i], CHUNK));
            VX_CUDA(c, cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
        }
        return VX_OK;
    }
    int upload(vx_ctx *c, void *dst, const uint8_t *src, size_t bytes) {
        for (size_t off = 0; off < bytes; off += CHUNK) {
            size_t n = std::min(CHUNK, bytes - off);
            VX_CUDA(c, cudaEventSynchronize(done[cur]));
            memcpy(pin[cur], src + off, n);
            VX_CUDA(c, cudaMemcpyAsync((char *)dst + off, pin[cur], n, cudaMemcpyHostToDevice, c->stream));
            VX_CUDA(c, cudaEventRecord(done[cur], c->stream));
            cur ^= 1;
        }
        return VX_OK;
    }
};

// alternativeGGUFNames (runtime/loader.go:388-403): the name, without ".weight", with a "model." prefix
const TensorInfo *find_alt(const vx_gguf *g, const std::string &name) {
    if (const TensorInfo *t = g->find(name)) return t;
    const std::string suf = ".weight";
    if (name.size() > suf.size() && name.compare(name.size() - suf.size(), suf.size(), suf) == 0)
        if (const TensorInfo *t = g->find(name.substr(0, name.size() - suf.size()))) return t;
    if (name.compare(0, 6, "model.") != 0)
        if (const TensorInfo *t = g->find("model." + name)) return t;
    return nullptr;
}

}  // namespace

extern "C" {

// gguf.Open (pkg/gguf/gguf.go:246-266): parses the header; tensor data stays in the mapping
int vx_gguf_open(const char *path, vx_gguf **out) {
    if (!path || !out) return VX_E_BAD_ARG;
    vx_gguf *g = new vx_gguf();
    *out = g;                                       // returned even on failure so that vx_gguf_error can be read; close it
    g->fd = open(path, O_RDONLY);
    if (g->fd < 0) return g->fail("failed to open file: %s", path);
    struct stat st;
    if (fstat(g->fd, &st) != 0 || st.st_size < 24) return g->fail("failed to read magic: file too short");
    g->size = (size_t)st.st_size;
    void *p = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (p == MAP_FAILED) return g->fail("mmap of %zu bytes failed", g->size);
    g->base = (const uint8_t *)p;
    return parse(g);
}

int vx_gguf_close(vx_gguf *g) {
    if (!g) return VX_E_BAD_ARG;
    if (g->base) munmap((void *)g->base, g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
    return VX_OK;
}

const char *vx_gguf_error(vx_gguf *g) { return g ? g->err : "nil gguf handle"; }

int vx_gguf_tensor_count(vx_gguf *g) { return g ? (int)g->tensors.size() : -1; }

// TensorInfo of tensor `index` (gguf.go:208-214); dims in GGUF order (ne[0] innermost); file_offset is absolute
int vx_gguf_tensor_info(vx_gguf *g, int index, char *name, int name_cap, int *ggml_type, int *n_dims, uint64_t *ne4, uint64_t *file_offset,
                        uint64_t *bytes) {
    if (!g || index < 0 || index >= (int)g->tensors.size()) return VX_E_BAD_ARG;
    const TensorInfo &t = g->tensors[index];
    if (name && name_cap > 0) snprintf(name, (size_t)name_cap, "%s", t.name.c_str());
    if (ggml_type) *ggml_type = (int)t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (ne4) for (int d = 0; d < 4; d++) ne4[d] = t.ne[d];
    if (file_offset) *file_offset = g->data_offset + t.offset;
    if (bytes) *bytes = t.bytes;
    return VX_OK;
}

// one metadata value as text (strings verbatim, numbers printed, arrays as "[type;len]"); VX_E_NO_SEQ when absent
int vx_gguf_meta(vx_gguf *g, const char *key, char *out, int cap) {
    if (!g || !key || !out || cap <= 0) return VX_E_BAD_ARG;
    const MetaValue *v = g->get(key);
    if (!v) return VX_E_NO_SEQ;
    switch (v->type) {
        case MT_STR: snprintf(out, (size_t)cap, "%s", v->s.c_str()); break;
        case MT_F32: case MT_F64: snprintf(out, (size_t)cap, "%.9g", v->f); break;
        case MT_BOOL: snprintf(out, (size_t)cap, "%s", v->b ? "true" : "false"); break;
        case MT_ARR: snprintf(out, (size_t)cap, "[%u;%llu]", v->arr_type, (unsigned long long)v->arr_len); break;
        case MT_I8: case MT_I16: case MT_I32: case MT_I64: snprintf(out, (size_t)cap, "%lld", (long long)v->i); break;
        default: snprintf(out, (size_t)cap, "%llu", (unsigned long long)v->u); break;
    }
    return VX_OK;
}

// extractModelConfig (pkg/gguf/gguf.go:503-584) followed by ModelConfigFromGGUF (runtime/config.go:388-507).
// Fills the architecture fields of *cfg; the pool and batch limits (max_*) are the caller's and are left alone.
int vx_gguf_model_config(vx_gguf *g, vx_model_config *cfg) {
    if (!g || !cfg) return VX_E_BAD_ARG;
    std::string arch = "llama";
    if (const MetaValue *v = g->get("general.architecture")) if (!v->s.empty()) arch = v->s;
    const std::string pre = arch + ".";
    auto u32 = [&](const std::string &k, uint32_t dflt) { const MetaValue *v = g->get(k); return v ? v->as_u32() : dflt; };
    auto f32 = [&](const std::string &k, float dflt) { const MetaValue *v = g->get(k); return v ? v->as_f32() : dflt; };
    cfg->n_layers = (int)u32(pre + "block_count", 0);
    cfg->hidden = (int)u32(pre + "embedding_length", 0);
    cfg->n_heads = (int)u32(pre + "attention.head_count", 0);
    cfg->n_kv_heads = (int)u32(pre + "attention.head_count_kv", (uint32_t)cfg->n_heads);       // default MHA
    cfg->ffn = (int)u32(pre + "feed_forward_length", 0);
    cfg->rope_theta = f32(pre + "rope.freq_base", 10000.0f);
    if (cfg->rope_theta == 0.f) cfg->rope_theta = 10000.0f;
    cfg->rms_eps = f32(pre + "attention.layer_norm_rms_epsilon", 0.f);
    if (cfg->rms_eps == 0.f) cfg->rms_eps = 1e-5f;
    cfg->head_dim = (int)u32(pre + "attention.key_length", 0);
    cfg->sliding_window = (int)u32(pre + "attention.sliding_window", 0);
    cfg->vocab = 0;
    if (const MetaValue *v = g->get("tokenizer.ggml.tokens")) if (v->type == MT_ARR) cfg->vocab = (int)v->arr_len;
    const TensorInfo *emb = find_alt(g, "token_embd.weight");
    if (cfg->vocab == 0 && emb && emb->n_dims == 2) cfg->vocab = (int)emb->ne[1];              // files without a tokenizer section
    if (cfg->n_layers <= 0 || cfg->hidden <= 0 || cfg->n_heads <= 0 || cfg->n_kv_heads <= 0 || cfg->ffn <= 0 || cfg->vocab <= 0)
        return g->fail("model metadata incomplete (arch %s: layers %d hidden %d heads %d/%d ffn %d vocab %d)", arch.c_str(), cfg->n_layers,
                       cfg->hidden, cfg->n_heads, cfg->n_kv_heads, cfg->ffn, cfg->vocab);
    if (cfg->head_dim == 0) cfg->head_dim = cfg->hidden / cfg->n_heads;                          // runtime/config.go:150-160
    uint32_t rope_dim = u32(pre + "rope.dimension_count", 0);
    if (rope_dim != 0 && (int)rope_dim != cfg->head_dim) {
        snprintf(g->err, sizeof(g->err), "partial rotary embedding (%u of %d dims) is outside the batched path", rope_dim, cfg->head_dim);
        return VX_E_UNSUPPORTED;
    }
    cfg->rope_neox = 0; cfg->geglu = 0; cfg->post_norms = 0; cfg->embed_scale = 0.f; cfg->attn_softcap = 0.f; cfg->window_alternating = 0;
    cfg->final_softcap = f32(arch + ".final_logit_softcapping", 0.f);
    if (arch == "llama" || arch == "mistral") {
    } else if (arch == "gemma") {
        cfg->geglu = 1; cfg->embed_scale = (float)std::sqrt((double)cfg->hidden);
    } else if (arch == "gemma2") {
        cfg->geglu = 1; cfg->embed_scale = (float)std::sqrt((double)cfg->hidden);
        cfg->attn_softcap = f32(arch + ".attn_logit_softcapping", 0.f);
        if (cfg->attn_softcap == 0.f) cfg->attn_softcap = 50.0f;
        cfg->window_alternating = 1; cfg->post_norms = 1;
    } else {
        snprintf(g->err, sizeof(g->err), "architecture %s needs biases, LayerNorm, fused or expert tensors that the batched path does not carry",
                 arch.c_str());
        return VX_E_UNSUPPORTED;
    }
    if (!cfg->window_alternating) cfg->sliding_window = 0;      // the paged path applies a window on alternating layers only (block.go:464-476)
    return VX_OK;
}

// LoadWeightsGGUF + CopyWeightsToDevice (runtime/loader.go:28-212, 507-708) for the batched path, then vx_model_finalize.
// Projection matrices keep their block format (Q4_0 / Q4_K / Q6_K); norm vectors must be float32; the token embedding
// becomes float32 unless it is Q4_0 (whose rows the lookup kernel expands to the same values); a missing output.weight
// ties the head to the embedding (loader.go:597-600).
int vx_model_load_gguf(vx_model *m, vx_gguf *g) {
    if (!m || !g) return VX_E_BAD_ARG;
    vx_ctx *c = vx_model_ctx(m);
    VxGuard guard(c);
    vx_model_config cf;
    VX_TRY(vx_model_get_config(m, &cf));
    Stager st;
    VX_TRY(st.init(c));
    void *stage_dev = nullptr; size_t stage_cap = 0;
    auto dev_buf = [&](size_t bytes) -> int {
        if (bytes <= stage_cap) return VX_OK;
        if (stage_dev) cudaFree(stage_dev);
        stage_dev = nullptr; stage_cap = 0;
        if (cudaMalloc(&stage_dev, bytes) != cudaSuccess) { cudaGetLastError(); return vx_fail(c, VX_E_OOM, "cudaMalloc(%zu) for tensor staging failed", bytes); }
        stage_cap = bytes;
        return VX_OK;
    };
    auto finish = [&](int rc) { if (stage_dev) { cudaStreamSynchronize(c->stream); cudaFree(stage_dev); } return rc; };
    // one tensor: checks the shape, streams the bytes to the device and hands them to the model
    auto put = [&](const TensorInfo *t, int layer, int slot, int n, int k, bool norm, bool embed) -> int {
        uint64_t want_ne0 = (uint64_t)k, want_ne1 = (uint64_t)n;
        bool shape_ok = norm ? (t->n_dims == 1 && t->ne[0] == want_ne0) : (t->n_dims == 2 && t->ne[0] == want_ne0 && t->ne[1] == want_ne1);
        if (!shape_ok)
            return vx_fail(c, VX_E_BAD_ARG, "tensor %s has shape [%llu, %llu] (GGUF order), the model wants [%d, %d]", t->name.c_str(),
                           (unsigned long long)t->ne[0], (unsigned long long)t->ne[1], k, norm ? 1 : n);
        int type = (int)t->type;
        const bool known = type == VX_T_F32 || type == VX_T_F16 || type == VX_T_Q4_0 || type == VX_T_Q4_K || type == VX_T_Q6_K;
        if (!known || t->bytes == 0) return vx_fail(c, VX_E_UNSUPPORTED, "tensor %s has GGUF type %d, which has no device kernel here", t->name.c_str(), type);
        VX_TRY(dev_buf(t->bytes));
        VX_TRY(st.upload(c, stage_dev, g->base + g->data_offset + t->offset, (size_t)t->bytes));
        const bool expand = (norm && type != VX_T_F32) || (embed && type != VX_T_Q4_0 && type != VX_T_F32);
        if (expand) {                                   // gguf.Dequantize on the device (loader.go:186-199)
            void *f32 = nullptr; size_t ne = (size_t)n * k;
            if (cudaMalloc(&f32, ne * 4) != cudaSuccess) { cudaGetLastError(); return vx_fail(c, VX_E_OOM, "cudaMalloc(%zu) failed", ne * 4); }
            int rc = vx_dequantize(c, type, (vx_dptr)stage_dev, (vx_dptr)f32, (int64_t)ne);
            if (rc == VX_OK) rc = vx_model_set_tensor(m, layer, slot, VX_T_F32, f32, ne * 4, 1);
            cudaStreamSynchronize(c->stream); cudaFree(f32);
            return rc;
        }
        return vx_model_set_tensor(m, layer, slot, type, stage_dev, (size_t)t->bytes, 1);
    };
    const int H = cf.hidden, qd = cf.n_heads * cf.head_dim, kvd = cf.n_kv_heads * cf.head_dim, F = cf.ffn;
    struct SlotName { int slot; const char *suffix; int n, k; bool norm, optional; };
    const SlotName per_layer[] = {                                       // GetLayerTensorName (pkg/gguf/loader.go:132-229)
        {VX_W_ATTN_NORM, "attn_norm.weight", 1, H, true, false},
        {VX_W_WQ, "attn_q.weight", qd, H, false, false}, {VX_W_WK, "attn_k.weight", kvd, H, false, false},
        {VX_W_WV, "attn_v.weight", kvd, H, false, false}, {VX_W_WO, "attn_output.weight", H, qd, false, false},
        {VX_W_POST_ATTN_NORM, "post_attention_norm.weight", 1, H, true, !cf.post_norms},
        {VX_W_FFN_NORM, "ffn_norm.weight", 1, H, true, false},
        {VX_W_W1, "ffn_gate.weight", F, H, false, false}, {VX_W_W3, "ffn_up.weight", F, H, false, false},
        {VX_W_W2, "ffn_down.weight", H, F, false, false},
        {VX_W_POST_FFN_NORM, "post_ffw_norm.weight", 1, H, true, !cf.post_norms},
    };
    for (int l = 0; l < cf.n_layers; l++)
        for (const SlotName &s : per_layer) {
            if (s.optional) continue;
            std::string name = "blk." + std::to_string(l) + "." + s.suffix;
            const TensorInfo *t = find_alt(g, name);
            if (!t) return finish(vx_fail(c, VX_E_BAD_ARG, "tensor %s not found", name.c_str()));
            int rc = put(t, l, s.slot, s.n, s.k, s.norm, false);
            if (rc != VX_OK) return finish(rc);
        }
    const TensorInfo *emb = find_alt(g, "token_embd.weight"), *fin = find_alt(g, "output_norm.weight"), *head = find_alt(g, "output.weight");
    if (!emb || !fin) return finish(vx_fail(c, VX_E_BAD_ARG, "tensor %s not found", emb ? "output_norm.weight" : "token_embd.weight"));
    int rc = put(emb, -1, VX_G_EMBED, cf.vocab, H, false, true);
    if (rc == VX_OK) rc = put(fin, -1, VX_G_FINAL_NORM, 1, H, true, false);
    if (rc == VX_OK) rc = put(head ? head : emb, -1, VX_G_OUTPUT, cf.vocab, H, false, false);   // tied weights when output.weight is absent
    if (rc != VX_OK) return finish(rc);
    rc = finish(VX_OK);
    if (rc != VX_OK) return rc;
    return vx_model_finalize(m);
}

}  // extern "C"
