// GGUF v3 reader and tensor binding (host code): the file side of the path.
//
// Follows the reference's `mod gguf` (recipe.rs:9786-10326): little-endian header (magic "GGUF",
// version 3, tensor count, metadata pair count), metadata values of the thirteen GGUF kinds with
// nested arrays, tensor descriptors (name, dimensions, GGML type, offset into the data section),
// the data section aligned to general.alignment (32 unless the file says otherwise), every tensor
// checked to lie inside the file. Split models (split.count shards named
// <stem>-0000i-of-0000n.gguf) are opened together. The file is mapped read-only; a tensor's bytes are
// a pointer into the mapping, in the GGML block layout the kernels take, so binding a tensor is
// rq_weight_prepare on that pointer. Expert slices follow GgufTensor::expert (recipe.rs:9862-9869):
// expert e of a [k, n, experts] tensor is rows e*n .. (e+1)*n.
//
// Nothing here touches a GPU except rq_gguf_bind / rq_gguf_bind_experts, which upload.
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <vector>

#include "rq_internal.cuh"

namespace {

struct Layout { const char* name; int block, stride; };
// GGML type id -> name, elements per block, bytes per block (layout(), recipe.rs:9925-9962; QUANTIZATIONS :15811-15822)
bool layout_of(uint32_t kind, Layout* out) {
    switch (kind) {
        case 0: *out = {"F32", 1, 4}; return true;
        case 1: *out = {"F16", 1, 2}; return true;
        case 24: *out = {"I8", 1, 1}; return true;
        case 25: *out = {"I16", 1, 2}; return true;
        case 26: *out = {"I32", 1, 4}; return true;
        case 27: *out = {"I64", 1, 8}; return true;
        case 28: *out = {"F64", 1, 8}; return true;
        case 30: *out = {"BF16", 1, 2}; return true;
        case 2: *out = {"q4_0", 32, 18}; return true;
        case 3: *out = {"q4_1", 32, 20}; return true;
        case 6: *out = {"q5_0", 32, 22}; return true;
        case 7: *out = {"q5_1", 32, 24}; return true;
        case 8: *out = {"q8_0", 32, 34}; return true;
        case 9: *out = {"q8_1", 32, 36}; return true;
        case 10: *out = {"q2k", 256, 84}; return true;
        case 11: *out = {"q3k", 256, 110}; return true;
        case 12: *out = {"q4k", 256, 144}; return true;
        case 13: *out = {"q5k", 256, 176}; return true;
        case 14: *out = {"q6k", 256, 210}; return true;
        case 15: *out = {"q8k", 256, 292}; return true;
        case 20: *out = {"iq4nl", 32, 18}; return true;
        case 23: *out = {"iq4xs", 256, 136}; return true;
        default: return false;
    }
}

struct Value {
    uint32_t kind = 0;          // GGUF value kind 0..12
    uint64_t bits = 0;          // integers, bool, float bits
    std::string text;           // kind 8
    uint32_t item_kind = 0;     // kind 9
    std::vector<Value> items;   // kind 9
};

struct Tensor {
    std::string name;
    std::vector<uint64_t> shape;
    uint32_t kind;
    uint64_t offset, bytes;
    int shard;
};

struct Shard {
    const uint8_t* base = nullptr;
    size_t length = 0;
    size_t data = 0;  // where the data section starts
};

struct Reader {
    const uint8_t* bytes; size_t length, at; int depth; bool ok; std::string why;
    const uint8_t* take(size_t n) {
        if (!ok) return nullptr;
        if (n > length - at) { ok = false; why = "GGUF header is truncated"; return nullptr; }
        const uint8_t* p = bytes + at;
        at += n;
        return p;
    }
    uint32_t u32() { const uint8_t* p = take(4); uint32_t v = 0; if (p) memcpy(&v, p, 4); return v; }
    uint64_t u64() { const uint8_t* p = take(8); uint64_t v = 0; if (p) memcpy(&v, p, 8); return v; }
    std::string string() {
        const uint64_t n = u64();
        if (ok && n > length - at) { ok = false; why = "GGUF header is truncated"; }
        const uint8_t* p = take((size_t)n);
        return p ? std::string((const char*)p, (size_t)n) : std::string();
    }
    Value value(uint32_t kind) {
        Value v;
        v.kind = kind;
        switch (kind) {
            case 0: case 1: case 7: { const uint8_t* p = take(1); v.bits = p ? p[0] : 0; break; }
            case 2: case 3: { const uint8_t* p = take(2); uint16_t h = 0; if (p) memcpy(&h, p, 2); v.bits = h; break; }
            case 4: case 5: case 6: v.bits = u32(); break;
            case 8: v.text = string(); break;
            case 9: {
                v.item_kind = u32();
                const uint64_t count = u64();
                if (++depth > 64) { ok = false; why = "GGUF arrays nest deeper than 64 levels"; break; }
                if (ok && count > length - at) { ok = false; why = "GGUF header is truncated"; break; }  // every item takes at least a byte
                v.items.reserve((size_t)count);
                for (uint64_t i = 0; i < count && ok; ++i) v.items.push_back(value(v.item_kind));
                --depth;
                break;
            }
            case 10: case 11: case 12: v.bits = u64(); break;
            default: ok = false; why = "GGUF value type " + std::to_string(kind) + " is unsupported";
        }
        return v;
    }
};

// the value as a count or index, whichever integer width the file chose (GgufValue::integer, recipe.rs:9815-9828)
bool integer_of(const Value& v, uint64_t* out) {
    switch (v.kind) {
        case 0: case 2: case 4: case 10: *out = v.bits; return true;
        case 1: { const int8_t s = (int8_t)v.bits; if (s < 0) return false; *out = (uint64_t)s; return true; }
        case 3: { const int16_t s = (int16_t)v.bits; if (s < 0) return false; *out = (uint64_t)s; return true; }
        case 5: { const int32_t s = (int32_t)v.bits; if (s < 0) return false; *out = (uint64_t)s; return true; }
        case 11: { const int64_t s = (int64_t)v.bits; if (s < 0) return false; *out = (uint64_t)s; return true; }
        default: return false;
    }
}

}  // namespace

struct rq_gguf {
    std::vector<Shard> shards;
    std::vector<std::pair<std::string, Value>> metadata;  // the first shard's, in file order
    std::vector<Tensor> tensors;                          // every shard's, in file order
};

namespace {

const Value* find_value(const std::vector<std::pair<std::string, Value>>& md, const char* key) {
    for (const auto& kv : md) if (kv.first == key) return &kv.second;
    return nullptr;
}

int open_shard(const char* path, uint64_t index, Shard* shard, std::vector<std::pair<std::string, Value>>* metadata, std::vector<Tensor>* tensors) {
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return rq_fail(RQ_ERR_INVALID, "cannot open %s", path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size == 0) { close(fd); return rq_fail(RQ_ERR_INVALID, "%s is empty", path); }
    void* map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return rq_fail(RQ_ERR_ALLOC, "cannot map %s", path);
    shard->base = (const uint8_t*)map;
    shard->length = (size_t)st.st_size;
    Reader r{shard->base, shard->length, 0, 0, true, {}};
    auto fail = [&](const std::string& text) {
        munmap(map, shard->length);
        shard->base = nullptr;
        return rq_fail(RQ_ERR_INVALID, "%s: %s", path, text.c_str());
    };
    if (r.u32() != 0x46554747u || !r.ok) return fail("is not a GGUF file");
    const uint32_t version = r.u32();
    if (version != 3) return fail("is GGUF version " + std::to_string(version) + "; version 3 is supported");
    const uint64_t tensor_count = r.u64(), pair_count = r.u64();
    for (uint64_t i = 0; i < pair_count && r.ok; ++i) {
        std::string key = r.string();
        const uint32_t kind = r.u32();
        metadata->emplace_back(std::move(key), r.value(kind));
    }
    if (!r.ok) return fail(r.why);
    uint64_t alignment = 32;
    if (const Value* v = find_value(*metadata, "general.alignment")) integer_of(*v, &alignment);
    if (alignment == 0 || (alignment & (alignment - 1))) return fail("declares alignment " + std::to_string(alignment));
    if (const Value* v = find_value(*metadata, "split.no")) {
        uint64_t declared = 0;
        if (integer_of(*v, &declared) && declared != index) return fail("is shard " + std::to_string(declared) + ", expected shard " + std::to_string(index));
    }
    for (uint64_t i = 0; i < tensor_count && r.ok; ++i) {
        Tensor t;
        t.name = r.string();
        const uint32_t dims = r.u32();
        if (dims > 8) return fail("tensor " + t.name + " declares " + std::to_string(dims) + " dimensions");
        uint64_t elements = 1;
        for (uint32_t d = 0; d < dims && r.ok; ++d) {
            const uint64_t extent = r.u64();
            t.shape.push_back(extent);
            if (extent != 0 && elements > UINT64_MAX / extent) return fail("tensor " + t.name + " shape overflows");
            elements *= extent;
        }
        t.kind = r.u32();
        t.offset = r.u64();
        if (!r.ok) break;
        Layout lay;
        if (!layout_of(t.kind, &lay)) return fail("GGUF tensor type " + std::to_string(t.kind) + " is unsupported");
        if (elements % (uint64_t)lay.block) return fail("tensor " + t.name + " holds " + std::to_string(elements) + " elements, not a multiple of its " + std::to_string(lay.block) + "-element block");
        t.bytes = elements / (uint64_t)lay.block * (uint64_t)lay.stride;
        t.shard = 0;
        tensors->push_back(std::move(t));
    }
    if (!r.ok) return fail(r.why);
    shard->data = (size_t)((r.at + alignment - 1) / alignment * alignment);
    for (const Tensor& t : *tensors)
        if (t.offset > shard->length || shard->data > shard->length - t.offset || t.bytes > shard->length - t.offset - shard->data)
            return fail("tensor " + t.name + " runs past the end of the file");
    return RQ_OK;
}

// <stem>-00001-of-0000n.gguf -> the sibling shard `index` of `count`
std::string sibling_path(const std::string& first, uint64_t index, uint64_t count) {
    char tail[64];
    snprintf(tail, sizeof(tail), "-%05llu-of-%05llu.gguf", (unsigned long long)(index + 1), (unsigned long long)count);
    char head[64];
    snprintf(head, sizeof(head), "-%05d-of-%05llu.gguf", 1, (unsigned long long)count);
    const size_t at = first.rfind(head);
    if (at == std::string::npos || at + strlen(head) != first.size()) return std::string();
    return first.substr(0, at) + tail;
}

const Tensor* tensor_at(const rq_gguf* g, int index) { return g && index >= 0 && (size_t)index < g->tensors.size() ? &g->tensors[(size_t)index] : nullptr; }

}  // namespace

extern "C" int rq_gguf_open(const char* path, rq_gguf** out) {
    if (!path || !out) return rq_fail(RQ_ERR_INVALID, "rq_gguf_open: null argument");
    *out = nullptr;
    rq_gguf* g = new (std::nothrow) rq_gguf();
    if (!g) return rq_fail(RQ_ERR_ALLOC, "out of host memory");
    auto drop = [&](int rc) { for (Shard& s : g->shards) if (s.base) munmap((void*)s.base, s.length); delete g; return rc; };
    Shard first;
    std::vector<Tensor> tensors;
    int rc = open_shard(path, 0, &first, &g->metadata, &tensors);
    if (rc) return drop(rc);
    g->shards.push_back(first);
    g->tensors = std::move(tensors);
    uint64_t count = 1;
    if (const Value* v = find_value(g->metadata, "split.count")) integer_of(*v, &count);
    for (uint64_t i = 1; i < count; ++i) {
        const std::string next = sibling_path(path, i, count);
        if (next.empty()) return drop(rq_fail(RQ_ERR_INVALID, "%s names %llu shards but is not named <stem>-00001-of-%05llu.gguf", path, (unsigned long long)count, (unsigned long long)count));
        Shard s;
        std::vector<std::pair<std::string, Value>> md;
        std::vector<Tensor> ts;
        rc = open_shard(next.c_str(), i, &s, &md, &ts);
        if (rc) return drop(rc);
        g->shards.push_back(s);
        for (Tensor& t : ts) { t.shard = (int)i; g->tensors.push_back(std::move(t)); }
    }
    if (const Value* v = find_value(g->metadata, "split.tensors.count")) {
        uint64_t declared = 0;
        if (integer_of(*v, &declared) && declared != g->tensors.size())
            return drop(rq_fail(RQ_ERR_INVALID, "GGUF split declares %llu tensors and holds %zu", (unsigned long long)declared, g->tensors.size()));
    }
    *out = g;
    return RQ_OK;
}

extern "C" void rq_gguf_close(rq_gguf* g) {
    if (!g) return;
    for (Shard& s : g->shards) if (s.base) munmap((void*)s.base, s.length);
    delete g;
}

extern "C" int rq_gguf_tensor_count(const rq_gguf* g) { return g ? (int)g->tensors.size() : 0; }

extern "C" int rq_gguf_find(const rq_gguf* g, const char* name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); ++i) if (g->tensors[i].name == name) return (int)i;
    return -1;
}

extern "C" const char* rq_gguf_tensor_name(const rq_gguf* g, int index) { const Tensor* t = tensor_at(g, index); return t ? t->name.c_str() : nullptr; }
extern "C" int rq_gguf_tensor_type(const rq_gguf* g, int index) { const Tensor* t = tensor_at(g, index); return t ? (int)t->kind : -1; }
extern "C" int rq_gguf_tensor_dims(const rq_gguf* g, int index, int64_t* shape, int capacity) {
    const Tensor* t = tensor_at(g, index);
    if (!t) return -1;
    for (size_t d = 0; d < t->shape.size() && (int)d < capacity; ++d) shape[d] = (int64_t)t->shape[d];
    return (int)t->shape.size();
}
extern "C" int64_t rq_gguf_tensor_bytes(const rq_gguf* g, int index) { const Tensor* t = tensor_at(g, index); return t ? (int64_t)t->bytes : -1; }
extern "C" const void* rq_gguf_tensor_data(const rq_gguf* g, int index) {
    const Tensor* t = tensor_at(g, index);
    if (!t) return nullptr;
    const Shard& s = g->shards[(size_t)t->shard];
    return s.base + s.data + t->offset;
}

extern "C" int rq_gguf_meta_count(const rq_gguf* g) { return g ? (int)g->metadata.size() : 0; }
extern "C" const char* rq_gguf_meta_key(const rq_gguf* g, int index) { return g && index >= 0 && (size_t)index < g->metadata.size() ? g->metadata[(size_t)index].first.c_str() : nullptr; }
extern "C" int rq_gguf_meta_kind(const rq_gguf* g, const char* key) { const Value* v = g && key ? find_value(g->metadata, key) : nullptr; return v ? (int)v->kind : -1; }
extern "C" int rq_gguf_meta_integer(const rq_gguf* g, const char* key, uint64_t* out) {
    const Value* v = g && key ? find_value(g->metadata, key) : nullptr;
    if (!v || !out) return rq_fail(RQ_ERR_INVALID, "%s is absent", key ? key : "(null)");
    if (v->kind == 7) { *out = v->bits != 0; return RQ_OK; }
    if (!integer_of(*v, out)) return rq_fail(RQ_ERR_INVALID, "%s is not a nonnegative integer", key);
    return RQ_OK;
}
extern "C" int rq_gguf_meta_float(const rq_gguf* g, const char* key, double* out) {
    const Value* v = g && key ? find_value(g->metadata, key) : nullptr;
    if (!v || !out) return rq_fail(RQ_ERR_INVALID, "%s is absent", key ? key : "(null)");
    if (v->kind == 6) { float f; const uint32_t b = (uint32_t)v->bits; memcpy(&f, &b, 4); *out = f; return RQ_OK; }
    if (v->kind == 12) { memcpy(out, &v->bits, 8); return RQ_OK; }
    return rq_fail(RQ_ERR_INVALID, "%s is not a float", key);
}
extern "C" const char* rq_gguf_meta_text(const rq_gguf* g, const char* key) {
    const Value* v = g && key ? find_value(g->metadata, key) : nullptr;
    return v && v->kind == 8 ? v->text.c_str() : nullptr;
}
extern "C" int64_t rq_gguf_meta_array_length(const rq_gguf* g, const char* key) {
    const Value* v = g && key ? find_value(g->metadata, key) : nullptr;
    return v && v->kind == 9 ? (int64_t)v->items.size() : -1;
}
extern "C" const char* rq_gguf_meta_array_text(const rq_gguf* g, const char* key, int64_t index) {
    const Value* v = g && key ? find_value(g->metadata, key) : nullptr;
    if (!v || v->kind != 9 || index < 0 || (size_t)index >= v->items.size() || v->items[(size_t)index].kind != 8) return nullptr;
    return v->items[(size_t)index].text.c_str();
}

// Rows [row_first, row_first + row_count) of a [k, n] or [k, n, experts] tensor (rows of the first dimension, all
// experts' rows one after another) as a resident weight. row_count <= 0: every row.
extern "C" int rq_gguf_bind(rq_ctx* ctx, const rq_gguf* g, const char* name, int64_t row_first, int64_t row_count, rq_weight** out) {
    if (!ctx || !g || !name || !out) return rq_fail(RQ_ERR_INVALID, "rq_gguf_bind: null argument");
    *out = nullptr;
    const int index = rq_gguf_find(g, name);
    if (index < 0) return rq_fail(RQ_ERR_INVALID, "tensor %s is absent", name);
    const Tensor& t = g->tensors[(size_t)index];
    if (!rq_block_values((int)t.kind)) {
        Layout lay;
        layout_of(t.kind, &lay);
        return rq_fail(RQ_ERR_UNSUPPORTED, "tensor %s is stored as %s, which this library does not dot; it serves Q4_0(2) Q8_0(8) Q4_K(12) Q6_K(14)", name, lay.name);
    }
    if (t.shape.size() < 2) return rq_fail(RQ_ERR_INVALID, "tensor %s has %zu dimensions; a row slice takes at least [k, n]", name, t.shape.size());
    const int64_t cols = (int64_t)t.shape[0];
    int64_t rows = 1;
    for (size_t d = 1; d < t.shape.size(); ++d) rows *= (int64_t)t.shape[d];
    if (row_count <= 0) { row_first = 0; row_count = rows; }
    return rq_weight_prepare(ctx, (int)t.kind, rq_gguf_tensor_data(g, index), rows, cols, row_first, row_count, out);
}

// The expert tables of one gguf_moe block from their three [k, n, experts] tensors (ffn_gate_exps, ffn_up_exps,
// ffn_down_exps) and, optionally, a gated shared expert's three [k, n] tensors and fp32 gate vector.
extern "C" int rq_gguf_bind_experts(rq_ctx* ctx, const rq_gguf* g, const char* gate, const char* up, const char* down, int expert_first, int expert_count,
                                    const char* shared_gate, const char* shared_up, const char* shared_down, const char* shared_gate_vector, rq_moe** out) {
    if (!ctx || !g || !gate || !up || !down || !out) return rq_fail(RQ_ERR_INVALID, "rq_gguf_bind_experts: null argument");
    *out = nullptr;
    const int gi = rq_gguf_find(g, gate), ui = rq_gguf_find(g, up), di = rq_gguf_find(g, down);
    if (gi < 0 || ui < 0 || di < 0) return rq_fail(RQ_ERR_INVALID, "expert tensor %s is absent", gi < 0 ? gate : (ui < 0 ? up : down));
    const Tensor &tg = g->tensors[(size_t)gi], &tu = g->tensors[(size_t)ui], &td = g->tensors[(size_t)di];
    if (tg.shape.size() != 3 || tu.shape != tg.shape || td.shape.size() != 3)
        return rq_fail(RQ_ERR_INVALID, "expert tensors take the shape [k, n, experts]; %s has %zu dimensions", gate, tg.shape.size());
    const int hidden = (int)tg.shape[0], ffn = (int)tg.shape[1], experts = (int)tg.shape[2];
    if ((int)td.shape[0] != ffn || (int)td.shape[1] != hidden || (int)td.shape[2] != experts || tu.kind != tg.kind || td.kind != tg.kind)
        return rq_fail(RQ_ERR_INVALID, "expert tensors %s / %s / %s do not describe one bank ([hidden, ffn, experts] x 2, [ffn, hidden, experts], one format)", gate, up, down);
    if (expert_count <= 0) { expert_first = 0; expert_count = experts; }
    const void *sg = nullptr, *su = nullptr, *sd = nullptr;
    const float* sv = nullptr;
    if (shared_gate || shared_up || shared_down || shared_gate_vector) {
        const int a = shared_gate ? rq_gguf_find(g, shared_gate) : -1, b = shared_up ? rq_gguf_find(g, shared_up) : -1, c = shared_down ? rq_gguf_find(g, shared_down) : -1,
                  d = shared_gate_vector ? rq_gguf_find(g, shared_gate_vector) : -1;
        if (a < 0 || b < 0 || c < 0 || d < 0) return rq_fail(RQ_ERR_INVALID, "a shared expert needs its gate, up and down tensors and its gate vector; one is absent");
        if (g->tensors[(size_t)a].kind != tg.kind || g->tensors[(size_t)b].kind != tg.kind || g->tensors[(size_t)c].kind != tg.kind || g->tensors[(size_t)d].kind != 0)
            return rq_fail(RQ_ERR_INVALID, "the shared expert must be stored in the bank's format and its gate vector as F32");
        sg = rq_gguf_tensor_data(g, a); su = rq_gguf_tensor_data(g, b); sd = rq_gguf_tensor_data(g, c);
        sv = (const float*)rq_gguf_tensor_data(g, d);
    }
    return rq_moe_prepare(ctx, (int)tg.kind, rq_gguf_tensor_data(g, gi), rq_gguf_tensor_data(g, ui), rq_gguf_tensor_data(g, di), experts, expert_first, expert_count,
                          hidden, ffn, sg, su, sd, sv, out);
}
