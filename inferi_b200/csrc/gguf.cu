// GGUF container reader (host code) and the GGUF -> device loader of the Llama model.
//
// Replaces `Gguf::from_bytes` / `load_header` / `load_metadata` / `load_tensors` (crates/inferi/src/gguf.rs:516-692),
// `Llama2Config::from_gguf` (crates/inferi/src/models/llama2/cpu.rs:74-107) and `Llama2Weights::from_gguf`
// (crates/inferi/src/models/llama2/transformer.rs:294-394).
//
// Differences by design: the file is memory-mapped and tensors are handed to the device straight from the mapping
// (the reference copies every tensor into typed vectors first, gguf.rs:611-689); `token_embd` stays quantized (the
// reference dequantizes the whole table to f32, transformer.rs:367-374); a tensor-parallel rank uploads only its slice;
// every read is bounds-checked and a malformed file is an error code, not a panic (rank > 4: gguf.rs:583-586).
#include "common.cuh"

#include <errno.h>
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <unordered_map>
#include <vector>

using namespace ib;

namespace {

constexpr uint32_t GGUF_MAGIC_LE = 0x46554747u;   // "GGUF" (gguf.rs:19)

// metadata value types (gguf.rs:397-428)
enum MetaType : int32_t { MT_U8 = 0, MT_I8, MT_U16, MT_I16, MT_U32, MT_I32, MT_F32, MT_BOOL, MT_STRING, MT_ARRAY, MT_U64, MT_I64, MT_F64 };

struct MetaValue {
    int32_t type = -1;
    uint64_t u = 0;          // integer / bool payload (sign-extended for signed types)
    double f = 0.0;          // float payload
    const char *str = nullptr;
    uint64_t str_len = 0;
    int32_t elem_type = -1;  // arrays
    uint64_t count = 0;
    uint64_t data_off = 0;   // file offset of the first array element
    std::vector<uint64_t> str_offsets;   // filled on first indexed access of a string array
};

struct TensorRec {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};   // slowest first, as the reference keeps them (gguf.rs:587-593)
    int32_t type = -1;
    uint64_t offset = 0;               // from the start of the file
    uint64_t nbytes = 0;               // 0: a type this reader does not size
};

// bytes per block / elements per block of the ggml tensor types (gguf.rs:74-106 names the ids)
bool type_size(int32_t t, uint32_t &bytes, uint32_t &elems) {
    switch (t) {
    case 0: bytes = 4; elems = 1; return true;       // F32
    case 1: bytes = 2; elems = 1; return true;       // F16
    case 2: bytes = 18; elems = 32; return true;     // Q4_0
    case 3: bytes = 20; elems = 32; return true;     // Q4_1
    case 6: bytes = 22; elems = 32; return true;     // Q5_0
    case 7: bytes = 24; elems = 32; return true;     // Q5_1
    case 8: bytes = 34; elems = 32; return true;     // Q8_0
    case 12: bytes = 144; elems = 256; return true;  // Q4_K
    case 13: bytes = 176; elems = 256; return true;  // Q5_K
    case 14: bytes = 210; elems = 256; return true;  // Q6_K
    case 15: bytes = 292; elems = 256; return true;  // Q8_K
    default: return false;
    }
}

}  // namespace

struct ib_gguf {
    const uint8_t *base = nullptr;
    uint64_t size = 0;
    bool mapped = false;
    uint32_t version = 0, alignment = 32;
    uint64_t n_tensors = 0, n_meta = 0, data_start = 0;
    std::unordered_map<std::string, MetaValue> meta;
    std::vector<std::string> meta_keys;
    std::vector<TensorRec> tensors;
    std::unordered_map<std::string, size_t> by_name;
};

namespace {

struct Cursor {
    const uint8_t *base;
    uint64_t size, off = 0;
    bool ok = true;
    template <typename T> T pod() {
        T v{};
        if (!ok || off > size || size - off < sizeof(T)) { ok = false; return v; }
        memcpy(&v, base + off, sizeof(T));   // unaligned reads (gguf.rs `read_pod`)
        off += sizeof(T);
        return v;
    }
    bool skip(uint64_t n) {
        if (!ok || off > size || size - off < n) { ok = false; return false; }
        off += n;
        return true;
    }
    // u64 length + bytes (gguf.rs:727-731)
    bool string(const char *&s, uint64_t &len) {
        len = pod<uint64_t>();
        if (!ok || size - off < len) { ok = false; return false; }
        s = reinterpret_cast<const char *>(base + off);
        off += len;
        return true;
    }
};

uint32_t scalar_size(int32_t t) {
    switch (t) {
    case MT_U8: case MT_I8: case MT_BOOL: return 1;
    case MT_U16: case MT_I16: return 2;
    case MT_U32: case MT_I32: case MT_F32: return 4;
    case MT_U64: case MT_I64: case MT_F64: return 8;
    default: return 0;
    }
}

bool skip_array(Cursor &c, int32_t elem_type, uint64_t count, int depth) {
    if (depth > 8) { c.ok = false; return false; }
    const uint32_t ss = scalar_size(elem_type);
    if (ss) {
        if (count > c.size) { c.ok = false; return false; }   // also guards count * ss against overflow
        return c.skip(count * ss);
    }
    if (elem_type == MT_STRING) {
        for (uint64_t i = 0; i < count && c.ok; i++) {
            const char *s; uint64_t n;
            c.string(s, n);
        }
        return c.ok;
    }
    if (elem_type == MT_ARRAY) {   // nested arrays: element type + length each (gguf.rs:502-510)
        for (uint64_t i = 0; i < count && c.ok; i++) {
            const int32_t et = (int32_t)c.pod<uint32_t>();
            const uint64_t n = c.pod<uint64_t>();
            if (!skip_array(c, et, n, depth + 1)) return false;
        }
        return c.ok;
    }
    c.ok = false;
    return false;
}

bool read_value(Cursor &c, int32_t type, MetaValue &v) {
    v.type = type;
    switch (type) {
    case MT_U8: v.u = c.pod<uint8_t>(); break;
    case MT_I8: v.u = (uint64_t)(int64_t)c.pod<int8_t>(); break;
    case MT_U16: v.u = c.pod<uint16_t>(); break;
    case MT_I16: v.u = (uint64_t)(int64_t)c.pod<int16_t>(); break;
    case MT_U32: v.u = c.pod<uint32_t>(); break;
    case MT_I32: v.u = (uint64_t)(int64_t)c.pod<int32_t>(); break;
    case MT_F32: v.f = c.pod<float>(); break;
    case MT_BOOL: v.u = c.pod<uint8_t>() != 0; break;
    case MT_U64: v.u = c.pod<uint64_t>(); break;
    case MT_I64: v.u = (uint64_t)c.pod<int64_t>(); break;
    case MT_F64: v.f = c.pod<double>(); break;
    case MT_STRING: c.string(v.str, v.str_len); break;
    case MT_ARRAY:
        v.elem_type = (int32_t)c.pod<uint32_t>();
        v.count = c.pod<uint64_t>();
        v.data_off = c.off;
        skip_array(c, v.elem_type, v.count, 0);
        break;
    default: c.ok = false;
    }
    if (type == MT_F32 || type == MT_F64) v.u = (uint64_t)(int64_t)v.f;
    else if (type != MT_STRING && type != MT_ARRAY) v.f = (type == MT_I8 || type == MT_I16 || type == MT_I32 || type == MT_I64) ? (double)(int64_t)v.u : (double)v.u;
    return c.ok;
}

int32_t parse(ib_gguf *g) {
    Cursor c{g->base, g->size};
    const uint32_t magic = c.pod<uint32_t>();
    if (!c.ok || magic != GGUF_MAGIC_LE) return set_error(IB_ERR_INVALID, "gguf: bad magic 0x%08x (expected 0x%08x)", magic, GGUF_MAGIC_LE);
    g->version = c.pod<uint32_t>();
    g->n_tensors = c.pod<uint64_t>();
    g->n_meta = c.pod<uint64_t>();
    if (!c.ok) return set_error(IB_ERR_INVALID, "gguf: truncated header");
    if (g->version < 2 || g->version > 3) return set_error(IB_ERR_UNSUPPORTED, "gguf: version %u (supported: 2, 3)", g->version);
    if (g->n_tensors > g->size || g->n_meta > g->size) return set_error(IB_ERR_INVALID, "gguf: implausible counts in the header");
    for (uint64_t i = 0; i < g->n_meta; i++) {
        const char *k; uint64_t kl;
        c.string(k, kl);
        const int32_t type = (int32_t)c.pod<uint32_t>();
        MetaValue v;
        if (!c.ok || !read_value(c, type, v))
            return set_error(IB_ERR_INVALID, "gguf: metadata entry %llu is truncated or has an unknown value type %d", (unsigned long long)i, type);
        std::string key(k, kl);
        if (!g->meta.count(key)) g->meta_keys.push_back(key);
        g->meta[key] = std::move(v);
    }
    // data alignment (gguf.rs:520-528)
    auto al = g->meta.find("general.alignment");
    if (al != g->meta.end() && al->second.type == MT_U32 && al->second.u > 0) g->alignment = (uint32_t)al->second.u;
    g->tensors.reserve((size_t)g->n_tensors);
    for (uint64_t i = 0; i < g->n_tensors; i++) {
        TensorRec t;
        const char *nm; uint64_t nl;
        c.string(nm, nl);
        t.n_dims = c.pod<uint32_t>();
        if (!c.ok || t.n_dims > 4) return set_error(IB_ERR_INVALID, "gguf: tensor %llu is truncated or has rank %u > 4", (unsigned long long)i, t.n_dims);
        uint64_t ne[4] = {1, 1, 1, 1};
        for (uint32_t d = 0; d < t.n_dims; d++) ne[d] = c.pod<uint64_t>();
        for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = ne[t.n_dims - 1 - d];   // stored fastest first; kept slowest first
        t.type = (int32_t)c.pod<uint32_t>();
        t.offset = c.pod<uint64_t>();   // relative to the data section for now
        if (!c.ok) return set_error(IB_ERR_INVALID, "gguf: tensor table truncated at entry %llu", (unsigned long long)i);
        t.name.assign(nm, nl);
        g->tensors.push_back(std::move(t));
    }
    g->data_start = (c.off + g->alignment - 1) / g->alignment * g->alignment;   // gguf.rs:609, 776-778
    for (size_t i = 0; i < g->tensors.size(); i++) {
        TensorRec &t = g->tensors[i];
        uint32_t bb, be;
        // element count: every factor and every running product is bounded by what the file could hold (a product of four
        // 64-bit dims can wrap even 128 bits; largest block length is 256, smallest block one byte)
        unsigned __int128 n = 1;
        const unsigned __int128 most = (unsigned __int128)g->size * 256u;
        for (int d = 0; d < 4; d++) {
            if (t.dims[d] == 0 || t.dims[d] > most) return set_error(IB_ERR_INVALID, "gguf: tensor %s has a dimension of %llu", t.name.c_str(), (unsigned long long)t.dims[d]);
            n *= t.dims[d];
            if (n > most) return set_error(IB_ERR_INVALID, "gguf: tensor %s is larger than the file", t.name.c_str());
        }
        if (type_size(t.type, bb, be)) {
            if (n % be) return set_error(IB_ERR_INVALID, "gguf: tensor %s has %llu elements, not a multiple of its block length %u", t.name.c_str(), (unsigned long long)n, be);
            const unsigned __int128 bytes = n / be * bb;
            if (bytes > g->size) return set_error(IB_ERR_INVALID, "gguf: tensor %s is larger than the file", t.name.c_str());
            t.nbytes = (uint64_t)bytes;
        }
        if (t.offset > g->size - (g->data_start < g->size ? g->data_start : g->size))
            return set_error(IB_ERR_INVALID, "gguf: tensor %s starts outside the file", t.name.c_str());
        t.offset += g->data_start;
        if (t.offset > g->size || g->size - t.offset < t.nbytes)
            return set_error(IB_ERR_INVALID, "gguf: tensor %s (%llu bytes at %llu) runs past the end of the file (%llu bytes)", t.name.c_str(),
                             (unsigned long long)t.nbytes, (unsigned long long)t.offset, (unsigned long long)g->size);
        g->by_name[t.name] = i;
    }
    return IB_OK;
}

void fill_info(const ib_gguf *g, const TensorRec &t, ib_gguf_tensor_info *info) {
    info->type = t.type;
    info->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) info->dims[d] = t.dims[d];
    info->offset = t.offset;
    info->nbytes = t.nbytes;
    info->data = g->base + t.offset;
}

const MetaValue *find_meta(const ib_gguf *g, const char *key) {
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

int32_t ib_gguf_open_memory(const void *bytes, uint64_t nbytes, ib_gguf **out) {
    IB_REQUIRE(bytes && out, "ib_gguf_open_memory: null argument");
    *out = nullptr;
    ib_gguf *g = new (std::nothrow) ib_gguf();
    if (!g) return set_error(IB_ERR_OOM, "host allocation failed");
    g->base = (const uint8_t *)bytes;
    g->size = nbytes;
    const int32_t rc = parse(g);
    if (rc != IB_OK) { delete g; return rc; }
    *out = g;
    return IB_OK;
}

int32_t ib_gguf_open(const char *path, ib_gguf **out) {
    IB_REQUIRE(path && out, "ib_gguf_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return set_error(IB_ERR_INVALID, "ib_gguf_open: cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        return set_error(IB_ERR_INVALID, "ib_gguf_open: %s is empty or cannot be examined", path);
    }
    void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);   // the mapping keeps the file
    if (map == MAP_FAILED) return set_error(IB_ERR_OOM, "ib_gguf_open: mmap of %s failed: %s", path, strerror(errno));
    ib_gguf *g = new (std::nothrow) ib_gguf();
    if (!g) { munmap(map, (size_t)st.st_size); return set_error(IB_ERR_OOM, "host allocation failed"); }
    g->base = (const uint8_t *)map;
    g->size = (uint64_t)st.st_size;
    g->mapped = true;
    const int32_t rc = parse(g);
    if (rc != IB_OK) { munmap(map, (size_t)st.st_size); delete g; return rc; }
    *out = g;
    return IB_OK;
}

int32_t ib_gguf_close(ib_gguf *g) {
    if (!g) return IB_OK;
    if (g->mapped) munmap((void *)g->base, (size_t)g->size);
    delete g;
    return IB_OK;
}

int32_t ib_gguf_counts(const ib_gguf *g, uint32_t *version, uint64_t *n_tensors, uint64_t *n_metadata, uint32_t *alignment) {
    IB_REQUIRE(g, "ib_gguf_counts: null file");
    if (version) *version = g->version;
    if (n_tensors) *n_tensors = g->tensors.size();
    if (n_metadata) *n_metadata = g->meta_keys.size();
    if (alignment) *alignment = g->alignment;
    return IB_OK;
}

int32_t ib_gguf_tensor_by_name(const ib_gguf *g, const char *name, ib_gguf_tensor_info *info) {
    IB_REQUIRE(g && name && info, "ib_gguf_tensor_by_name: null argument");
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return set_error(IB_ERR_INVALID, "gguf: no tensor named %s", name);
    fill_info(g, g->tensors[it->second], info);
    return IB_OK;
}

int32_t ib_gguf_tensor_by_index(const ib_gguf *g, uint64_t index, char *name_out, uint64_t name_cap, ib_gguf_tensor_info *info) {
    IB_REQUIRE(g && info, "ib_gguf_tensor_by_index: null argument");
    IB_REQUIRE(index < g->tensors.size(), "gguf: tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    const TensorRec &t = g->tensors[index];
    if (name_out && name_cap) {
        const size_t n = t.name.size() < name_cap - 1 ? t.name.size() : (size_t)name_cap - 1;
        memcpy(name_out, t.name.data(), n);
        name_out[n] = 0;
    }
    fill_info(g, t, info);
    return IB_OK;
}

int32_t ib_gguf_meta_key(const ib_gguf *g, uint64_t index, char *key_out, uint64_t key_cap, int32_t *type) {
    IB_REQUIRE(g && key_out && key_cap, "ib_gguf_meta_key: null argument");
    IB_REQUIRE(index < g->meta_keys.size(), "gguf: metadata index %llu of %zu", (unsigned long long)index, g->meta_keys.size());
    const std::string &k = g->meta_keys[index];
    const size_t n = k.size() < key_cap - 1 ? k.size() : (size_t)key_cap - 1;
    memcpy(key_out, k.data(), n);
    key_out[n] = 0;
    if (type) *type = g->meta.at(k).type;
    return IB_OK;
}

int32_t ib_gguf_meta_u64(const ib_gguf *g, const char *key, uint64_t *value) {
    IB_REQUIRE(g && key && value, "ib_gguf_meta_u64: null argument");
    const MetaValue *v = find_meta(g, key);
    if (!v) return set_error(IB_ERR_INVALID, "gguf: no metadata key %s", key);
    if (v->type == MT_STRING || v->type == MT_ARRAY) return set_error(IB_ERR_INVALID, "gguf: metadata %s is not a number", key);
    *value = v->u;
    return IB_OK;
}

int32_t ib_gguf_meta_f64(const ib_gguf *g, const char *key, double *value) {
    IB_REQUIRE(g && key && value, "ib_gguf_meta_f64: null argument");
    const MetaValue *v = find_meta(g, key);
    if (!v) return set_error(IB_ERR_INVALID, "gguf: no metadata key %s", key);
    if (v->type == MT_STRING || v->type == MT_ARRAY) return set_error(IB_ERR_INVALID, "gguf: metadata %s is not a number", key);
    *value = v->f;
    return IB_OK;
}

int32_t ib_gguf_meta_str(const ib_gguf *g, const char *key, char *out, uint64_t cap, uint64_t *len) {
    IB_REQUIRE(g && key, "ib_gguf_meta_str: null argument");
    const MetaValue *v = find_meta(g, key);
    if (!v) return set_error(IB_ERR_INVALID, "gguf: no metadata key %s", key);
    if (v->type != MT_STRING) return set_error(IB_ERR_INVALID, "gguf: metadata %s is not a string", key);
    if (len) *len = v->str_len;
    if (out && cap) {
        const uint64_t n = v->str_len < cap - 1 ? v->str_len : cap - 1;
        memcpy(out, v->str, n);
        out[n] = 0;
    }
    return IB_OK;
}

int32_t ib_gguf_meta_array(const ib_gguf *g, const char *key, int32_t *elem_type, uint64_t *count, const void **data) {
    IB_REQUIRE(g && key, "ib_gguf_meta_array: null argument");
    const MetaValue *v = find_meta(g, key);
    if (!v) return set_error(IB_ERR_INVALID, "gguf: no metadata key %s", key);
    if (v->type != MT_ARRAY) return set_error(IB_ERR_INVALID, "gguf: metadata %s is not an array", key);
    if (elem_type) *elem_type = v->elem_type;
    if (count) *count = v->count;
    if (data) *data = g->base + v->data_off;   // packed little-endian scalars; for strings use ib_gguf_meta_array_str
    return IB_OK;
}

int32_t ib_gguf_meta_array_str(ib_gguf *g, const char *key, uint64_t index, char *out, uint64_t cap, uint64_t *len) {
    IB_REQUIRE(g && key, "ib_gguf_meta_array_str: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return set_error(IB_ERR_INVALID, "gguf: no metadata key %s", key);
    MetaValue &v = it->second;
    if (v.type != MT_ARRAY || v.elem_type != MT_STRING) return set_error(IB_ERR_INVALID, "gguf: metadata %s is not an array of strings", key);
    IB_REQUIRE(index < v.count, "gguf: index %llu outside %s (%llu entries)", (unsigned long long)index, key, (unsigned long long)v.count);
    if (v.str_offsets.empty()) {   // one walk over the array, then indexed access
        v.str_offsets.reserve((size_t)v.count);
        Cursor c{g->base, g->size, v.data_off};
        for (uint64_t i = 0; i < v.count; i++) {
            v.str_offsets.push_back(c.off);
            const char *s; uint64_t n;
            c.string(s, n);
        }
    }
    Cursor c{g->base, g->size, v.str_offsets[(size_t)index]};
    const char *s; uint64_t n;
    c.string(s, n);
    if (len) *len = n;
    if (out && cap) {
        const uint64_t m = n < cap - 1 ? n : cap - 1;
        memcpy(out, s, m);
        out[m] = 0;
    }
    return IB_OK;
}

int32_t ib_gguf_llama_config(const ib_gguf *g, const char *arch, ib_llama_config *out) {
    IB_REQUIRE(g && out, "ib_gguf_llama_config: null argument");
    const std::string a = arch ? arch : "llama";
    auto need = [&](const std::string &key, uint32_t &dst) -> int32_t {
        const MetaValue *v = find_meta(g, key.c_str());
        if (!v || v->type == MT_STRING || v->type == MT_ARRAY) return set_error(IB_ERR_INVALID, "gguf: metadata key %s is missing or not a number", key.c_str());
        dst = (uint32_t)v->u;
        return IB_OK;
    };
    int32_t rc;
    if ((rc = need(a + ".embedding_length", out->hidden_size))) return rc;
    if ((rc = need(a + ".feed_forward_length", out->intermediate_size))) return rc;
    if ((rc = need(a + ".block_count", out->num_hidden_layers))) return rc;
    if ((rc = need(a + ".attention.head_count", out->num_attention_heads))) return rc;
    if ((rc = need(a + ".attention.head_count_kv", out->num_key_value_heads))) return rc;
    if ((rc = need(a + ".context_length", out->max_position_embeddings))) return rc;
    // vocabulary: length of tokenizer.ggml.tokens (cpu.rs:93); files without a tokenizer: rows of token_embd.weight
    const MetaValue *tok = find_meta(g, "tokenizer.ggml.tokens");
    if (tok && tok->type == MT_ARRAY) out->vocab_size = (uint32_t)tok->count;
    else {
        auto it = g->by_name.find("token_embd.weight");
        if (it == g->by_name.end()) return set_error(IB_ERR_INVALID, "gguf: neither tokenizer.ggml.tokens nor token_embd.weight gives the vocabulary size");
        out->vocab_size = (uint32_t)g->tensors[it->second].dims[0];
    }
    // defaults of cpu.rs:95-106
    const MetaValue *fb = find_meta(g, (a + ".rope.freq_base").c_str());
    out->rope_theta = (fb && fb->type != MT_STRING && fb->type != MT_ARRAY) ? (float)fb->f : 10000.0f;
    const MetaValue *eps = find_meta(g, (a + ".attention.layer_norm_rms_epsilon").c_str());
    out->rms_norm_eps = (eps && eps->type != MT_STRING && eps->type != MT_ARRAY) ? (float)eps->f : 1.0e-6f;
    // LlamaModelType::rope_variant (crates/inferi/src/models/llama2/mod.rs:24-29)
    out->rope_variant = a == "qwen2" ? IB_ROPE_NEOX : IB_ROPE_ORIGINAL;
    return IB_OK;
}

}  // extern "C"

// ---- GGUF -> device ----
namespace {

struct Loaded {
    std::vector<ib_qtensor *> tensors;
    std::vector<void *> device;
    void release() {
        for (ib_qtensor *t : tensors) ib_qtensor_destroy(t);
        for (void *p : device) cudaFree(p);
        tensors.clear();
        device.clear();
    }
};

// Uploads rows [r0, r1) x columns [c0, c1) of a quantized [rows, cols] matrix, padded with `pad_rows` all-zero rows and
// `pad_cols` columns of all-zero blocks (zero blocks dequantize to 0).  A pure row range goes up straight from the mapping.
int32_t upload_part(ib_ctx *ctx, const ib_gguf_tensor_info &ti, const char *name, uint64_t r0, uint64_t r1, uint64_t c0, uint64_t c1, uint64_t pad_rows,
                    uint64_t pad_cols, Loaded &keep, const ib_qtensor **out) {
    uint32_t bb, be;
    if (!type_size(ti.type, bb, be) || !(ti.type == IB_Q8_0 || ti.type == IB_Q4_K || ti.type == IB_Q5_K || ti.type == IB_Q6_K))
        return set_error(IB_ERR_UNSUPPORTED, "gguf: tensor %s has type %d; the fused kernels take Q8_0, Q4_K, Q5_K, Q6_K", name, ti.type);
    if (ti.n_dims != 2) return set_error(IB_ERR_INVALID, "gguf: tensor %s has rank %u, expected a matrix", name, ti.n_dims);
    const uint64_t rows = ti.dims[0], cols = ti.dims[1];
    if (r1 > rows || r0 >= r1 || c1 > cols || c0 >= c1 || c0 % be || c1 % be || pad_cols % be)
        return set_error(IB_ERR_INVALID, "gguf: slice [%llu,%llu) x [%llu,%llu) does not fit tensor %s (%llux%llu, block length %u)", (unsigned long long)r0,
                         (unsigned long long)r1, (unsigned long long)c0, (unsigned long long)c1, name, (unsigned long long)rows, (unsigned long long)cols, be);
    const uint64_t row_bytes = cols / be * bb;
    const uint8_t *src = (const uint8_t *)ti.data;
    ib_qtensor *qt = nullptr;
    int32_t rc;
    const uint64_t out_rows = r1 - r0 + pad_rows, out_cols = c1 - c0 + pad_cols;
    if (c0 == 0 && c1 == cols && pad_cols == 0 && pad_rows == 0) {
        rc = ib_qtensor_upload(ctx, ti.type, out_rows, out_cols, src + r0 * row_bytes, out_rows * row_bytes, 0, &qt);
    } else {
        const uint64_t out_row_bytes = out_cols / be * bb, part = (c1 - c0) / be * bb;
        std::vector<uint8_t> stage;
        try { stage.assign((size_t)(out_rows * out_row_bytes), 0); } catch (...) { return set_error(IB_ERR_OOM, "host staging of %s failed", name); }
        for (uint64_t r = r0; r < r1; r++) memcpy(stage.data() + (r - r0) * out_row_bytes, src + r * row_bytes + c0 / be * bb, (size_t)part);
        rc = ib_qtensor_upload(ctx, ti.type, out_rows, out_cols, stage.data(), stage.size(), 0, &qt);
    }
    if (rc != IB_OK) return rc;
    keep.tensors.push_back(qt);
    *out = qt;
    return IB_OK;
}

// Uploads elements [e0, e1) of an f32 vector of `n` values.
int32_t upload_f32(const ib_gguf *g, const char *name, uint64_t n, Loaded &keep, const float **out, uint64_t e0 = 0, uint64_t e1 = ~0ull) {
    ib_gguf_tensor_info ti;
    int32_t rc = ib_gguf_tensor_by_name(g, name, &ti);
    if (rc) return rc;
    if (ti.type != IB_F32 || ti.nbytes != n * 4) return set_error(IB_ERR_INVALID, "gguf: tensor %s must be %llu f32 values", name, (unsigned long long)n);
    if (e1 == ~0ull) e1 = n;
    if (e0 >= e1 || e1 > n) return set_error(IB_ERR_INVALID, "gguf: slice [%llu,%llu) of tensor %s", (unsigned long long)e0, (unsigned long long)e1, name);
    void *dev = nullptr;
    IB_CHECK_CUDA(cudaMalloc(&dev, (e1 - e0) * 4));
    keep.device.push_back(dev);
    IB_CHECK_CUDA(cudaMemcpy(dev, (const float *)ti.data + e0, (e1 - e0) * 4, cudaMemcpyHostToDevice));
    *out = (const float *)dev;
    return IB_OK;
}

}  // namespace

namespace ib {
// defined in llama.cu: the model frees these with itself
void llama_adopt(ib_llama *m, std::vector<ib_qtensor *> &&tensors, std::vector<void *> &&device);
}  // namespace ib

extern "C" int32_t ib_gguf_load_llama(ib_ctx *ctx, const ib_gguf *g, const char *arch, int32_t kv_dtype, uint32_t max_context, int32_t tp_rank, int32_t tp_size,
                                      ib_llama **out) {
    IB_REQUIRE(ctx && g && out, "ib_gguf_load_llama: null argument");
    *out = nullptr;
    IB_REQUIRE(cudaSetDevice(ctx->device) == cudaSuccess, "cudaSetDevice failed");
    IB_REQUIRE(tp_size >= 1 && tp_rank >= 0 && tp_rank < tp_size, "ib_gguf_load_llama: bad tensor-parallel rank %d of %d", tp_rank, tp_size);
    ib_llama_config c;
    int32_t rc = ib_gguf_llama_config(g, arch, &c);
    if (rc) return rc;
    if (max_context && max_context < c.max_position_embeddings) c.max_position_embeddings = max_context;
    IB_REQUIRE(c.num_attention_heads && c.num_key_value_heads && c.hidden_size % c.num_attention_heads == 0 && c.num_attention_heads % c.num_key_value_heads == 0,
               "gguf: head counts do not divide the hidden size");
    const uint64_t tp = (uint64_t)tp_size, rk = (uint64_t)tp_rank;
    IB_REQUIRE(c.num_key_value_heads % tp == 0 && c.vocab_size % (4 * tp) == 0 && c.intermediate_size % (256 * tp) == 0,
               "gguf: %d ranks do not divide the kv heads / vocabulary / FFN width of this model", tp_size);
    const uint64_t H = c.hidden_size, kv = (uint64_t)c.hidden_size * c.num_key_value_heads / c.num_attention_heads, F = c.intermediate_size, V = c.vocab_size;

    // `keep` goes to the model; `rotated` holds q / k matrices and biases of a NeoX model, which ib_llama_create copies in
    // its own row order and which are freed once it has
    Loaded keep, rotated;
    Loaded &qk = c.rope_variant == IB_ROPE_NEOX ? rotated : keep;
    std::vector<ib_llama_layer_weights> layers(c.num_hidden_layers);
    auto fail = [&](int32_t code) { keep.release(); rotated.release(); return code; };
    auto mat = [&](const std::string &name, ib_gguf_tensor_info &ti) { return ib_gguf_tensor_by_name(g, name.c_str(), &ti); };
    for (uint32_t l = 0; l < c.num_hidden_layers; l++) {
        const std::string p = "blk." + std::to_string(l) + ".";
        ib_llama_layer_weights &w = layers[l];
        ib_gguf_tensor_info ti;
        // rows of q / k / v (whole heads), gate / up (FFN units); columns of attn_output / ffn_down
        if ((rc = mat(p + "attn_q.weight", ti)) || (rc = upload_part(ctx, ti, "attn_q", rk * H / tp, (rk + 1) * H / tp, 0, ti.dims[1], 0, 0, qk, &w.attn_q))) return fail(rc);
        if ((rc = mat(p + "attn_k.weight", ti)) || (rc = upload_part(ctx, ti, "attn_k", rk * kv / tp, (rk + 1) * kv / tp, 0, ti.dims[1], 0, 0, qk, &w.attn_k))) return fail(rc);
        if ((rc = mat(p + "attn_v.weight", ti)) || (rc = upload_part(ctx, ti, "attn_v", rk * kv / tp, (rk + 1) * kv / tp, 0, ti.dims[1], 0, 0, keep, &w.attn_v))) return fail(rc);
        if ((rc = mat(p + "attn_output.weight", ti)) || (rc = upload_part(ctx, ti, "attn_output", 0, ti.dims[0], rk * H / tp, (rk + 1) * H / tp, 0, 0, keep, &w.attn_output)))
            return fail(rc);
        ib_gguf_tensor_info dn;
        if ((rc = mat(p + "ffn_down.weight", dn))) return fail(rc);
        // Q6_K rows can only be cut every 2048 columns (device layout): a rank's FFN slice is padded with zero blocks
        const uint64_t real = F / tp, unit = (tp > 1 && dn.type == IB_Q6_K) ? 2048 : 256, padded = tp > 1 ? (real + unit - 1) / unit * unit : real;
        const uint64_t f0 = rk * real, f1 = f0 + real, pad = padded - real;
        if ((rc = mat(p + "ffn_gate.weight", ti)) || (rc = upload_part(ctx, ti, "ffn_gate", f0, f1, 0, ti.dims[1], pad, 0, keep, &w.ffn_gate))) return fail(rc);
        if ((rc = mat(p + "ffn_up.weight", ti)) || (rc = upload_part(ctx, ti, "ffn_up", f0, f1, 0, ti.dims[1], pad, 0, keep, &w.ffn_up))) return fail(rc);
        if ((rc = upload_part(ctx, dn, "ffn_down", 0, dn.dims[0], f0, f1, 0, pad, keep, &w.ffn_down))) return fail(rc);
        if ((rc = upload_f32(g, (p + "attn_norm.weight").c_str(), H, keep, &w.attn_norm_dev))) return fail(rc);
        if ((rc = upload_f32(g, (p + "ffn_norm.weight").c_str(), H, keep, &w.ffn_norm_dev))) return fail(rc);
        // optional biases (transformer.rs:307-335), this rank's heads
        if (g->by_name.count(p + "attn_q.bias") && (rc = upload_f32(g, (p + "attn_q.bias").c_str(), H, qk, &w.attn_q_bias_dev, rk * H / tp, (rk + 1) * H / tp))) return fail(rc);
        if (g->by_name.count(p + "attn_k.bias") && (rc = upload_f32(g, (p + "attn_k.bias").c_str(), kv, qk, &w.attn_k_bias_dev, rk * kv / tp, (rk + 1) * kv / tp))) return fail(rc);
        if (g->by_name.count(p + "attn_v.bias") && (rc = upload_f32(g, (p + "attn_v.bias").c_str(), kv, keep, &w.attn_v_bias_dev, rk * kv / tp, (rk + 1) * kv / tp))) return fail(rc);
    }
    ib_llama_weights W{};
    W.layers = layers.data();
    ib_gguf_tensor_info te;
    if ((rc = ib_gguf_tensor_by_name(g, "token_embd.weight", &te))) return fail(rc);
    if (te.n_dims != 2 || te.dims[0] != V || te.dims[1] != H) return fail(set_error(IB_ERR_INVALID, "gguf: token_embd.weight is not [%llu, %llu]", (unsigned long long)V, (unsigned long long)H));
    if ((rc = upload_part(ctx, te, "token_embd", 0, V, 0, H, 0, 0, keep, &W.token_embd))) return fail(rc);
    // classifier: output.weight, else the embedding table (transformer.rs:376-382); a rank keeps its vocabulary slice
    ib_gguf_tensor_info ot = te;
    const bool tied = !g->by_name.count("output.weight");
    if (!tied && (rc = ib_gguf_tensor_by_name(g, "output.weight", &ot))) return fail(rc);
    if (tied && tp == 1) W.output = nullptr;   // ib_llama_create falls back to token_embd
    else if ((rc = upload_part(ctx, ot, "output", rk * V / tp, (rk + 1) * V / tp, 0, H, 0, 0, keep, &W.output))) return fail(rc);
    if ((rc = upload_f32(g, "output_norm.weight", H, keep, &W.output_norm_dev))) return fail(rc);

    ib_llama *m = nullptr;
    if ((rc = ib_llama_create(ctx, &c, &W, kv_dtype, tp_rank, tp_size, &m))) return fail(rc);
    rotated.release();
    llama_adopt(m, std::move(keep.tensors), std::move(keep.device));
    *out = m;
    return IB_OK;
}
