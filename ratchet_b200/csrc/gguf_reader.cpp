// GGUF container reader and tensor loader (host side, no CUDA in this file).
//
// Follows the behaviour of the reference's loader, crates/ratchet-loader/src/gguf/gguf.rs:
//   VersionedMagic::read   (39-53)   magic "GGUF" in either byte order, versions 1..3
//   read_string            (165-180) u32 length in v1, u64 in v2/v3; trailing NULs dropped
//   Value::read            (343-383) thirteen value types, arrays nest
//   Header::read           (409-480) counts, metadata, tensor infos (dimensions REVERSED so the
//                                    outermost comes first), data offset rounded up to
//                                    general.alignment (default 32)
//   TensorInfo::read       (62-84)   numel must divide by the block size; bytes are read at
//                                    tensor_data_offset + offset
//   ratchet_from_gguf      (113-141) F32, F16 pass through; Q8_0 is transcoded to the split
//                                    layout (gguf/dtype.rs:44-110)
// Q4_K tensors load as the raw super-blocks (an extension: the reference rejects them).
// The file is read with plain buffered reads; the parser never trusts a length it has not
// checked against the file size, so a truncated or hostile file is an error, not a fault.
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "spec.hpp"

namespace rt {
Status transcode_gguf_q8_0(const uint8_t *blocks, uint64_t n_blocks, rt_dtype dt, uint8_t *out);
Status dtype_segments(rt_dtype dt, uint64_t numel, rt_segment *segs, int *n);
} // namespace rt

using rt::fail;
using rt::Status;

namespace {

constexpr uint64_t kDefaultAlignment = 32; // gguf.rs:13

struct Value {
    int32_t type = 0;
    int32_t elem_type = -1;
    uint64_t u64 = 0;
    int64_t i64 = 0;
    double f64 = 0.0;
    std::string str;
    std::vector<Value> items;
};

struct TensorRec {
    std::string name;
    uint32_t ggml_type = 0;
    rt_shape shape{};
    uint64_t offset = 0;
    uint64_t nbytes = 0;
    uint64_t numel = 0;
};

// block element count and byte size per ggml type id
// (crates/ratchet-loader/src/lib.rs:57-80,102-137; k_quants.rs:23-134)
bool ggml_block(uint32_t t, uint64_t *numel, uint64_t *bytes) {
    switch (t) {
    case 0: *numel = 1, *bytes = 4; return true;      // F32
    case 1: *numel = 1, *bytes = 2; return true;      // F16
    case 2: *numel = 32, *bytes = 18; return true;    // Q4_0
    case 3: *numel = 32, *bytes = 20; return true;    // Q4_1
    case 6: *numel = 32, *bytes = 22; return true;    // Q5_0
    case 7: *numel = 32, *bytes = 24; return true;    // Q5_1
    case 8: *numel = 32, *bytes = 34; return true;    // Q8_0
    case 9: *numel = 32, *bytes = 36; return true;    // Q8_1
    case 10: *numel = 256, *bytes = 84; return true;  // Q2K
    case 11: *numel = 256, *bytes = 110; return true; // Q3K
    case 12: *numel = 256, *bytes = 144; return true; // Q4K
    case 13: *numel = 256, *bytes = 176; return true; // Q5K
    case 14: *numel = 256, *bytes = 210; return true; // Q6K
    case 15: *numel = 256, *bytes = 292; return true; // Q8K
    default: return false;
    }
}

const char *ggml_name(uint32_t t) {
    static const char *names[16] = {"F32", "F16", "Q4_0", "Q4_1", "?", "?", "Q5_0", "Q5_1",
                                    "Q8_0", "Q8_1", "Q2K", "Q3K", "Q4K", "Q5K", "Q6K", "Q8K"};
    return t < 16 ? names[t] : "?";
}

struct Reader {
    FILE *f = nullptr;
    uint64_t size = 0, pos = 0;
    std::string err;

    bool take(void *dst, uint64_t n) {
        if (!err.empty()) return false;
        if (n > size - pos) {
            err = "unexpected end of file at byte " + std::to_string(pos) + " (wanted " + std::to_string(n) + " more)";
            return false;
        }
        if (n && std::fread(dst, 1, n, f) != n) {
            err = "read failed at byte " + std::to_string(pos);
            return false;
        }
        pos += n;
        return true;
    }
    template <typename T> T le() {
        // GGUF is little-endian and so is every host this library builds for
        T v{};
        take(&v, sizeof(T));
        return v;
    }
    uint64_t len(int version) { return version == 1 ? uint64_t(le<uint32_t>()) : le<uint64_t>(); }
    std::string string(int version) {
        uint64_t n = len(version);
        if (!err.empty()) return {};
        if (n > size - pos) {
            err = "string of " + std::to_string(n) + " bytes at byte " + std::to_string(pos) + " runs past the end of the file";
            return {};
        }
        std::string s(n, '\0');
        take(s.data(), n);
        while (!s.empty() && s.back() == '\0') s.pop_back(); // gguf.rs:174-177
        return s;
    }
};

bool read_value(Reader &r, int version, int32_t type, Value *v, int depth) {
    v->type = type;
    switch (type) {
    case RT_GGUF_U8: v->u64 = r.le<uint8_t>(); v->i64 = int64_t(v->u64); v->f64 = double(v->u64); break;
    case RT_GGUF_I8: v->i64 = r.le<int8_t>(); v->u64 = uint64_t(v->i64); v->f64 = double(v->i64); break;
    case RT_GGUF_U16: v->u64 = r.le<uint16_t>(); v->i64 = int64_t(v->u64); v->f64 = double(v->u64); break;
    case RT_GGUF_I16: v->i64 = r.le<int16_t>(); v->u64 = uint64_t(v->i64); v->f64 = double(v->i64); break;
    case RT_GGUF_U32: v->u64 = r.le<uint32_t>(); v->i64 = int64_t(v->u64); v->f64 = double(v->u64); break;
    case RT_GGUF_I32: v->i64 = r.le<int32_t>(); v->u64 = uint64_t(v->i64); v->f64 = double(v->i64); break;
    case RT_GGUF_U64: v->u64 = r.le<uint64_t>(); v->i64 = int64_t(v->u64); v->f64 = double(v->u64); break;
    case RT_GGUF_I64: v->i64 = r.le<int64_t>(); v->u64 = uint64_t(v->i64); v->f64 = double(v->i64); break;
    case RT_GGUF_F32: v->f64 = double(r.le<float>()); break;
    case RT_GGUF_F64: v->f64 = r.le<double>(); break;
    case RT_GGUF_BOOL: {
        uint8_t b = r.le<uint8_t>();
        if (r.err.empty() && b > 1) r.err = "unexpected bool value " + std::to_string(int(b)); // gguf.rs:359-363
        v->u64 = b, v->i64 = b, v->f64 = b;
        break;
    }
    case RT_GGUF_STRING: v->str = r.string(version); v->u64 = v->str.size(); break;
    case RT_GGUF_ARRAY: {
        if (depth > 8) {
            r.err = "arrays nest deeper than 8 levels";
            return false;
        }
        uint32_t et = r.le<uint32_t>();
        if (r.err.empty() && et > RT_GGUF_F64) r.err = "unrecognized value-type " + std::to_string(et); // gguf.rs:403
        uint64_t n = r.len(version);
        if (!r.err.empty()) return false;
        static const uint8_t fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};
        uint64_t lenb = version == 1 ? 4 : 8;
        uint64_t least = et == RT_GGUF_STRING ? lenb : et == RT_GGUF_ARRAY ? 4 + lenb : fixed[et];
        if (n > (r.size - r.pos) / least) { // the smallest encoding of n such elements
            r.err = "array of " + std::to_string(n) + " elements at byte " + std::to_string(r.pos) + " runs past the end of the file";
            return false;
        }
        v->elem_type = int32_t(et);
        v->u64 = n;
        v->items.resize(n);
        for (uint64_t i = 0; i < n; i++)
            if (!read_value(r, version, int32_t(et), &v->items[i], depth + 1)) return false;
        break;
    }
    default: r.err = "unrecognized value-type " + std::to_string(type); return false;
    }
    return r.err.empty();
}

void publish(const Value &v, rt_gguf_value *out) {
    out->type = v.type;
    out->elem_type = v.elem_type;
    out->len = (v.type == RT_GGUF_STRING || v.type == RT_GGUF_ARRAY) ? v.u64 : 1;
    out->u64 = v.u64;
    out->i64 = v.i64;
    out->f64 = v.f64;
    out->str = v.type == RT_GGUF_STRING ? v.str.c_str() : nullptr;
    out->node = &v;
}

} // namespace

struct rt_gguf {
    std::string path;
    FILE *f = nullptr;
    uint64_t file_size = 0;
    int version = 0;
    uint64_t alignment = kDefaultAlignment;
    uint64_t data_offset = 0;
    std::vector<std::pair<std::string, Value>> metadata; // file order; a later duplicate wins a lookup
    std::map<std::string, size_t> meta_index;
    std::vector<TensorRec> tensors;                      // file order
    std::map<std::string, size_t> tensor_index;
    ~rt_gguf() {
        if (f) std::fclose(f);
    }
};

namespace {

void publish(const TensorRec &t, rt_gguf_tensor_info *out) {
    out->name = t.name.c_str();
    out->ggml_type = t.ggml_type;
    out->shape = t.shape;
    out->offset = t.offset;
    out->nbytes = t.nbytes;
}

Status device_dtype(const TensorRec &t, rt_dtype *dt) {
    switch (t.ggml_type) {
    case 0: *dt = RT_F32; return Status::Ok();
    case 1: *dt = RT_F16; return Status::Ok();
    case 8: *dt = RT_Q8_0H; return Status::Ok(); // every sm_100 device has f16 (gguf.rs:130-136)
    case 12: *dt = RT_Q4_K; return Status::Ok(); // extension
    default: return Status::Err(RT_ERR_UNSUPPORTED, std::string("unsupported ggml dtype ") + ggml_name(t.ggml_type)); // gguf.rs:139
    }
}

// Whether tensor `t` can load as `dt`, and the bytes its device layout takes.
Status loadable(const TensorRec &t, rt_dtype dt, uint64_t *need) {
    rt_dtype natural;
    Status st = device_dtype(t, &natural);
    if (!st.ok()) return st;
    if (!(dt == natural || (t.ggml_type == 8 && dt == RT_Q8_0F)))
        return Status::Err(RT_ERR_DTYPE, std::string("a ") + ggml_name(t.ggml_type) + " tensor does not load as " + rt::dtype_name(dt));
    uint64_t block_numel, block_bytes;
    ggml_block(t.ggml_type, &block_numel, &block_bytes);
    if (t.numel % block_numel != 0) // gguf.rs:70-76
        return Status::Err(RT_ERR_SHAPE, "the number of elements " + std::to_string(t.numel) + " is not divisible by the block size " +
                                             std::to_string(block_numel));
    rt_segment seg[4];
    int nseg = 4;
    st = rt::dtype_segments(dt, t.numel, seg, &nseg);
    if (!st.ok()) return st;
    *need = 0;
    for (int i = 0; i < nseg; i++) *need = std::max<uint64_t>(*need, seg[i].offset + seg[i].size);
    return Status::Ok();
}

// Reads the tensor's bytes and writes the device layout of `dt` to `out`.
Status read_tensor(rt_gguf *g, const TensorRec &t, rt_dtype dt, uint8_t *out, uint64_t out_bytes) {
    uint64_t need = 0;
    Status st = loadable(t, dt, &need);
    if (!st.ok()) return st;
    bool q8 = t.ggml_type == 8;
    if (out_bytes < need)
        return Status::Err(RT_ERR_ARG, "output holds " + std::to_string(out_bytes) + " bytes, the tensor needs " + std::to_string(need));
    uint64_t start = g->data_offset + t.offset;
    if (start > g->file_size || t.nbytes > g->file_size - start)
        return Status::Err(RT_ERR_ARG, "tensor " + t.name + " (" + std::to_string(t.nbytes) + " bytes at " + std::to_string(start) +
                                           ") runs past the end of the file");
#if defined(_WIN32)
    if (_fseeki64(g->f, (long long)start, SEEK_SET) != 0)
#else
    if (fseeko(g->f, (off_t)start, SEEK_SET) != 0)
#endif
        return Status::Err(RT_ERR_ARG, "seek failed in " + g->path);
    if (!q8) {
        std::memset(out, 0, need); // the padding a short plain tensor carries (min 16 bytes)
        if (t.nbytes && std::fread(out, 1, t.nbytes, g->f) != t.nbytes) return Status::Err(RT_ERR_ARG, "read failed in " + g->path);
        return Status::Ok();
    }
    std::vector<uint8_t> raw(t.nbytes);
    if (t.nbytes && std::fread(raw.data(), 1, t.nbytes, g->f) != t.nbytes) return Status::Err(RT_ERR_ARG, "read failed in " + g->path);
    return rt::transcode_gguf_q8_0(raw.data(), t.numel / 32, dt, out);
}

} // namespace

extern "C" {

rt_status rt_gguf_open(const char *path, rt_gguf **out) {
    if (!path || !out) return fail(RT_ERR_ARG, "rt_gguf_open: null argument");
    *out = nullptr;
    std::unique_ptr<rt_gguf> g(new (std::nothrow) rt_gguf);
    if (!g) return fail(RT_ERR_NOMEM, "out of host memory");
    g->path = path;
    g->f = std::fopen(path, "rb");
    if (!g->f) return fail(RT_ERR_ARG, std::string("cannot open ") + path);
    std::fseek(g->f, 0, SEEK_END);
#if defined(_WIN32)
    g->file_size = uint64_t(_ftelli64(g->f));
#else
    g->file_size = uint64_t(ftello(g->f));
#endif
    std::fseek(g->f, 0, SEEK_SET);
    Reader r;
    r.f = g->f;
    r.size = g->file_size;
    auto bad = [&](const std::string &m) { return fail(RT_ERR_ARG, "gguf: " + m + " (" + g->path + ")"); };

    uint32_t magic = r.le<uint32_t>();
    if (!r.err.empty()) return bad(r.err);
    if (magic != 0x46554747u && magic != 0x47475546u) { // gguf.rs:23-26
        char buf[16];
        std::snprintf(buf, sizeof buf, "0x%08x", magic);
        return bad(std::string("unknown magic ") + buf);
    }
    uint32_t version = r.le<uint32_t>();
    if (!r.err.empty()) return bad(r.err);
    if (version < 1 || version > 3) return bad("unsupported magic/version Gguf/" + std::to_string(version)); // gguf.rs:49
    g->version = int(version);
    uint64_t n_tensors = r.len(g->version);
    uint64_t n_meta = r.len(g->version);
    if (!r.err.empty()) return bad(r.err);
    // a key takes at least 4+4 bytes and a tensor record at least 4+4+4+8
    if (n_meta > g->file_size / 8 || n_tensors > g->file_size / 20) return bad("counts exceed what the file can hold");

    g->metadata.reserve(n_meta);
    for (uint64_t i = 0; i < n_meta; i++) {
        std::string key = r.string(g->version);
        uint32_t vt = r.le<uint32_t>();
        if (!r.err.empty()) return bad(r.err);
        Value v;
        if (!read_value(r, g->version, int32_t(vt), &v, 0)) return bad(r.err);
        g->meta_index[key] = g->metadata.size();
        g->metadata.emplace_back(std::move(key), std::move(v));
    }
    g->tensors.reserve(n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        TensorRec t;
        t.name = r.string(g->version);
        uint32_t nd = r.le<uint32_t>();
        if (!r.err.empty()) return bad(r.err);
        if (nd > RT_MAX_RANK) return bad("tensor " + t.name + " has " + std::to_string(nd) + " dimensions");
        uint64_t dims[RT_MAX_RANK];
        for (uint32_t d = 0; d < nd; d++) dims[d] = r.len(g->version);
        t.shape.rank = int32_t(nd);
        t.numel = 1;
        for (uint32_t d = 0; d < nd; d++) { // gguf.rs:452: the file lists the innermost first
            uint64_t e = dims[nd - 1 - d];
            if (e > (uint64_t(1) << 40) || (e && t.numel > (uint64_t(1) << 62) / e)) return bad("tensor " + t.name + " is too large");
            t.shape.dims[d] = int64_t(e);
            t.numel *= e;
        }
        t.ggml_type = r.le<uint32_t>();
        t.offset = r.le<uint64_t>();
        if (!r.err.empty()) return bad(r.err);
        uint64_t bn, bb;
        if (!ggml_block(t.ggml_type, &bn, &bb)) return fail(RT_ERR_DTYPE, "gguf: invalid dtype " + std::to_string(t.ggml_type) + " for tensor " + t.name);
        t.nbytes = t.numel / bn * bb; // TensorInfo::size_in_bytes (gguf.rs:93-98)
        g->tensor_index[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    // gguf.rs:466-476: general.alignment of an integer type up to 32 bits, non-negative
    auto it = g->meta_index.find("general.alignment");
    if (it != g->meta_index.end()) {
        const Value &v = g->metadata[it->second].second;
        switch (v.type) {
        case RT_GGUF_U8: case RT_GGUF_U16: case RT_GGUF_U32: g->alignment = v.u64; break;
        case RT_GGUF_I8: case RT_GGUF_I16: case RT_GGUF_I32: if (v.i64 >= 0) g->alignment = uint64_t(v.i64); break;
        default: break;
        }
    }
    if (g->alignment == 0) return bad("general.alignment is 0");
    g->data_offset = (r.pos + g->alignment - 1) / g->alignment * g->alignment;
    *out = g.release();
    return RT_OK;
}

rt_status rt_gguf_close(rt_gguf *g) {
    delete g;
    return RT_OK;
}

int32_t rt_gguf_version(const rt_gguf *g) { return g ? g->version : 0; }
uint64_t rt_gguf_alignment(const rt_gguf *g) { return g ? g->alignment : 0; }
uint64_t rt_gguf_tensor_data_offset(const rt_gguf *g) { return g ? g->data_offset : 0; }
uint64_t rt_gguf_tensor_count(const rt_gguf *g) { return g ? g->tensors.size() : 0; }
uint64_t rt_gguf_metadata_count(const rt_gguf *g) { return g ? g->metadata.size() : 0; }

rt_status rt_gguf_metadata_at(const rt_gguf *g, uint64_t index, const char **key, rt_gguf_value *value) {
    if (!g || !key || !value) return fail(RT_ERR_ARG, "rt_gguf_metadata_at: null argument");
    if (index >= g->metadata.size()) return fail(RT_ERR_ARG, "rt_gguf_metadata_at: index out of range");
    *key = g->metadata[index].first.c_str();
    publish(g->metadata[index].second, value);
    return RT_OK;
}

rt_status rt_gguf_metadata_find(const rt_gguf *g, const char *key, rt_gguf_value *value) {
    if (!g || !key || !value) return fail(RT_ERR_ARG, "rt_gguf_metadata_find: null argument");
    auto it = g->meta_index.find(key);
    if (it == g->meta_index.end()) return fail(RT_ERR_ARG, std::string("missing key ") + key); // gguf.rs:149-153
    publish(g->metadata[it->second].second, value);
    return RT_OK;
}

rt_status rt_gguf_array_item(const rt_gguf_value *array, uint64_t index, rt_gguf_value *item) {
    if (!array || !item || !array->node) return fail(RT_ERR_ARG, "rt_gguf_array_item: null argument");
    const Value *v = static_cast<const Value *>(array->node);
    if (v->type != RT_GGUF_ARRAY) return fail(RT_ERR_ARG, "rt_gguf_array_item: not an array");
    if (index >= v->items.size()) return fail(RT_ERR_ARG, "rt_gguf_array_item: index out of range");
    publish(v->items[index], item);
    return RT_OK;
}

rt_status rt_gguf_tensor_at(const rt_gguf *g, uint64_t index, rt_gguf_tensor_info *info) {
    if (!g || !info) return fail(RT_ERR_ARG, "rt_gguf_tensor_at: null argument");
    if (index >= g->tensors.size()) return fail(RT_ERR_ARG, "rt_gguf_tensor_at: index out of range");
    publish(g->tensors[index], info);
    return RT_OK;
}

rt_status rt_gguf_tensor_find(const rt_gguf *g, const char *name, rt_gguf_tensor_info *info) {
    if (!g || !name || !info) return fail(RT_ERR_ARG, "rt_gguf_tensor_find: null argument");
    auto it = g->tensor_index.find(name);
    if (it == g->tensor_index.end()) return fail(RT_ERR_ARG, std::string("cannot find tensor info for ") + name); // gguf.rs:490-493
    publish(g->tensors[it->second], info);
    return RT_OK;
}

rt_status rt_gguf_tensor_dtype(const rt_gguf *g, const char *name, rt_dtype *dt) {
    if (!g || !name || !dt) return fail(RT_ERR_ARG, "rt_gguf_tensor_dtype: null argument");
    auto it = g->tensor_index.find(name);
    if (it == g->tensor_index.end()) return fail(RT_ERR_ARG, std::string("cannot find tensor info for ") + name);
    Status st = device_dtype(g->tensors[it->second], dt);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_gguf_tensor_nbytes(const rt_gguf *g, const char *name, rt_dtype dt, uint64_t *nbytes) {
    if (!g || !name || !nbytes) return fail(RT_ERR_ARG, "rt_gguf_tensor_nbytes: null argument");
    auto it = g->tensor_index.find(name);
    if (it == g->tensor_index.end()) return fail(RT_ERR_ARG, std::string("cannot find tensor info for ") + name);
    Status st = loadable(g->tensors[it->second], dt, nbytes);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_gguf_read_tensor(rt_gguf *g, const char *name, rt_dtype dt, void *out, uint64_t out_bytes) {
    if (!g || !name || !out) return fail(RT_ERR_ARG, "rt_gguf_read_tensor: null argument");
    auto it = g->tensor_index.find(name);
    if (it == g->tensor_index.end()) return fail(RT_ERR_ARG, std::string("cannot find tensor info for ") + name);
    Status st = read_tensor(g, g->tensors[it->second], dt, static_cast<uint8_t *>(out), out_bytes);
    return st.ok() ? RT_OK : fail(st);
}

rt_status rt_gguf_load_tensor(rt_gguf *g, rt_device *dev, const char *name, rt_dtype dt, rt_buffer **buf, rt_shape *shape) {
    if (!g || !dev || !name || !buf) return fail(RT_ERR_ARG, "rt_gguf_load_tensor: null argument");
    *buf = nullptr;
    auto it = g->tensor_index.find(name);
    if (it == g->tensor_index.end()) return fail(RT_ERR_ARG, std::string("cannot find tensor info for ") + name);
    const TensorRec &t = g->tensors[it->second];
    uint64_t nbytes = 0;
    Status ok = loadable(t, dt, &nbytes);
    if (!ok.ok()) return fail(ok);
    void *staging = nullptr;
    rt_status rc = rt_host_alloc(nbytes, &staging); // pinned, so the upload is one DMA
    if (rc != RT_OK) return rc;
    Status st = read_tensor(g, t, dt, static_cast<uint8_t *>(staging), nbytes);
    if (!st.ok()) {
        rt_host_free(staging);
        return fail(st);
    }
    rt_buffer *b = nullptr;
    rc = rt_buffer_alloc(dev, nbytes, &b);
    if (rc == RT_OK) rc = rt_upload(dev, b, 0, staging, nbytes, 1);
    std::string keep = rc == RT_OK ? std::string() : rt::last_error();
    rt_host_free(staging);
    if (rc != RT_OK) {
        if (b) rt_buffer_free(b);
        return fail(rc, keep);
    }
    if (shape) *shape = t.shape;
    *buf = b;
    return RT_OK;
}

} // extern "C"
