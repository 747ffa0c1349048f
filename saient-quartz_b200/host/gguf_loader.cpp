// GGUF reader + device loader (see gguf_loader.h).  File format as the reference reads it
// (src/gguf.rs:62-117): u32 magic "GGUF", u32 version (1..3), tensor count, kv count (u32 in v1, u64
// later), kv pairs (string key, u32 value type, value), tensor infos (string name, u32 n_dims, dims,
// u32 type, u64 offset), then the data section at the next multiple of general.alignment (32).
#include "gguf_loader.h"

#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/quartz_b200.h"

namespace {

thread_local std::string g_err;

enum ValueType : uint32_t {
    VT_U8 = 0, VT_I8, VT_U16, VT_I16, VT_U32, VT_I32, VT_F32, VT_BOOL, VT_STRING, VT_ARRAY, VT_U64, VT_I64, VT_F64
};

struct MetaValue {
    uint32_t type = 0;
    uint64_t bits = 0;          // scalar payload, little-endian as stored
    std::string str;            // VT_STRING
    uint32_t elem_type = 0;     // VT_ARRAY
    uint64_t count = 0;         // VT_ARRAY
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0, type = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0;
};

// bytes of n elements of a ggml type: the table of src/gguf.rs:172-191 plus the three formats this
// library adds (Q4_0, Q4_1, IQ3_XXS); 0 = unknown
uint64_t type_bytes(uint32_t t, uint64_t n)
{
    switch (t) {
    case 0: return n * 4;
    case 1: case 30: return n * 2;
    case 2: return n / 32 * 18;
    case 3: return n / 32 * 20;
    case 6: return n / 32 * 22;
    case 7: return n / 32 * 24;
    case 8: return n / 32 * 34;
    case 20: return n / 32 * 18;
    case 10: return n / 256 * 84;
    case 12: return n / 256 * 144;
    case 13: return n / 256 * 176;
    case 14: return n / 256 * 210;
    case 16: return n / 256 * 66;
    case 17: return n / 256 * 74;
    case 18: return n / 256 * 98;
    case 21: return n / 256 * 110;
    case 22: return n / 256 * 82;
    default: return 0;
    }
}

struct Cursor {
    const uint8_t *p;
    size_t size, pos = 0;
    bool ok = true;
    template <class T>
    T get()
    {
        T v{};
        if (!ok || pos + sizeof(T) > size) {
            ok = false;
            return v;
        }
        memcpy(&v, p + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    std::string str(bool v1)
    {
        const uint64_t n = v1 ? get<uint32_t>() : get<uint64_t>();
        if (!ok || n > size - pos) {
            ok = false;
            return {};
        }
        std::string s((const char *)p + pos, (size_t)n);
        pos += (size_t)n;
        return s;
    }
    void skip(uint64_t n)
    {
        if (!ok || n > size - pos) ok = false;
        else pos += (size_t)n;
    }
};

size_t scalar_size(uint32_t t)
{
    switch (t) {
    case VT_U8: case VT_I8: case VT_BOOL: return 1;
    case VT_U16: case VT_I16: return 2;
    case VT_U32: case VT_I32: case VT_F32: return 4;
    case VT_U64: case VT_I64: case VT_F64: return 8;
    default: return 0;
    }
}

bool read_value(Cursor &c, bool v1, MetaValue &out, int depth = 0)
{
    out.type = c.get<uint32_t>();
    if (!c.ok) return false;
    if (out.type == VT_STRING) {
        out.str = c.str(v1);
        return c.ok;
    }
    if (out.type == VT_ARRAY) {
        out.elem_type = c.get<uint32_t>();
        out.count = v1 ? c.get<uint32_t>() : c.get<uint64_t>();
        if (!c.ok) return false;
        if (const size_t es = scalar_size(out.elem_type)) {
            c.skip(out.count * es);
        } else if (out.elem_type == VT_STRING) {
            for (uint64_t i = 0; i < out.count && c.ok; i++) c.str(v1);   // token lists: walked, not kept
        } else if (out.elem_type == VT_ARRAY && depth < 4) {
            for (uint64_t i = 0; i < out.count && c.ok; i++) {
                MetaValue inner;
                // a nested array stores its own element type and count, without the leading value type
                inner.elem_type = c.get<uint32_t>();
                inner.count = v1 ? c.get<uint32_t>() : c.get<uint64_t>();
                const size_t es = scalar_size(inner.elem_type);
                if (!es) return false;
                c.skip(inner.count * es);
            }
        } else {
            return false;
        }
        return c.ok;
    }
    const size_t n = scalar_size(out.type);
    if (!n) return false;
    uint64_t bits = 0;
    if (c.pos + n > c.size) return false;
    memcpy(&bits, c.p + c.pos, n);
    c.pos += n;
    out.bits = bits;
    return true;
}

}  // namespace

struct qg_file {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;
    std::vector<Tensor> tensors;
    std::unordered_map<std::string, int> by_name;
    std::unordered_map<std::string, MetaValue> meta;
};

extern "C" {

const char *qg_last_error(void) { return g_err.c_str(); }

void qg_close(qg_file *f)
{
    if (!f) return;
    if (f->map) munmap((void *)f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

qg_file *qg_open(const char *path)
{
    g_err.clear();
    qg_file *f = new qg_file();
    auto fail = [&](const std::string &why) -> qg_file * {
        g_err = why;
        qg_close(f);
        return nullptr;
    };
    f->fd = open(path, O_RDONLY);
    if (f->fd < 0) return fail(std::string("cannot open ") + path);
    struct stat st;
    if (fstat(f->fd, &st) != 0 || st.st_size < 16) return fail("file too small to be GGUF");
    f->size = (size_t)st.st_size;
    void *m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) return fail("mmap failed");
    f->map = (const uint8_t *)m;

    Cursor c{f->map, f->size};
    if (c.get<uint32_t>() != 0x46554747u) return fail("not a GGUF file (bad magic)");
    f->version = c.get<uint32_t>();
    if (f->version < 1 || f->version > 3) return fail("unsupported GGUF version " + std::to_string(f->version));
    const bool v1 = f->version == 1;
    const uint64_t n_tensors = v1 ? c.get<uint32_t>() : c.get<uint64_t>();
    const uint64_t n_kv = v1 ? c.get<uint32_t>() : c.get<uint64_t>();
    if (!c.ok || n_tensors > (1u << 24) || n_kv > (1u << 24)) return fail("implausible header counts");
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key = c.str(v1);
        MetaValue v;
        if (!c.ok || !read_value(c, v1, v)) return fail("truncated or malformed metadata at key '" + key + "'");
        f->meta.emplace(std::move(key), std::move(v));
    }
    f->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        Tensor t;
        t.name = c.str(v1);
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims > 4) return fail("malformed tensor table");
        for (uint32_t d = 0; d < t.n_dims; d++) t.dims[d] = v1 ? c.get<uint32_t>() : c.get<uint64_t>();
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail("truncated tensor table");
        f->by_name.emplace(t.name, (int)f->tensors.size());
        f->tensors.push_back(std::move(t));
    }
    uint32_t align = 32;   // src/gguf.rs:107-108
    qg_meta_u32(f, "general.alignment", &align);
    if (align == 0) align = 32;
    f->data_offset = (c.pos + align - 1) / align * align;
    return f;
}

uint32_t qg_version(const qg_file *f) { return f ? f->version : 0; }
uint64_t qg_data_offset(const qg_file *f) { return f ? f->data_offset : 0; }
int qg_n_tensors(const qg_file *f) { return f ? (int)f->tensors.size() : 0; }

int qg_find_tensor(const qg_file *f, const char *name)
{
    if (!f || !name) return -1;
    auto it = f->by_name.find(name);
    return it == f->by_name.end() ? -1 : it->second;
}

static const Tensor *tensor_at(const qg_file *f, int i)
{
    return (f && i >= 0 && i < (int)f->tensors.size()) ? &f->tensors[(size_t)i] : nullptr;
}
const char *qg_tensor_name(const qg_file *f, int i) { const Tensor *t = tensor_at(f, i); return t ? t->name.c_str() : nullptr; }
uint32_t qg_tensor_type(const qg_file *f, int i) { const Tensor *t = tensor_at(f, i); return t ? t->type : 0xFFFFFFFFu; }
int qg_tensor_n_dims(const qg_file *f, int i) { const Tensor *t = tensor_at(f, i); return t ? (int)t->n_dims : 0; }
uint64_t qg_tensor_dim(const qg_file *f, int i, int d)
{
    const Tensor *t = tensor_at(f, i);
    return (t && d >= 0 && d < 4) ? t->dims[d] : 0;
}
uint64_t qg_tensor_bytes(const qg_file *f, int i)
{
    const Tensor *t = tensor_at(f, i);
    if (!t) return 0;
    uint64_t n = 1;
    for (uint32_t d = 0; d < t->n_dims; d++) n *= t->dims[d];
    return type_bytes(t->type, n);
}
const void *qg_tensor_data(const qg_file *f, int i)
{
    const Tensor *t = tensor_at(f, i);
    const uint64_t bytes = qg_tensor_bytes(f, i);
    if (!t || !bytes) return nullptr;
    const uint64_t start = f->data_offset + t->offset;
    if (start > f->size || bytes > f->size - start) return nullptr;   // the file is shorter than its table says
    return f->map + start;
}

static const MetaValue *meta_at(const qg_file *f, const char *key)
{
    if (!f || !key) return nullptr;
    auto it = f->meta.find(key);
    return it == f->meta.end() ? nullptr : &it->second;
}
int qg_meta_u32(const qg_file *f, const char *key, uint32_t *out)
{
    const MetaValue *v = meta_at(f, key);
    if (!v || (v->type != VT_U32 && v->type != VT_I32)) return 0;   // src/gguf.rs:19-25
    if (out) *out = (uint32_t)v->bits;
    return 1;
}
int qg_meta_u64(const qg_file *f, const char *key, uint64_t *out)
{
    const MetaValue *v = meta_at(f, key);
    if (!v || (v->type != VT_U64 && v->type != VT_U32)) return 0;   // src/gguf.rs:26-32
    if (out) *out = v->type == VT_U32 ? (uint32_t)v->bits : v->bits;
    return 1;
}
int qg_meta_f32(const qg_file *f, const char *key, float *out)
{
    const MetaValue *v = meta_at(f, key);
    if (!v || v->type != VT_F32) return 0;
    if (out) {
        const uint32_t b = (uint32_t)v->bits;
        memcpy(out, &b, 4);
    }
    return 1;
}
const char *qg_meta_str(const qg_file *f, const char *key)
{
    const MetaValue *v = meta_at(f, key);
    return (v && v->type == VT_STRING) ? v->str.c_str() : nullptr;
}
int qg_meta_bool(const qg_file *f, const char *key, int *out)
{
    const MetaValue *v = meta_at(f, key);
    if (!v || v->type != VT_BOOL) return 0;
    if (out) *out = (v->bits & 0xFF) != 0;
    return 1;
}
int qg_meta_array_len(const qg_file *f, const char *key, uint64_t *out)
{
    const MetaValue *v = meta_at(f, key);
    if (!v || v->type != VT_ARRAY) return 0;
    if (out) *out = v->count;
    return 1;
}

void *qg_upload_tensor(const qg_file *f, int i, int repack, int *repacked_out)
{
    if (repacked_out) *repacked_out = 0;
    const Tensor *t = tensor_at(f, i);
    const uint8_t *src = (const uint8_t *)qg_tensor_data(f, i);
    const uint64_t bytes = qg_tensor_bytes(f, i);
    if (!t || !src || !bytes) {
        g_err = "tensor missing, of unknown type, or outside the file";
        return nullptr;
    }
    uint8_t *dev = (uint8_t *)cuda_alloc((size_t)bytes);
    if (!dev) {
        g_err = "cuda_alloc failed";
        return nullptr;
    }
    // two page-locked staging buffers: while chunk k travels to the device, chunk k+1 is copied out of the mapping
    const size_t CHUNK = (size_t)16 << 20;
    static uint8_t *stage[2] = {nullptr, nullptr};
    if (!stage[0]) {
        stage[0] = (uint8_t *)cuda_host_alloc(CHUNK);
        stage[1] = (uint8_t *)cuda_host_alloc(CHUNK);
    }
    if (!stage[0] || !stage[1]) {
        cuda_h2d(dev, src, (size_t)bytes);   // no page-locked memory to be had: the reference's plain copy
    } else {
        int which = 0;
        for (uint64_t off = 0; off < bytes; off += CHUNK, which ^= 1) {
            const size_t n = (size_t)std::min<uint64_t>(CHUNK, bytes - off);
            // this buffer's previous transfer (two chunks ago) was waited for one iteration ago; the transfer
            // of the previous chunk, from the other buffer, runs while this chunk is copied out of the mapping
            memcpy(stage[which], src + off, n);
            if (off) cuda_sync();
            cuda_h2d_async(dev + off, stage[which], n);
        }
        cuda_sync();
    }
    if (repack && t->n_dims >= 2 && t->type != 0 && t->type != 1 && t->type != 30) {
        const int mats = t->n_dims >= 3 ? (int)t->dims[2] : 1;
        const int r = cuda_repack_weights(t->type, dev, (int)t->dims[0], (int)t->dims[1], mats);
        if (repacked_out) *repacked_out = r;
    }
    return dev;
}

}  // extern "C"
