// GGUF container reader (host code only) behind the C-ABI of strix_gguf.h.
//
// Follows the reference's parser for what it accepts and what it refuses
// (crates/strix-models/src/gguf.rs:120-177, 288-378): little-endian, magic "GGUF", versions 2 and 3,
// u64 counts, length-prefixed strings, typed metadata values (0..12, arrays of non-array elements),
// tensor infos (name, n_dims, dims u64[], ggml_type u32, offset u64), tensor data from the next
// multiple of general.alignment (default 32) after the header. Every read is bounds-checked; a short
// file is "unexpected EOF", never a read past the map.
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "strix_gguf.h"

namespace {

thread_local std::string g_err;

struct Meta {
    uint32_t type = 0;       // GGUF value type 0..12
    uint64_t u = 0;          // integers (sign-extended into i for signed kinds), bool
    int64_t i = 0;
    double f = 0.0;          // F32 / F64
    std::string s;           // STRING
    uint32_t elem_type = 0;  // ARRAY: element type and count (elements are skipped over, not kept:
    uint64_t count = 0;      // the matmul path needs no tokenizer tables)
};

struct Tensor {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0;
    uint64_t numel = 1;
};

size_t block_elems(uint32_t t) {
    switch (t) {
        case 0: case 1: return 1;
        case 2: case 3: case 6: case 7: case 8: case 9: return 32;
        case 10: case 11: case 12: case 13: case 14: case 15: return 256;
        default: return 0;
    }
}
size_t block_bytes(uint32_t t) {
    switch (t) {
        case 0: return 4;
        case 1: return 2;
        case 2: return 18;
        case 3: return 20;
        case 6: return 22;
        case 7: return 24;
        case 8: return 34;
        case 9: return 36;
        case 10: return 84;
        case 11: return 110;
        case 12: return 144;
        case 13: return 176;
        case 14: return 210;
        case 15: return 292;
        default: return 0;
    }
}

// Little-endian cursor with bounds checking (gguf.rs:280-327).
struct Cursor {
    const uint8_t *buf;
    size_t len, pos = 0;
    bool ok = true;
    const uint8_t *take(size_t n) {
        if (!ok || n > len - pos) {
            ok = false;
            return nullptr;
        }
        const uint8_t *p = buf + pos;
        pos += n;
        return p;
    }
    template <typename T>
    T rd() {
        T v{};
        if (const uint8_t *p = take(sizeof(T))) memcpy(&v, p, sizeof(T));
        return v;
    }
    std::string str() {
        const uint64_t n = rd<uint64_t>();
        if (!ok || n > len - pos) {
            ok = false;
            return std::string();
        }
        const uint8_t *p = take((size_t)n);
        return p ? std::string(reinterpret_cast<const char *>(p), (size_t)n) : std::string();
    }
};

size_t scalar_size(uint32_t ty) {
    switch (ty) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

// One metadata value of type ty (gguf.rs:335-377). false = error (g_err set, or c.ok false = EOF).
bool read_value(Cursor &c, uint32_t ty, Meta &m, bool keep) {
    m.type = ty;
    switch (ty) {
        case 0: m.u = c.rd<uint8_t>(); m.i = (int64_t)m.u; break;
        case 1: m.i = c.rd<int8_t>(); m.u = (uint64_t)m.i; break;
        case 2: m.u = c.rd<uint16_t>(); m.i = (int64_t)m.u; break;
        case 3: m.i = c.rd<int16_t>(); m.u = (uint64_t)m.i; break;
        case 4: m.u = c.rd<uint32_t>(); m.i = (int64_t)m.u; break;
        case 5: m.i = c.rd<int32_t>(); m.u = (uint64_t)m.i; break;
        case 6: m.f = c.rd<float>(); break;
        case 7: m.u = c.rd<uint8_t>() != 0; m.i = (int64_t)m.u; break;
        case 8:
            if (keep) m.s = c.str();
            else (void)c.str();
            break;
        case 9: {
            m.elem_type = c.rd<uint32_t>();
            m.count = c.rd<uint64_t>();
            if (!c.ok) return false;
            if (m.elem_type == 9) {
                g_err = "GGUF nested arrays";
                return false;
            }
            if (const size_t sz = scalar_size(m.elem_type)) {
                if (m.count > (c.len - c.pos) / sz) c.ok = false;
                else c.pos += (size_t)m.count * sz;
            } else if (m.elem_type == 8) {
                for (uint64_t k = 0; k < m.count && c.ok; k++) (void)c.str();
            } else {
                g_err = "GGUF metadata value type " + std::to_string(m.elem_type);
                return false;
            }
            break;
        }
        case 10: m.u = c.rd<uint64_t>(); m.i = (int64_t)m.u; break;
        case 11: m.i = c.rd<int64_t>(); m.u = (uint64_t)m.i; break;
        case 12: m.f = c.rd<double>(); break;
        default:
            g_err = "GGUF metadata value type " + std::to_string(ty);
            return false;
    }
    return c.ok;
}

}  // namespace

struct strix_gguf {
    const uint8_t *base = nullptr;
    size_t len = 0;
    bool mapped = false;  // base is our mmap (else borrowed memory)
    uint32_t version = 0;
    size_t alignment = 32, data_offset = 0;
    std::vector<std::string> meta_keys;  // file order
    std::unordered_map<std::string, Meta> meta;
    std::vector<Tensor> tensors;  // file order
    std::unordered_map<std::string, size_t> by_name;
};

namespace {

int parse(strix_gguf *g) {
    Cursor c{g->base, g->len};
    const uint32_t magic = c.rd<uint32_t>();
    if (!c.ok || magic != 0x46554747u) {
        char b[64];
        snprintf(b, sizeof b, "not a GGUF file (magic 0x%08x)", c.ok ? magic : 0u);
        g_err = b;
        return -1;
    }
    g->version = c.rd<uint32_t>();
    if (!c.ok || (g->version != 2 && g->version != 3)) {
        g_err = "GGUF version " + std::to_string(g->version);
        return -1;
    }
    const uint64_t tensor_count = c.rd<uint64_t>(), kv_count = c.rd<uint64_t>();
    if (!c.ok) {
        g_err = "GGUF: unexpected EOF";
        return -1;
    }
    for (uint64_t k = 0; k < kv_count; k++) {
        std::string key = c.str();
        const uint32_t ty = c.rd<uint32_t>();
        Meta m;
        g_err.clear();
        if (!c.ok || !read_value(c, ty, m, true)) {
            if (g_err.empty()) g_err = "GGUF: unexpected EOF";
            return -1;
        }
        if (!g->meta.count(key)) g->meta_keys.push_back(key);
        g->meta[key] = std::move(m);  // a repeated key: the last one wins, as with HashMap::insert
    }
    for (uint64_t k = 0; k < tensor_count; k++) {
        Tensor t;
        t.name = c.str();
        t.n_dims = c.rd<uint32_t>();
        if (!c.ok) break;
        if (t.n_dims > 4) {
            // (the reference accepts any count, gguf.rs:145-149; no GGUF writer emits more than four, and four is what
            // strix_gguf_tensor carries: a deliberate difference)
            g_err = "GGUF tensor `" + t.name + "`: " + std::to_string(t.n_dims) + " dimensions";
            return -1;
        }
        for (uint32_t d = 0; d < t.n_dims; d++) {
            t.dims[d] = c.rd<uint64_t>();
            // sizes in a file are untrusted: a product that wraps would let dims and byte count disagree
            if (__builtin_mul_overflow(t.numel, t.dims[d], &t.numel)) {
                g_err = "GGUF tensor `" + t.name + "`: element count overflows 64 bits";
                return -1;
            }
        }
        t.type = c.rd<uint32_t>();
        t.offset = c.rd<uint64_t>();
        if (!c.ok) break;
        if (block_elems(t.type) == 0) {
            g_err = "GGML type id " + std::to_string(t.type) + " unrecognized (IQ/TQ types not handled)";
            return -1;
        }
        g->by_name[t.name] = g->tensors.size();  // a repeated name: the last one wins
        g->tensors.push_back(std::move(t));
    }
    if (!c.ok) {
        g_err = "GGUF: unexpected EOF";
        return -1;
    }
    // general.alignment with the reference's widening (any non-negative integer kind)
    auto it = g->meta.find("general.alignment");
    if (it != g->meta.end()) {
        const Meta &m = it->second;
        const bool is_int = m.type <= 5 || m.type == 10 || m.type == 11;
        if (is_int && m.i >= 0) g->alignment = (size_t)m.u;
    }
    size_t padded = c.pos;
    if (g->alignment) {
        if (__builtin_add_overflow(c.pos, g->alignment - 1, &padded)) {
            g_err = "GGUF: general.alignment " + std::to_string(g->alignment) + " overflows the data offset";
            return -1;
        }
        padded = padded / g->alignment * g->alignment;
    }
    g->data_offset = padded;
    if (g->data_offset > g->len) {
        g_err = "GGUF tensor data offset past EOF";
        return -1;
    }
    return 1;
}

int fill(const strix_gguf *g, size_t i, strix_gguf_tensor *out) {
    const Tensor &t = g->tensors[i];
    if (t.numel % block_elems(t.type) != 0) {
        g_err = "tensor `" + t.name + "`: " + std::to_string(t.numel) + " elements are not whole blocks of " +
                std::to_string(block_elems(t.type));
        return -1;
    }
    uint64_t nbytes64 = 0, start = 0;
    if (__builtin_mul_overflow((uint64_t)(t.numel / block_elems(t.type)), (uint64_t)block_bytes(t.type), &nbytes64) ||
        __builtin_add_overflow((uint64_t)g->data_offset, t.offset, &start)) {
        g_err = "tensor `" + t.name + "`: size or offset overflows 64 bits";
        return -1;
    }
    const size_t nbytes = (size_t)nbytes64;
    if (start > g->len || nbytes > g->len - start) {
        g_err = "tensor `" + t.name + "` data [" + std::to_string(start) + ".." + std::to_string(start + nbytes) +
                "] past EOF " + std::to_string(g->len);
        return -1;
    }
    out->name = t.name.c_str();
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; d++) out->dims[d] = t.dims[d];
    out->ggml_type = t.type;
    out->offset = t.offset;
    out->data = g->base + start;
    out->nbytes = nbytes;
    return 1;
}

const Meta *find_meta(const strix_gguf *g, const char *key) {
    if (!g || !key) return nullptr;
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}

}  // namespace

extern "C" {

const char *strix_gguf_last_error(void) { return g_err.c_str(); }

int strix_gguf_open_memory(const uint8_t *bytes, size_t len, strix_gguf **out) {
    if (!bytes || !out) return -1;
    *out = nullptr;
    strix_gguf *g = new strix_gguf();
    g->base = bytes;
    g->len = len;
    if (parse(g) < 0) {
        delete g;
        return -1;
    }
    *out = g;
    return 1;
}

int strix_gguf_open(const char *path, strix_gguf **out) {
    if (!path || !out) return -1;
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) {
        g_err = std::string("open ") + path + ": " + strerror(errno);
        return -1;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        g_err = std::string(path) + ": empty or unreadable";
        close(fd);
        return -1;
    }
    void *p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) {
        g_err = std::string("mmap ") + path + ": " + strerror(errno);
        return -1;
    }
    strix_gguf *g = new strix_gguf();
    g->base = static_cast<const uint8_t *>(p);
    g->len = (size_t)st.st_size;
    g->mapped = true;
    if (parse(g) < 0) {
        strix_gguf_close(g);
        return -1;
    }
    *out = g;
    return 1;
}

void strix_gguf_close(strix_gguf *g) {
    if (!g) return;
    if (g->mapped && g->base) munmap(const_cast<uint8_t *>(g->base), g->len);
    delete g;
}

uint32_t strix_gguf_version(const strix_gguf *g) { return g ? g->version : 0; }
size_t strix_gguf_alignment(const strix_gguf *g) { return g ? g->alignment : 0; }
size_t strix_gguf_data_offset(const strix_gguf *g) { return g ? g->data_offset : 0; }
size_t strix_gguf_tensor_count(const strix_gguf *g) { return g ? g->tensors.size() : 0; }
size_t strix_gguf_meta_count(const strix_gguf *g) { return g ? g->meta_keys.size() : 0; }
size_t strix_ggml_block_elems(uint32_t t) { return block_elems(t); }
size_t strix_ggml_block_bytes(uint32_t t) { return block_bytes(t); }

int strix_gguf_tensor_at(const strix_gguf *g, size_t i, strix_gguf_tensor *out) {
    if (!g || !out) return -1;
    if (i >= g->tensors.size()) return 0;
    return fill(g, i, out);
}

int strix_gguf_find_tensor(const strix_gguf *g, const char *name, strix_gguf_tensor *out) {
    if (!g || !name || !out) return -1;
    auto it = g->by_name.find(name);
    if (it == g->by_name.end()) return 0;
    return fill(g, it->second, out);
}

}  // extern "C"

extern "C" {

// MetaValue::as_u64 (gguf.rs:43-56): unsigned kinds, and signed kinds when non-negative
int strix_gguf_meta_u64(const strix_gguf *g, const char *key, uint64_t *out) {
    const Meta *m = find_meta(g, key);
    if (!m || !out) return 0;
    switch (m->type) {
        case 0: case 2: case 4: case 10: *out = m->u; return 1;
        case 1: case 3: case 5: case 11:
            if (m->i < 0) return 0;
            *out = (uint64_t)m->i;
            return 1;
        default: return 0;
    }
}

// MetaValue::as_f32 (gguf.rs:59-65): f32, f64 narrowed, or an integer as_u64 accepts
int strix_gguf_meta_f32(const strix_gguf *g, const char *key, float *out) {
    const Meta *m = find_meta(g, key);
    if (!m || !out) return 0;
    if (m->type == 6 || m->type == 12) {
        *out = (float)m->f;
        return 1;
    }
    uint64_t u;
    if (strix_gguf_meta_u64(g, key, &u) != 1) return 0;
    *out = (float)u;
    return 1;
}

int strix_gguf_meta_str(const strix_gguf *g, const char *key, const char **out, size_t *len) {
    const Meta *m = find_meta(g, key);
    if (!m || !out || m->type != 8) return 0;
    *out = m->s.c_str();
    if (len) *len = m->s.size();
    return 1;
}

int strix_gguf_meta_array_len(const strix_gguf *g, const char *key, uint64_t *len, uint32_t *elem_type) {
    const Meta *m = find_meta(g, key);
    if (!m || m->type != 9) return 0;
    if (len) *len = m->count;
    if (elem_type) *elem_type = m->elem_type;
    return 1;
}

int strix_gguf_meta_key_at(const strix_gguf *g, size_t i, const char **key, uint32_t *value_type) {
    if (!g || !key) return -1;
    if (i >= g->meta_keys.size()) return 0;
    *key = g->meta_keys[i].c_str();
    if (value_type) *value_type = g->meta.at(g->meta_keys[i]).type;
    return 1;
}

void strix_gguf_advise_dontneed(const strix_gguf *g, const char *name) {
    strix_gguf_tensor t;
    if (!g || !g->mapped || strix_gguf_find_tensor(g, name, &t) != 1) return;
    const size_t page = 4096, start = (size_t)(t.data - g->base);
    const size_t a = (start + page - 1) / page * page;   // first whole page inside the tensor
    const size_t b = (start + t.nbytes) / page * page;   // last whole-page boundary
    if (b > a && b <= g->len) (void)madvise(const_cast<uint8_t *>(g->base) + a, b - a, MADV_DONTNEED);
}

int strix_cuda_upload_gguf_tensor(strix_cuda *h, const strix_gguf *g, const char *name, int drop_pages) {
    if (!h || !g || !name) return -1;
    strix_gguf_tensor t;
    const int f = strix_gguf_find_tensor(g, name, &t);
    if (f != 1) {
        if (f == 0) g_err = std::string("GGUF tensor `") + name + "` not found";
        return f == 0 ? -1 : f;
    }
    int rc = 0;
    if (t.n_dims == 2) {
        const size_t in_dim = (size_t)t.dims[0], out_dim = (size_t)t.dims[1];  // qwen3.rs:772-774
        switch (t.ggml_type) {
            case STRIX_GGML_Q4_0: rc = strix_cuda_upload_q4_0(h, name, t.data, t.nbytes, in_dim, out_dim); break;
            case STRIX_GGML_Q4_1: rc = strix_cuda_upload_q4_1(h, name, t.data, t.nbytes, in_dim, out_dim); break;
            case STRIX_GGML_Q8_0: rc = strix_cuda_upload_q8_0(h, name, t.data, t.nbytes, in_dim, out_dim); break;
            case STRIX_GGML_Q6_K: rc = strix_cuda_upload_q6_k(h, name, t.data, t.nbytes, in_dim, out_dim); break;
            default: rc = 0; break;  // no kernel for this format: the weight stays with the CPU path
        }
    } else if (t.n_dims == 1 && t.ggml_type == STRIX_GGML_F32) {
        // (a file with general.alignment below 4 can leave the vector on an odd address: it is declined, not cast)
        if (reinterpret_cast<uintptr_t>(t.data) % alignof(float) == 0)
            rc = strix_cuda_upload_f32(h, name, reinterpret_cast<const float *>(t.data), (size_t)t.dims[0]);
    }
    if (rc == 1 && drop_pages) strix_gguf_advise_dontneed(g, name);
    return rc;
}

int strix_cuda_upload_gguf(strix_cuda *h, const strix_gguf *g, int drop_pages, size_t *adopted, size_t *declined) {
    if (!h || !g) return -1;
    size_t a = 0, d = 0;
    for (const Tensor &t : g->tensors) {
        const int rc = strix_cuda_upload_gguf_tensor(h, g, t.name.c_str(), drop_pages);
        if (rc < 0) return rc;
        (rc == 1 ? a : d)++;
    }
    if (adopted) *adopted = a;
    if (declined) *declined = d;
    return 1;
}

}  // extern "C"
