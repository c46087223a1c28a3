// GGUF reader and transcoder (host code; no kernels).
//
// Stands in for ratchet-loader's GGUF path: the header / metadata / tensor-info parser
// (ratchet-loader/src/gguf/gguf.rs:422-509: versions 1-3, dimensions stored innermost first and reversed
// on load, tensor data starting at the next multiple of `general.alignment`, default 32) and the
// transcode from ggml's interleaved blocks to ratchet's segment layout
// (ratchet-loader/src/gguf/dtype.rs:39-198):
//   Q8_0  block {f16 d; i8 qs[32]}                      -> [qs ...][d ... as f16 (Q8_0H) or f32 (Q8_0F)]
//   Q4_K  block {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} -> [qs][scales][dmin][d], d/dmin as f16 or f32
//   F32 / F16                                            -> copied
// each segment padded to 256 bytes, which is the layout every kernel of this library reads.  The file
// is memory-mapped; transcoding writes into a caller-provided host buffer that is then uploaded with
// rcu_h2d, as `Tensor::from_quantized` does.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

thread_local char g_gguf_error[512] = "";

rcu_status gguf_fail(rcu_status st, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_gguf_error, sizeof(g_gguf_error), fmt, ap);
    va_end(ap);
    return st;
}

enum GgmlType { GGML_F32 = 0, GGML_F16 = 1, GGML_Q8_0 = 8, GGML_Q4_K = 12 };

struct TensorInfo {
    std::string name;
    uint32_t rank = 0;
    uint64_t shape[4] = {1, 1, 1, 1};   // ratchet order: outermost first
    uint32_t ggml_type = 0;
    uint64_t offset = 0;                // relative to the data section
    uint64_t numel = 1;
    uint64_t file_bytes = 0;
};

struct MetaValue {
    uint32_t type = 0;
    uint64_t u = 0;        // integers and bool
    double f = 0.0;        // floats
    std::string s;         // strings
    uint64_t array_len = 0;
};

// cursor over the mapped file with bounds checks
struct Cursor {
    const uint8_t* base;
    uint64_t size, pos;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (pos > size || sizeof(T) > size - pos) { ok = false; return v; }     // lengths come from the file: no sum that can wrap
        memcpy(&v, base + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    uint64_t len(int version) { return version == 1 ? get<uint32_t>() : get<uint64_t>(); }
    std::string str(int version) {
        const uint64_t n = len(version);
        if (!ok || pos > size || n > size - pos) { ok = false; return {}; }
        std::string s((const char*)base + pos, (size_t)n);
        pos += n;
        while (version == 1 && !s.empty() && s.back() == '\0') s.pop_back();   // v1 strings carry their terminator
        return s;
    }
};

size_t value_size(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

bool read_value(Cursor& c, int version, uint32_t type, MetaValue* out, int depth = 0) {
    out->type = type;
    switch (type) {
        case 0: out->u = c.get<uint8_t>(); break;
        case 1: out->u = (uint64_t)(int64_t)c.get<int8_t>(); break;
        case 2: out->u = c.get<uint16_t>(); break;
        case 3: out->u = (uint64_t)(int64_t)c.get<int16_t>(); break;
        case 4: out->u = c.get<uint32_t>(); break;
        case 5: out->u = (uint64_t)(int64_t)c.get<int32_t>(); break;
        case 6: out->f = c.get<float>(); break;
        case 7: out->u = c.get<uint8_t>() != 0; break;
        case 8: out->s = c.str(version); break;
        case 9: {
            if (depth > 4) return false;
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = c.len(version);
            out->array_len = n;
            if (et == 8) {
                for (uint64_t i = 0; i < n && c.ok; ++i) c.str(version);
            } else if (et == 9) {
                MetaValue tmp;
                for (uint64_t i = 0; i < n && c.ok; ++i)
                    if (!read_value(c, version, 9, &tmp, depth + 1)) return false;
            } else {
                const size_t es = value_size(et);
                uint64_t bytes = 0;
                if (es == 0 || __builtin_mul_overflow(n, (uint64_t)es, &bytes) || c.pos > c.size || bytes > c.size - c.pos) return false;
                c.pos += bytes;
            }
            break;
        }
        case 10: out->u = c.get<uint64_t>(); break;
        case 11: out->u = (uint64_t)c.get<int64_t>(); break;
        case 12: out->f = c.get<double>(); break;
        default: return false;
    }
    return c.ok;
}

bool block_layout(uint32_t ggml_type, uint64_t* block_numel, uint64_t* type_size) {
    switch (ggml_type) {
        case GGML_F32: *block_numel = 1; *type_size = 4; return true;
        case GGML_F16: *block_numel = 1; *type_size = 2; return true;
        case GGML_Q8_0: *block_numel = 32; *type_size = 34; return true;
        case GGML_Q4_K: *block_numel = 256; *type_size = 144; return true;
        default: return false;
    }
}

float f16_bits_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

struct rcu_gguf {
    int fd = -1;
    const uint8_t* map = nullptr;
    uint64_t size = 0;
    int version = 0;
    uint64_t data_offset = 0;
    std::vector<TensorInfo> tensors;
    std::map<std::string, size_t> by_name;
    std::map<std::string, MetaValue> meta;
};

extern "C" {

const char* rcu_gguf_last_error(void) { return g_gguf_error; }

void rcu_gguf_close(rcu_gguf* g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

rcu_status rcu_gguf_open(const char* path, rcu_gguf** out) {
    if (!path || !out) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: null argument");
    rcu_gguf* g = new rcu_gguf();
    g->fd = open(path, O_RDONLY);
    struct stat sb;
    if (g->fd < 0 || fstat(g->fd, &sb) != 0) {
        rcu_gguf_close(g);
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: cannot open %s", path);
    }
    g->size = (uint64_t)sb.st_size;
    void* m = g->size ? mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0) : MAP_FAILED;
    if (m == MAP_FAILED) {
        rcu_gguf_close(g);
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: cannot map %s (%llu bytes)", path, (unsigned long long)g->size);
    }
    g->map = (const uint8_t*)m;
    Cursor c{g->map, g->size, 0};
    const uint32_t magic = c.get<uint32_t>();
    const uint32_t version = c.get<uint32_t>();
    // "GGUF" little endian; the reference also accepts the byte-swapped spelling of the magic
    if (!c.ok || (magic != 0x46554747u && magic != 0x47475546u) || version < 1 || version > 3) {
        rcu_gguf_close(g);
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: %s is not a GGUF v1-v3 file (magic %08x, version %u)", path, magic, version);
    }
    g->version = (int)version;
    const uint64_t n_tensors = c.len(g->version), n_kv = c.len(g->version);
    for (uint64_t i = 0; i < n_kv && c.ok; ++i) {
        std::string key = c.str(g->version);
        const uint32_t vt = c.get<uint32_t>();
        MetaValue v;
        if (!c.ok || !read_value(c, g->version, vt, &v)) {
            rcu_gguf_close(g);
            return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: bad metadata entry %llu ('%s', value type %u)", (unsigned long long)i, key.c_str(), vt);
        }
        g->meta[key] = v;
    }
    for (uint64_t i = 0; i < n_tensors && c.ok; ++i) {
        TensorInfo t;
        t.name = c.str(g->version);
        t.rank = c.get<uint32_t>();
        if (!c.ok || t.rank < 1 || t.rank > 4) {
            rcu_gguf_close(g);
            return gguf_fail(RCU_ERR_UNSUPPORTED, "gguf: tensor %llu has rank %u (1..4 supported)", (unsigned long long)i, t.rank);
        }
        uint64_t dims[4];
        for (uint32_t d = 0; d < t.rank; ++d) dims[d] = c.len(g->version);
        bool overflow = false;
        for (uint32_t d = 0; d < t.rank; ++d) {             // stored innermost first
            t.shape[d] = dims[t.rank - 1 - d];
            overflow = overflow || __builtin_mul_overflow(t.numel, t.shape[d], &t.numel);
        }
        if (overflow || t.numel > (1ull << 48)) {           // no tensor of a real file comes near; larger counts would wrap the byte arithmetic below
            rcu_gguf_close(g);
            return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: tensor %llu ('%s') has an impossible shape", (unsigned long long)i, t.name.c_str());
        }
        t.ggml_type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        uint64_t bn = 0, ts = 0;
        if (block_layout(t.ggml_type, &bn, &ts) && t.numel % bn == 0) t.file_bytes = t.numel / bn * ts;
        g->by_name[t.name] = g->tensors.size();
        g->tensors.push_back(t);
    }
    if (!c.ok) {
        rcu_gguf_close(g);
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: %s is truncated inside its header", path);
    }
    uint64_t alignment = 32;
    auto it = g->meta.find("general.alignment");
    if (it != g->meta.end() && it->second.type <= 5 && (int64_t)it->second.u > 0) alignment = it->second.u;
    g->data_offset = (c.pos + alignment - 1) / alignment * alignment;
    *out = g;
    return RCU_OK;
}

uint32_t rcu_gguf_version(const rcu_gguf* g) { return g ? (uint32_t)g->version : 0; }
uint64_t rcu_gguf_tensor_count(const rcu_gguf* g) { return g ? g->tensors.size() : 0; }

int64_t rcu_gguf_find(const rcu_gguf* g, const char* name) {
    if (!g || !name) return -1;
    auto it = g->by_name.find(name);
    return it == g->by_name.end() ? -1 : (int64_t)it->second;
}

rcu_status rcu_gguf_tensor(const rcu_gguf* g, uint64_t index, rcu_gguf_tensor_info* out) {
    if (!g || !out || index >= g->tensors.size()) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: tensor index out of range");
    const TensorInfo& t = g->tensors[index];
    out->name = t.name.c_str();
    out->rank = t.rank;
    for (int i = 0; i < 4; ++i) out->shape[i] = t.shape[i];
    out->ggml_type = t.ggml_type;
    out->numel = t.numel;
    out->file_bytes = t.file_bytes;
    return RCU_OK;
}

rcu_status rcu_gguf_meta_u64(const rcu_gguf* g, const char* key, uint64_t* out) {
    if (!g || !key || !out) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: no metadata key '%s'", key);
    const MetaValue& v = it->second;
    if (v.type == 6 || v.type == 12 || v.type == 8 || v.type == 9) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: '%s' is not an integer", key);
    *out = v.u;
    return RCU_OK;
}

rcu_status rcu_gguf_meta_f64(const rcu_gguf* g, const char* key, double* out) {
    if (!g || !key || !out) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end()) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: no metadata key '%s'", key);
    if (it->second.type != 6 && it->second.type != 12) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: '%s' is not a float", key);
    *out = it->second.f;
    return RCU_OK;
}

rcu_status rcu_gguf_meta_str(const rcu_gguf* g, const char* key, char* buf, uint64_t buf_bytes) {
    if (!g || !key || !buf || buf_bytes == 0) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: null argument");
    auto it = g->meta.find(key);
    if (it == g->meta.end() || it->second.type != 8) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: no string metadata key '%s'", key);
    snprintf(buf, (size_t)buf_bytes, "%s", it->second.s.c_str());
    return RCU_OK;
}

int32_t rcu_gguf_target_dtype(uint32_t ggml_type, int f16_device) {
    switch (ggml_type) {
        case GGML_F32: return RCU_F32;
        case GGML_F16: return RCU_F16;
        case GGML_Q8_0: return f16_device ? RCU_Q8_0H : RCU_Q8_0F;      // gguf.rs:128-141
        case GGML_Q4_K: return f16_device ? RCU_Q4_KH : RCU_Q4_KF;      // gguf.rs:142-155
        default: return -1;
    }
}

rcu_status rcu_gguf_transcode(const rcu_gguf* g, uint64_t index, int32_t dt, void* host_out, uint64_t out_bytes) {
    if (!g || !host_out || index >= g->tensors.size()) return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: bad argument");
    const TensorInfo& t = g->tensors[index];
    uint64_t bn = 0, ts = 0;
    if (!block_layout(t.ggml_type, &bn, &ts)) return gguf_fail(RCU_ERR_UNSUPPORTED, "unsupported ggml dtype %u ('%s')", t.ggml_type, t.name.c_str());
    if (t.numel % bn != 0)
        return gguf_fail(RCU_ERR_INVALID_ARG, "the number of elements %llu is not divisible by the block size %llu", (unsigned long long)t.numel,
                         (unsigned long long)bn);                         // gguf.rs:119-123
    if (g->data_offset > g->size || t.offset > g->size - g->data_offset || t.file_bytes > g->size - g->data_offset - t.offset)
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: tensor '%s' runs past the end of the file", t.name.c_str());
    const uint64_t begin = g->data_offset + t.offset;
    const uint64_t need = rcu_dtype_nbytes(dt, t.numel);
    if (need == 0 || out_bytes < need)
        return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: '%s' as dtype %d needs %llu bytes, buffer has %llu", t.name.c_str(), dt, (unsigned long long)need,
                         (unsigned long long)out_bytes);
    const uint8_t* src = g->map + begin;
    uint8_t* dst = (uint8_t*)host_out;
    uint64_t off[4] = {0, 0, 0, 0};
    const int nseg = rcu_dtype_segments(dt, t.numel, off);
    (void)nseg;
    const uint64_t nblocks = t.numel / bn;
    switch (t.ggml_type) {
        case GGML_F32:
            if (dt != RCU_F32) break;
            memcpy(dst, src, t.numel * 4);
            return RCU_OK;
        case GGML_F16:
            if (dt != RCU_F16) break;
            memcpy(dst, src, t.numel * 2);
            return RCU_OK;
        case GGML_Q8_0: {
            if (dt != RCU_Q8_0F && dt != RCU_Q8_0H) break;
            memset(dst, 0, need);
            for (uint64_t b = 0; b < nblocks; ++b) {
                const uint8_t* blk = src + b * 34;
                uint16_t d;
                memcpy(&d, blk, 2);
                memcpy(dst + off[0] + b * 32, blk + 2, 32);
                if (dt == RCU_Q8_0H) memcpy(dst + off[1] + b * 2, &d, 2);
                else { const float f = f16_bits_to_f32(d); memcpy(dst + off[1] + b * 4, &f, 4); }
            }
            return RCU_OK;
        }
        case GGML_Q4_K: {
            if (dt != RCU_Q4_KF && dt != RCU_Q4_KH) break;
            memset(dst, 0, need);
            for (uint64_t b = 0; b < nblocks; ++b) {
                const uint8_t* blk = src + b * 144;
                uint16_t d, dmin;
                memcpy(&d, blk, 2);
                memcpy(&dmin, blk + 2, 2);
                memcpy(dst + off[1] + b * 12, blk + 4, 12);
                memcpy(dst + off[0] + b * 128, blk + 16, 128);
                if (dt == RCU_Q4_KH) {
                    memcpy(dst + off[2] + b * 2, &dmin, 2);
                    memcpy(dst + off[3] + b * 2, &d, 2);
                } else {
                    const float fm = f16_bits_to_f32(dmin), fd = f16_bits_to_f32(d);
                    memcpy(dst + off[2] + b * 4, &fm, 4);
                    memcpy(dst + off[3] + b * 4, &fd, 4);
                }
            }
            return RCU_OK;
        }
    }
    return gguf_fail(RCU_ERR_INVALID_ARG, "gguf: '%s' (ggml dtype %u) cannot be loaded as dtype %d", t.name.c_str(), t.ggml_type, dt);
}

}  // extern "C"
