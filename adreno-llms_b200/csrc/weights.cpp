// Weight bundle loader: the role of class Weights in the reference
// (src/models/lfm2-5-350m/src/weights.h:13-51, weights.cpp:169-297).
//
// Reads the flat little-endian bundle written by scripts/convert_hf_to_bin.py
// (build_layout / make_meta, lines 103-169) and by the per-model
// scripts/quantize_weights.py / quantize_q4.py: tensor bytes at
// meta.tensors[name].offset, `size_bytes` (older files: `size`), `shape`, `dtype` in
// {float32, float16, bfloat16, int8, q4_packed}; a q4_packed shape is [N, K/2] bytes.
// The file is mmapped; a tensor is uploaded to the GPU the first time it is asked
// for and stays until nn_weights_free (the reference releases in ~Weights).
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

#include "../../include/nnopt_b200.h"
#include "internal.h"

namespace {

struct TensorMeta {
    size_t offset = 0, size_bytes = 0, num_elements = 0;
    std::string dtype = "float32";
    std::vector<int> shape;
    void* dev = nullptr;
};

// ---- a small JSON reader (objects, arrays, strings, numbers, literals) -------------
struct JVal {
    enum T { NUL, BOOL, NUM, STR, ARR, OBJ } t = NUL;
    double num = 0;
    bool b = false;
    std::string str;
    std::vector<JVal> arr;
    std::vector<std::pair<std::string, JVal>> obj;  // keeps file order
    const JVal* get(const char* k) const {
        for (auto& kv : obj)
            if (kv.first == k) return &kv.second;
        return nullptr;
    }
};

struct JParser {
    const char* p;
    const char* end;
    bool ok = true;
    void ws() { while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p; }
    bool parse_string(std::string& out) {
        if (p >= end || *p != '"') return ok = false;
        ++p;
        while (p < end && *p != '"') {
            if (*p == '\\' && p + 1 < end) {
                ++p;
                switch (*p) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': {  // keep BMP escapes as UTF-8
                        if (p + 4 >= end) return ok = false;
                        unsigned cp = (unsigned)strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16);
                        if (cp < 0x80) out += (char)cp;
                        else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
                        else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
                        p += 4;
                        break;
                    }
                    default: out += *p;
                }
                ++p;
            } else {
                out += *p++;
            }
        }
        if (p >= end) return ok = false;
        ++p;
        return true;
    }
    bool parse(JVal& v, int depth = 0) {
        if (depth > 64) return ok = false;
        ws();
        if (p >= end) return ok = false;
        if (*p == '{') {
            v.t = JVal::OBJ;
            ++p;
            ws();
            if (p < end && *p == '}') { ++p; return true; }
            while (ok) {
                ws();
                std::string k;
                if (!parse_string(k)) return false;
                ws();
                if (p >= end || *p != ':') return ok = false;
                ++p;
                v.obj.emplace_back(k, JVal());
                if (!parse(v.obj.back().second, depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == '}') { ++p; return true; }
                return ok = false;
            }
        } else if (*p == '[') {
            v.t = JVal::ARR;
            ++p;
            ws();
            if (p < end && *p == ']') { ++p; return true; }
            while (ok) {
                v.arr.emplace_back();
                if (!parse(v.arr.back(), depth + 1)) return false;
                ws();
                if (p < end && *p == ',') { ++p; continue; }
                if (p < end && *p == ']') { ++p; return true; }
                return ok = false;
            }
        } else if (*p == '"') {
            v.t = JVal::STR;
            return parse_string(v.str);
        } else if (!strncmp(p, "true", 4) && end - p >= 4) { v.t = JVal::BOOL; v.b = true; p += 4; return true; }
        else if (!strncmp(p, "false", 5) && end - p >= 5) { v.t = JVal::BOOL; v.b = false; p += 5; return true; }
        else if (!strncmp(p, "null", 4) && end - p >= 4) { v.t = JVal::NUL; p += 4; return true; }
        else {
            char* e = nullptr;
            v.num = strtod(p, &e);
            if (e == p) return ok = false;
            v.t = JVal::NUM;
            p = e;
            return true;
        }
        return ok;
    }
};

size_t bytes_per_element(const std::string& dt) {
    if (dt == "float16" || dt == "bfloat16") return 2;
    if (dt == "int8" || dt == "q4_packed") return 1;  // q4_packed shape counts bytes
    return 4;
}

float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (!man) bits = sign;
        else {
            int sh = 0;
            while (!(man & 0x400u)) { man <<= 1; ++sh; }
            bits = sign | ((uint32_t)(113 - sh) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112u) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

struct nn_weights {
    nn_context* ctx = nullptr;
    uint8_t* mapped = nullptr;
    size_t mapped_size = 0;
    int fd = -1;
    std::map<std::string, TensorMeta> tensors;  // sorted, like the bundle
    std::vector<std::string> keys;
};

extern "C" int nn_weights_free(nn_weights* w) {
    if (!w) return NN_OK;
    if (w->ctx) {
        cudaSetDevice(w->ctx->device);
        cudaStreamSynchronize(w->ctx->stream);
    }
    for (auto& kv : w->tensors) {
        if (kv.second.dev) {
            if (w->ctx) {
                auto it = w->ctx->registry.find((uintptr_t)kv.second.dev);
                if (it != w->ctx->registry.end()) {
                    free_scale_pad(it->second);
                    w->ctx->registry.erase(it);
                }
            }
            cudaFree(kv.second.dev);
        }
    }
    if (w->mapped && w->mapped != MAP_FAILED) munmap(w->mapped, w->mapped_size);
    if (w->fd >= 0) close(w->fd);
    delete w;
    return NN_OK;
}

extern "C" int nn_weights_load(nn_context* ctx, const char* bin_path, const char* meta_path, nn_weights** out) {
    // ctx may be null for host-only use (metadata and nn_weights_get_host_f32); get_buffer then fails.
    if (!bin_path || !meta_path || !out) return NN_FAIL(NN_ERR_ARG, "nn_weights_load: null argument");
    *out = nullptr;
    nn_weights* w = new nn_weights();
    w->ctx = ctx;
    w->fd = open(bin_path, O_RDONLY);
    if (w->fd < 0) {
        int rc = NN_FAIL(NN_ERR_IO, "weights: failed to open %s (errno=%d)", bin_path, errno);
        nn_weights_free(w);
        return rc;
    }
    struct stat st;
    if (fstat(w->fd, &st) != 0 || st.st_size <= 0) {
        int rc = NN_FAIL(NN_ERR_IO, "weights: fstat failed or empty file %s (errno=%d)", bin_path, errno);
        nn_weights_free(w);
        return rc;
    }
    w->mapped_size = (size_t)st.st_size;
    w->mapped = (uint8_t*)mmap(nullptr, w->mapped_size, PROT_READ, MAP_PRIVATE, w->fd, 0);
    if (w->mapped == MAP_FAILED) {
        w->mapped = nullptr;
        int rc = NN_FAIL(NN_ERR_IO, "weights: mmap of %s failed (errno=%d)", bin_path, errno);
        nn_weights_free(w);
        return rc;
    }
    std::ifstream mf(meta_path);
    if (!mf.is_open()) {
        int rc = NN_FAIL(NN_ERR_IO, "weights: failed to open metadata %s", meta_path);
        nn_weights_free(w);
        return rc;
    }
    std::stringstream ss;
    ss << mf.rdbuf();
    const std::string text = ss.str();
    JParser jp{text.data(), text.data() + text.size()};
    JVal root;
    if (!jp.parse(root) || root.t != JVal::OBJ) {
        int rc = NN_FAIL(NN_ERR_IO, "weights: could not parse metadata %s", meta_path);
        nn_weights_free(w);
        return rc;
    }
    // {"tensors": {name: {...}}} or the flat form {name: {...}} the reference also accepts
    const JVal* tens = root.get("tensors");
    if (!tens || tens->t != JVal::OBJ) tens = &root;
    for (auto& kv : tens->obj) {
        const JVal& o = kv.second;
        if (o.t != JVal::OBJ) continue;
        const JVal* off = o.get("offset");
        const JVal* sz = o.get("size_bytes");
        if (!sz) sz = o.get("size");
        if (!off || !sz || off->t != JVal::NUM || sz->t != JVal::NUM) continue;
        TensorMeta m;
        m.offset = (size_t)off->num;
        m.size_bytes = (size_t)sz->num;
        if (const JVal* dt = o.get("dtype"))
            if (dt->t == JVal::STR) m.dtype = dt->str;
        if (const JVal* sh = o.get("shape"))
            if (sh->t == JVal::ARR)
                for (auto& d : sh->arr) m.shape.push_back((int)d.num);
        m.num_elements = m.size_bytes / bytes_per_element(m.dtype);
        if (m.size_bytes > 0) w->tensors[kv.first] = m;
    }
    if (w->tensors.empty()) {
        int rc = NN_FAIL(NN_ERR_IO, "weights: no tensors found in %s", meta_path);
        nn_weights_free(w);
        return rc;
    }
    for (auto& kv : w->tensors) w->keys.push_back(kv.first);
    *out = w;
    return NN_OK;
}

static const TensorMeta* find(const nn_weights* w, const char* key) {
    if (!w || !key) return nullptr;
    auto it = w->tensors.find(key);
    return it == w->tensors.end() ? nullptr : &it->second;
}

extern "C" int nn_weights_has_tensor(const nn_weights* w, const char* key) { return find(w, key) ? 1 : 0; }

extern "C" nn_buf nn_weights_get_buffer(nn_weights* w, const char* key, int optional) {
    if (!w || !key) { NN_FAIL(NN_ERR_ARG, "nn_weights_get_buffer: null argument"); return nullptr; }
    auto it = w->tensors.find(key);
    if (it == w->tensors.end()) {
        if (!optional) NN_FAIL(NN_ERR_NOTFOUND, "weight key not found: '%s'", key);
        return nullptr;
    }
    TensorMeta& m = it->second;
    if (m.dev) return m.dev;
    if (!w->ctx) {
        NN_FAIL(NN_ERR_ARG, "nn_weights_get_buffer: bundle was loaded without a context");
        return nullptr;
    }
    if (m.offset + m.size_bytes > w->mapped_size) {
        NN_FAIL(NN_ERR_IO, "tensor %s exceeds file bounds (offset %zu + %zu > %zu)", key, m.offset, m.size_bytes, w->mapped_size);
        return nullptr;
    }
    cudaSetDevice(w->ctx->device);
    cudaError_t e = cudaMalloc(&m.dev, m.size_bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(m.dev, w->mapped + m.offset, m.size_bytes, cudaMemcpyHostToDevice, w->ctx->stream);
    if (e != cudaSuccess) {
        NN_FAIL(NN_ERR_CUDA, "failed to create buffer for %s: %s", key, cudaGetErrorString(e));
        if (m.dev) cudaFree(m.dev);
        m.dev = nullptr;
    }
    return m.dev;
}

extern "C" const char* nn_weights_get_dtype(const nn_weights* w, const char* key) {
    const TensorMeta* m = find(w, key);
    return m ? m->dtype.c_str() : "";
}
extern "C" int nn_weights_get_shape(const nn_weights* w, const char* key, int* dims, int max_dims) {
    const TensorMeta* m = find(w, key);
    if (!m) return 0;
    for (int i = 0; i < (int)m->shape.size() && i < max_dims; ++i)
        if (dims) dims[i] = m->shape[i];
    return (int)m->shape.size();
}
extern "C" size_t nn_weights_get_size_bytes(const nn_weights* w, const char* key) {
    const TensorMeta* m = find(w, key);
    return m ? m->size_bytes : 0;
}
extern "C" size_t nn_weights_get_num_elements(const nn_weights* w, const char* key) {
    const TensorMeta* m = find(w, key);
    return m ? m->num_elements : 0;
}
extern "C" int nn_weights_num_keys(const nn_weights* w) { return w ? (int)w->keys.size() : 0; }
extern "C" const char* nn_weights_key_at(const nn_weights* w, int i) {
    return (w && i >= 0 && i < (int)w->keys.size()) ? w->keys[i].c_str() : nullptr;
}

// get_host_vec: decode to fp32 on the host.  int8 gives the codes, q4_packed the bytes.
extern "C" int nn_weights_get_host_f32(const nn_weights* w, const char* key, float* out, size_t max_elems) {
    const TensorMeta* m = find(w, key);
    if (!m) return NN_FAIL(NN_ERR_NOTFOUND, "weight key not found: '%s'", key ? key : "(null)");
    if (!out) return NN_FAIL(NN_ERR_ARG, "nn_weights_get_host_f32: null output");
    if (m->offset + m->size_bytes > w->mapped_size) return NN_FAIL(NN_ERR_IO, "tensor %s exceeds file bounds", key);
    const size_t n = m->num_elements < max_elems ? m->num_elements : max_elems;
    const uint8_t* base = w->mapped + m->offset;
    if (m->dtype == "float16") {
        for (size_t i = 0; i < n; ++i) out[i] = f16_to_f32(((const uint16_t*)base)[i]);
    } else if (m->dtype == "bfloat16") {
        for (size_t i = 0; i < n; ++i) {
            uint32_t b = (uint32_t)((const uint16_t*)base)[i] << 16;
            memcpy(&out[i], &b, 4);
        }
    } else if (m->dtype == "int8") {
        for (size_t i = 0; i < n; ++i) out[i] = (float)((const int8_t*)base)[i];
    } else if (m->dtype == "q4_packed") {
        for (size_t i = 0; i < n; ++i) out[i] = (float)base[i];
    } else {
        memcpy(out, base, n * sizeof(float));
    }
    return NN_OK;
}

extern "C" int nn_weights_register_quantized(nn_context* ctx, nn_weights* w) {
    if (!ctx || !w) return NN_FAIL(NN_ERR_ARG, "nn_weights_register_quantized: null argument");
    int registered = 0;
    for (const std::string& name : w->keys) {
        const TensorMeta& m = w->tensors[name];
        const bool i8 = m.dtype == "int8", q4 = m.dtype == "q4_packed";
        if (!i8 && !q4) continue;
        const std::string sname = name + ".scale";
        auto sit = w->tensors.find(sname);
        if (sit == w->tensors.end() || m.shape.size() != 2) continue;
        int N = m.shape[0], K = m.shape[1];
        if (q4) {
            // shape is [N, K/2] packed bytes; the unpacked K comes from the scale columns
            if (sit->second.shape.size() != 2) continue;
            K = sit->second.shape[1] * 32;
        }
        nn_buf W = nn_weights_get_buffer(w, name.c_str(), 0);
        nn_buf S = nn_weights_get_buffer(w, sname.c_str(), 0);
        if (!W || !S) continue;
        const int rc = i8 ? nn_register_int8_weight(ctx, W, S, N, K) : nn_register_q4_weight(ctx, W, S, N, K);
        if (rc == NN_OK) ++registered;
    }
    return registered;
}
