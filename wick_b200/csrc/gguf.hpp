// Minimal GGUF v3 reader over an in-memory image, with the acceptance rules of
// wick's parser (wick/src/gguf.rs:407-559): magic "GGUF", version 3 only,
// `general.alignment` (UINT32, default 32), tensor offsets relative to the aligned end
// of the header, every tensor checked against the image size.  Metadata getters are
// type-strict like wick's (gguf.rs:570-654): a UINT32 key stored as INT32 is "missing".
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace wick {

struct GgufTensor {
    std::vector<uint64_t> dims;  // ggml order: dims[0] is the innermost (row length k)
    uint32_t type = 0;
    uint64_t offset = 0;  // absolute
    uint64_t size = 0;    // bytes, 0 if the type is not one we understand
};

struct GgufValue {
    uint32_t type = 0;       // GGUF value type id
    uint32_t elem_type = 0;  // for arrays
    uint64_t u = 0;          // integer / bool payload
    double f = 0;            // float payload
    std::string s;
    std::vector<int64_t> ints;  // integer arrays
    uint64_t count = 0;         // array length
};

class GgufImage {
  public:
    GgufImage(const uint8_t* data, size_t len) : p_(data), n_(len) { parse(); }

    const GgufValue* find(const std::string& key) const {
        auto it = kv_.find(key);
        return it == kv_.end() ? nullptr : &it->second;
    }
    bool get_u32(const std::string& key, uint32_t* out) const {
        const GgufValue* v = find(key);
        if (!v || v->type != 4) return false;
        *out = (uint32_t)v->u;
        return true;
    }
    bool get_f32(const std::string& key, float* out) const {
        const GgufValue* v = find(key);
        if (!v || v->type != 6) return false;
        *out = (float)v->f;
        return true;
    }
    bool get_str(const std::string& key, std::string* out) const {
        const GgufValue* v = find(key);
        if (!v || v->type != 8) return false;
        *out = v->s;
        return true;
    }
    bool get_i32_array(const std::string& key, std::vector<int32_t>* out) const {
        const GgufValue* v = find(key);
        if (!v || v->type != 9 || v->elem_type != 5) return false;
        out->assign(v->ints.begin(), v->ints.end());
        return true;
    }
    const GgufTensor* tensor(const std::string& name) const {
        auto it = tensors_.find(name);
        return it == tensors_.end() ? nullptr : &it->second;
    }
    const uint8_t* data() const { return p_; }

  private:
    const uint8_t* p_;
    size_t n_;
    size_t pos_ = 0;
    std::map<std::string, GgufValue> kv_;
    std::map<std::string, GgufTensor> tensors_;

    void need(size_t k) const {
        if (pos_ + k > n_ || pos_ + k < pos_) throw std::runtime_error("GGUF: truncated header");
    }
    template <class T>
    T rd() {
        need(sizeof(T));
        T v;
        memcpy(&v, p_ + pos_, sizeof(T));
        pos_ += sizeof(T);
        return v;
    }
    std::string rd_str() {
        uint64_t len = rd<uint64_t>();
        need(len);
        std::string s((const char*)p_ + pos_, (size_t)len);
        pos_ += len;
        return s;
    }
    static size_t scalar_size(uint32_t t) {
        switch (t) {
            case 0: case 1: case 7: return 1;
            case 2: case 3: return 2;
            case 4: case 5: case 6: return 4;
            case 10: case 11: case 12: return 8;
            default: return 0;
        }
    }
    void rd_scalar(uint32_t t, GgufValue& v) {
        switch (t) {
            case 0: v.u = rd<uint8_t>(); break;
            case 1: v.u = (uint64_t)(int64_t)rd<int8_t>(); break;
            case 2: v.u = rd<uint16_t>(); break;
            case 3: v.u = (uint64_t)(int64_t)rd<int16_t>(); break;
            case 4: v.u = rd<uint32_t>(); break;
            case 5: v.u = (uint64_t)(int64_t)rd<int32_t>(); break;
            case 6: v.f = rd<float>(); break;
            case 7: v.u = rd<uint8_t>(); break;
            case 10: v.u = rd<uint64_t>(); break;
            case 11: v.u = (uint64_t)rd<int64_t>(); break;
            case 12: v.f = rd<double>(); break;
            default: throw std::runtime_error("GGUF: unknown metadata value type " + std::to_string(t));
        }
    }
    void rd_value(uint32_t t, GgufValue& v) {
        v.type = t;
        if (t == 8) {
            v.s = rd_str();
        } else if (t == 9) {
            v.elem_type = rd<uint32_t>();
            v.count = rd<uint64_t>();
            if (v.elem_type == 8) {
                for (uint64_t i = 0; i < v.count; i++) {  // strings (tokenizer tables): skipped
                    uint64_t len = rd<uint64_t>();
                    need(len);
                    pos_ += len;
                }
            } else if (v.elem_type == 9) {
                throw std::runtime_error("GGUF: nested arrays are not supported");
            } else {
                size_t es = scalar_size(v.elem_type);
                if (!es) throw std::runtime_error("GGUF: unknown array element type");
                bool is_int = v.elem_type != 6 && v.elem_type != 12;
                if (is_int && v.count <= (1u << 20)) {
                    v.ints.reserve(v.count);
                    for (uint64_t i = 0; i < v.count; i++) {
                        GgufValue e;
                        rd_scalar(v.elem_type, e);
                        v.ints.push_back((int64_t)e.u);
                    }
                } else {
                    if (es != 0 && v.count > (n_ - pos_) / es) throw std::runtime_error("GGUF: truncated header");  // (the product could wrap)
                    need(es * v.count);
                    pos_ += es * v.count;
                }
            }
        } else {
            rd_scalar(t, v);
        }
    }
    static uint64_t type_size(uint32_t type, uint64_t n_elems) {
        switch (type) {
            case 0: return n_elems * 4;             // F32
            case 1: return n_elems * 2;             // F16
            case 2: return n_elems / 32 * 18;       // Q4_0
            case 8: return n_elems / 32 * 34;       // Q8_0
            case 14: return n_elems / 256 * 210;    // Q6_K
            default: return 0;
        }
    }
    void parse() {
        if (n_ < 24) throw std::runtime_error("GGUF buffer too small (" + std::to_string(n_) + " bytes; need at least 24 for the header)");
        uint32_t magic = rd<uint32_t>();
        if (magic != 0x46554747u) throw std::runtime_error("not a GGUF file (bad magic)");
        uint32_t version = rd<uint32_t>();
        if (version != 3) throw std::runtime_error("unsupported GGUF version " + std::to_string(version) + " (expected 3)");
        uint64_t n_tensors = rd<uint64_t>();
        uint64_t n_kv = rd<uint64_t>();
        for (uint64_t i = 0; i < n_kv; i++) {
            std::string key = rd_str();
            uint32_t t = rd<uint32_t>();
            GgufValue v;
            rd_value(t, v);
            kv_[key] = std::move(v);
        }
        struct Raw { std::string name; GgufTensor t; };
        std::vector<Raw> raw;
        for (uint64_t i = 0; i < n_tensors; i++) {
            Raw r;
            r.name = rd_str();
            uint32_t nd = rd<uint32_t>();
            if (nd > 8) throw std::runtime_error("tensor " + r.name + " has too many dimensions");
            for (uint32_t d = 0; d < nd; d++) r.t.dims.push_back(rd<uint64_t>());
            r.t.type = rd<uint32_t>();
            r.t.offset = rd<uint64_t>();
            raw.push_back(std::move(r));
        }
        uint32_t align = 32;
        get_u32("general.alignment", &align);
        if (align == 0 || align > (1u << 20)) throw std::runtime_error("invalid GGUF alignment");
        uint64_t data0 = (pos_ + align - 1) / align * align;
        for (auto& r : raw) {
            uint64_t ne = 1;
            for (uint64_t d : r.t.dims) {
                // every dimension fits an int and the element count stays far below 2^64 (a wrapped count would pass the
                // size check below with a tiny size)
                if (d > 0x7fffffffull || (d != 0 && ne > (1ull << 40) / d)) throw std::runtime_error("tensor " + r.name + ": implausible shape");
                ne *= d;
            }
            r.t.size = type_size(r.t.type, ne);
            r.t.offset += data0;
            if (r.t.size && (r.t.offset + r.t.size > n_ || r.t.offset + r.t.size < r.t.offset))
                throw std::runtime_error("tensor " + r.name + " extends beyond file");
            tensors_[r.name] = r.t;
        }
    }
};

}  // namespace wick
