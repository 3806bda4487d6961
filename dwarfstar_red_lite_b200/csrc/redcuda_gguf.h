// Minimal read-only GGUF (v2/v3) view over an mmap'd file: metadata scalars, architecture, vocabulary size, tensor
// directory. Written against the public GGUF layout; it accepts what the reference's reader accepts for the
// qwen3next files this backend serves (native/redlite_native_gguf_dir.c:320-384) and rejects truncated input.
#pragma once
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <fcntl.h>
#include <unistd.h>

#include <map>
#include <string>

namespace rc {

struct GgufTensor {
    uint32_t type = 0, n_dims = 0;
    uint64_t shape[4] = {1, 1, 1, 1};
    uint64_t offset = 0;      // absolute file offset
    uint64_t bytes = 0;
};

class GgufFile {
public:
    std::string path, architecture, error;
    std::map<std::string, double> scalars;      // every numeric / bool metadata value
    std::map<std::string, GgufTensor> tensors;
    uint64_t vocab = 0, file_size = 0;
    const uint8_t *map = nullptr;

    ~GgufFile() { close_file(); }

    bool open_file(const char *p) {
        path = p;
        fd_ = ::open(p, O_RDONLY);
        if (fd_ < 0) { error = std::string("cannot open ") + p; return false; }
        struct stat st;
        if (fstat(fd_, &st) != 0 || st.st_size < 24) { error = "GGUF file too small"; return false; }
        file_size = (uint64_t)st.st_size;
        void *m = mmap(nullptr, file_size, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (m == MAP_FAILED) { error = "mmap failed"; return false; }
        map = (const uint8_t *)m;
        return parse();
    }
    void close_file() {
        if (map) munmap((void *)map, file_size);
        if (fd_ >= 0) ::close(fd_);
        map = nullptr; fd_ = -1;
    }
    const GgufTensor *find(const std::string &name) const { auto it = tensors.find(name); return it == tensors.end() ? nullptr : &it->second; }
    const GgufTensor *find_layer(uint32_t layer, const char *suffix) const { return find("blk." + std::to_string(layer) + "." + suffix); }
    const uint8_t *data(const GgufTensor *t) const { return map + t->offset; }
    uint32_t u32(const char *key) const { auto it = scalars.find(key); return it == scalars.end() || it->second < 0 ? 0u : (uint32_t)it->second; }
    float f32(const char *key) const { auto it = scalars.find(key); return it == scalars.end() ? 0.f : (float)it->second; }

    // bytes of a tensor of this type and shape, 0 when the type is not one this backend can hold
    static uint64_t tensor_bytes(uint32_t type, uint32_t n_dims, const uint64_t *shape) {
        uint64_t row;
        const uint64_t n0 = shape[0];
        if (n0 > (1ull << 40)) return 0;                 // hostile shapes must not wrap the products below
        switch (type) {
            case 0: row = n0 * 4u; break;
            case 1: row = n0 * 2u; break;
            case 8: if (n0 % 32u) return 0; row = n0 / 32u * 34u; break;          // Q8_0
            case 10: if (n0 % 256u) return 0; row = n0 / 256u * 84u; break;       // Q2_K
            case 12: if (n0 % 256u) return 0; row = n0 / 256u * 144u; break;      // Q4_K
            case 13: if (n0 % 256u) return 0; row = n0 / 256u * 176u; break;      // Q5_K
            case 14: if (n0 % 256u) return 0; row = n0 / 256u * 210u; break;
            case 16: if (n0 % 256u) return 0; row = n0 / 256u * 66u; break;
            case 21: if (n0 % 256u) return 0; row = n0 / 256u * 110u; break;
            default: return 0;
        }
        for (uint32_t d = 1; d < n_dims; ++d) {
            if (shape[d] && row > UINT64_MAX / shape[d]) return 0;     // overflow: reported as an unsupported tensor
            row *= shape[d];
        }
        return row;
    }

private:
    int fd_ = -1;
    uint64_t pos_ = 0;

    bool need(uint64_t n) { if (n > file_size - pos_) { error = "GGUF truncated"; return false; } return true; }
    bool rd(void *dst, uint64_t n) { if (!need(n)) return false; memcpy(dst, map + pos_, n); pos_ += n; return true; }
    bool rd_str(std::string &s) {
        uint64_t n = 0;
        if (!rd(&n, 8) || n > (1u << 24) || !need(n)) { error = "GGUF string parse failed"; return false; }
        s.assign((const char *)map + pos_, (size_t)n); pos_ += n;
        return true;
    }
    static uint64_t scalar_size(uint32_t t) { switch (t) { case 0: case 1: case 7: return 1; case 2: case 3: return 2; case 4: case 5: case 6: return 4; case 10: case 11: case 12: return 8; default: return 0; } }
    bool rd_scalar(uint32_t t, double &v) {
        uint8_t b[8] = {0};
        const uint64_t n = scalar_size(t);
        if (!n || !rd(b, n)) return false;
        switch (t) {
            case 0: v = b[0]; break; case 1: v = (int8_t)b[0]; break; case 7: v = b[0] ? 1 : 0; break;
            case 2: { uint16_t x; memcpy(&x, b, 2); v = x; break; } case 3: { int16_t x; memcpy(&x, b, 2); v = x; break; }
            case 4: { uint32_t x; memcpy(&x, b, 4); v = x; break; } case 5: { int32_t x; memcpy(&x, b, 4); v = x; break; }
            case 6: { float x; memcpy(&x, b, 4); v = x; break; }
            case 10: { uint64_t x; memcpy(&x, b, 8); v = (double)x; break; } case 11: { int64_t x; memcpy(&x, b, 8); v = (double)x; break; }
            case 12: { memcpy(&v, b, 8); break; }
        }
        return true;
    }
    bool skip_value(uint32_t t, const std::string &key) {
        if (t == 8) { std::string s; if (!rd_str(s)) return false; if (key == "general.architecture") architecture = s; return true; }
        if (t == 9) {
            uint32_t sub = 0; uint64_t cnt = 0;
            if (!rd(&sub, 4) || !rd(&cnt, 8) || sub == 9) { error = "GGUF array parse failed"; return false; }
            if (key == "tokenizer.ggml.tokens" && sub == 8) vocab = cnt;
            const uint64_t ss = scalar_size(sub);
            if (ss) { if (cnt > (file_size - pos_) / ss) { error = "GGUF array exceeds the file"; return false; } pos_ += cnt * ss; return true; }
            if (sub != 8) { error = "GGUF array of unknown element type"; return false; }
            for (uint64_t i = 0; i < cnt; ++i) { uint64_t n = 0; if (!rd(&n, 8) || !need(n)) { error = "GGUF string array parse failed"; return false; } pos_ += n; }
            return true;
        }
        double v = 0;
        if (!rd_scalar(t, v)) { error = "GGUF scalar parse failed"; return false; }
        scalars[key] = v;
        return true;
    }
    bool parse() {
        uint32_t version = 0; uint64_t n_tensors = 0, n_kv = 0;
        if (memcmp(map, "GGUF", 4) != 0) { error = "not a GGUF file"; return false; }
        pos_ = 4;
        if (!rd(&version, 4) || (version != 2u && version != 3u) || !rd(&n_tensors, 8) || !rd(&n_kv, 8) || n_tensors > (1u << 24) || n_kv > (1u << 24)) {
            error = "invalid GGUF header"; return false;
        }
        for (uint64_t i = 0; i < n_kv; ++i) {
            std::string key; uint32_t t = 0;
            if (!rd_str(key) || !rd(&t, 4) || !skip_value(t, key)) { if (error.empty()) error = "GGUF metadata parse failed"; return false; }
        }
        struct Pending { std::string name; GgufTensor t; };
        std::map<std::string, GgufTensor> rel;
        for (uint64_t i = 0; i < n_tensors; ++i) {
            std::string name; GgufTensor t;
            if (!rd_str(name) || !rd(&t.n_dims, 4) || t.n_dims == 0 || t.n_dims > 4) { error = "tensor descriptor parse failed"; return false; }
            for (uint32_t d = 0; d < t.n_dims; ++d) if (!rd(&t.shape[d], 8)) return false;
            if (!rd(&t.type, 4) || !rd(&t.offset, 8)) return false;
            t.bytes = tensor_bytes(t.type, t.n_dims, t.shape);
            rel[name] = t;
        }
        uint64_t align = u32("general.alignment");
        if (!align) align = 32;
        const uint64_t base = (pos_ + align - 1) / align * align;
        if (base > file_size) { error = "invalid GGUF data base"; return false; }
        for (auto &kv : rel) {
            GgufTensor t = kv.second;
            if (t.offset > file_size - base || (t.bytes && t.bytes > file_size - base - t.offset)) { error = "tensor " + kv.first + " lies beyond the file"; return false; }
            t.offset += base;
            tensors[kv.first] = t;
        }
        return true;
    }
};

}  // namespace rc
