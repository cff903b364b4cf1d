// Weights by tensor name from a single safetensors file, checked against what the model's parts
// declare, with ONE error that lists every missing tensor, every unexpected tensor and every wrong
// shape.
//
// Format (src/models/loader.cpp:213-227): an unsigned 64-bit little-endian header length, a JSON
// header mapping each tensor name to dtype, shape and data_offsets (relative to the end of the
// header), then the raw little-endian data; "__metadata__" is skipped.  The file is mapped
// read-only; every malformed input the reference rejects (src/models/loader.cpp:79-140, 214-252)
// is rejected here.  (The reference collects missing keys the same way,
// src/models/model_param_validation.cpp:152-154, checks shapes one by one, :156-195, and only
// warns about leftovers, :198-218; here leftovers are part of the one error.)
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.hpp"

namespace easygpt::engine {

struct SafetensorsError : std::runtime_error {
    using std::runtime_error::runtime_error;
};
struct WeightError : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

enum class Stored { BF16, F16, F32, I32, I64 };

inline float bf16_to_float(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
// round to nearest, ties to even; NaN stays NaN
inline uint16_t float_to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
inline float f16_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ffu, u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; ++shift; }
            u = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) u = sign | 0x7f800000u | (man << 13);
    else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

struct StoredTensor {
    Stored dtype;
    std::vector<long long> shape;
    const unsigned char* data = nullptr;
    size_t bytes = 0;
    long long numel() const {
        long long n = 1;
        for (long long s : shape) n *= s;
        return n;
    }
    // the values as float32 (integer tables are not floating point: refused)
    void to_float(float* out) const {
        const long long n = numel();
        if (dtype == Stored::F32) std::memcpy(out, data, (size_t)n * 4);
        else if (dtype == Stored::BF16) { const uint16_t* p = (const uint16_t*)data; for (long long i = 0; i < n; ++i) out[i] = bf16_to_float(p[i]); }
        else if (dtype == Stored::F16) { const uint16_t* p = (const uint16_t*)data; for (long long i = 0; i < n; ++i) out[i] = f16_to_float(p[i]); }
        else throw SafetensorsError("an integer tensor was asked for as floating point");
    }
};

class SafetensorsFile {
public:
    explicit SafetensorsFile(const std::string& path) : path_(path) {
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw SafetensorsError("cannot open " + path + ": " + std::strerror(errno));
        struct stat st;
        if (fstat(fd_, &st) != 0) { ::close(fd_); throw SafetensorsError("cannot stat " + path); }
        size_ = (size_t)st.st_size;
        if (size_ < 8) { ::close(fd_); throw SafetensorsError(path + ": file is smaller than the 8-byte header length"); }
        map_ = (const unsigned char*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
        if (map_ == MAP_FAILED) { ::close(fd_); throw SafetensorsError("cannot map " + path); }
        try {
            read_header();
        } catch (...) {
            munmap((void*)map_, size_);
            ::close(fd_);
            throw;
        }
    }
    ~SafetensorsFile() {
        if (map_ && map_ != MAP_FAILED) munmap((void*)map_, size_);
        if (fd_ >= 0) ::close(fd_);
    }
    SafetensorsFile(const SafetensorsFile&) = delete;
    SafetensorsFile& operator=(const SafetensorsFile&) = delete;

    const std::map<std::string, StoredTensor>& entries() const { return entries_; }
    const StoredTensor* find(const std::string& name) const {
        auto it = entries_.find(name);
        return it == entries_.end() ? nullptr : &it->second;
    }

private:
    static std::string shape_text(const json::Value& shape) {
        std::string s = "[";
        for (size_t i = 0; i < shape.array.size(); ++i) s += (i ? ", " : "") + std::to_string(shape.array[i].integer);
        return s + "]";
    }
    void read_header() {
        uint64_t hlen = 0;
        for (int i = 7; i >= 0; --i) hlen = (hlen << 8) | map_[i];
        if (hlen > size_ - 8) throw SafetensorsError(path_ + ": header length " + std::to_string(hlen) + " exceeds the file size " + std::to_string(size_));
        json::Value header;
        try {
            header = json::parse((const char*)map_ + 8, (size_t)hlen);
        } catch (const json::ParseError& e) {
            throw SafetensorsError(path_ + ": header is not JSON: " + e.what());
        }
        if (!header.is_object()) throw SafetensorsError(path_ + ": header is not a JSON object");
        const size_t base = 8 + (size_t)hlen;
        for (auto& kv : header.object) {
            const std::string& name = kv.first;
            if (name == "__metadata__") continue;
            const json::Value& meta = kv.second;
            const json::Value* dt = meta.find("dtype");
            if (!dt || !dt->is_string()) throw SafetensorsError("tensor '" + name + "': missing dtype");
            StoredTensor t;
            size_t elem;
            if (dt->string == "BF16") { t.dtype = Stored::BF16; elem = 2; }
            else if (dt->string == "F16") { t.dtype = Stored::F16; elem = 2; }
            else if (dt->string == "F32") { t.dtype = Stored::F32; elem = 4; }
            else if (dt->string == "I32") { t.dtype = Stored::I32; elem = 4; }
            else if (dt->string == "I64") { t.dtype = Stored::I64; elem = 8; }
            else throw SafetensorsError("tensor '" + name + "': Unsupported dtype " + dt->string);
            const json::Value* shape = meta.find("shape");
            if (!shape || !shape->is_array() || shape->array.empty())
                throw SafetensorsError("tensor '" + name + "': missing or empty shape (scalars are not supported)");
            for (auto& s : shape->array) {
                if (!s.is_number() || !s.is_integer || s.integer <= 0)
                    throw SafetensorsError("tensor '" + name + "': bad dimension in shape " + shape_text(*shape));
                t.shape.push_back(s.integer);
            }
            const json::Value* offs = meta.find("data_offsets");
            if (!offs || !offs->is_array() || offs->array.size() != 2 || !offs->array[0].is_integer || !offs->array[1].is_integer ||
                offs->array[0].integer < 0 || offs->array[1].integer < offs->array[0].integer)
                throw SafetensorsError("tensor '" + name + "': bad data_offsets");
            const size_t lo = (size_t)offs->array[0].integer, hi = (size_t)offs->array[1].integer;
            if (base + hi > size_) throw SafetensorsError("tensor '" + name + "': data runs past the end of the file");
            if (hi - lo != (size_t)t.numel() * elem)
                throw SafetensorsError("tensor '" + name + "': " + std::to_string(hi - lo) + " bytes stored, shape " + shape_text(*shape) +
                                       " of " + dt->string + " needs " + std::to_string((size_t)t.numel() * elem));
            t.data = map_ + base + lo;
            t.bytes = hi - lo;
            entries_.emplace(name, std::move(t));
        }
    }

    std::string path_;
    int fd_ = -1;
    size_t size_ = 0;
    const unsigned char* map_ = nullptr;
    std::map<std::string, StoredTensor> entries_;
};

// What a part asks of the file: a name and every shape it accepts (the first is the canonical one).
struct TensorRequest {
    std::string name;
    std::vector<std::vector<long long>> shapes;
    bool optional = false;
    static TensorRequest matrix(const std::string& name, long long rows, long long cols) { return {name, {{rows, cols}}, false}; }
    // a [n, 1] vector is accepted like [n] (src/models/model_param_validation.cpp:62-74)
    static TensorRequest vector(const std::string& name, long long n) { return {name, {{n}, {n, 1}}, false}; }
};

inline std::string shape_list(const std::vector<long long>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); ++i) out += (i ? ", " : "") + std::to_string(s[i]);
    return out + "]";
}

// One WeightError for everything that is wrong: missing, unexpected, wrong shapes.
inline void check_manifest(const std::vector<TensorRequest>& requests, const SafetensorsFile& file) {
    std::vector<std::string> missing, unexpected, wrong;
    std::set<std::string> wanted;
    for (auto& r : requests) {
        wanted.insert(r.name);
        const StoredTensor* t = file.find(r.name);
        if (!t) {
            if (!r.optional) missing.push_back(r.name);
            continue;
        }
        if (std::find(r.shapes.begin(), r.shapes.end(), t->shape) == r.shapes.end()) {
            std::string expected;
            for (size_t i = 0; i < r.shapes.size(); ++i) expected += (i ? " or " : "") + shape_list(r.shapes[i]);
            wrong.push_back("Invalid tensor shape for key '" + r.name + "': expected " + expected + ", got " + shape_list(t->shape));
        }
    }
    for (auto& kv : file.entries())
        if (!wanted.count(kv.first)) unexpected.push_back(kv.first);
    if (missing.empty() && unexpected.empty() && wrong.empty()) return;
    auto join = [](const std::vector<std::string>& v) {
        std::string s;
        for (size_t i = 0; i < v.size(); ++i) s += (i ? ", " : "") + v[i];
        return s;
    };
    std::vector<std::string> lines;
    if (!missing.empty()) lines.push_back("Missing required model weights: " + join(missing));
    if (!unexpected.empty()) lines.push_back("Unexpected tensors in the file: " + join(unexpected));
    for (auto& w : wrong) lines.push_back(w);
    std::string msg;
    for (size_t i = 0; i < lines.size(); ++i) msg += (i ? "\n" : "") + lines[i];
    throw WeightError(msg);
}

}  // namespace easygpt::engine
