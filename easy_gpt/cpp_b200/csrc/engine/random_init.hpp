// Random-weights mode: writes a model folder (config.json, model.safetensors) from a configuration and a seed.
// Every tensor is drawn from its own counter-based stream keyed by (seed, tensor name), so a tensor's values do not
// depend on which other tensors exist or in which order they are written.  Matrices and biases are N(0, std) /
// N(0, bias_std); norm gains are 1 + N(0, gain_std) (exactly 1 when gain_std is 0); values are stored in bfloat16.
// (The reference has only unused debug constructors with an unseeded generator, src/utils.cpp:14-15,
// src/models/linear.cpp:15-24.)
#pragma once
#include <cmath>
#include <cstdio>
#include <fstream>

#include "model.hpp"

namespace easygpt::engine {

class NormalStream {
public:
    NormalStream(uint64_t seed, const std::string& name) {
        uint64_t h = 0xcbf29ce484222325ull ^ seed;                       // FNV-1a over the name, started from the seed
        for (unsigned char c : name) h = (h ^ c) * 0x100000001b3ull;
        state_ = h;
    }
    float next() {
        if (have_spare_) {
            have_spare_ = false;
            return spare_;
        }
        const double u1 = (double)((mix() >> 11) + 1) / 9007199254740993.0;     // (0, 1]
        const double u2 = (double)(mix() >> 11) / 9007199254740992.0;
        const double r = std::sqrt(-2.0 * std::log(u1)), a = 6.283185307179586 * u2;
        spare_ = (float)(r * std::sin(a));
        have_spare_ = true;
        return (float)(r * std::cos(a));
    }

private:
    uint64_t mix() {
        uint64_t z = (state_ += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    uint64_t state_;
    bool have_spare_ = false;
    float spare_ = 0.f;
};

inline bool ends_with(const std::string& s, const std::string& tail) { return s.size() >= tail.size() && s.compare(s.size() - tail.size(), tail.size(), tail) == 0; }

inline void write_random_model(const std::string& folder, const std::string& config_text, uint64_t seed, double std_dev = 0.02, double bias_std = -1.0,
                               double gain_std = 0.0) {
    register_builtin_architectures();
    const json::Value config = json::parse(config_text);
    Model model(ArchitectureRegistry::instance().build(config), DType::BF16);       // refuses a configuration that cannot be run
    if (bias_std < 0) bias_std = std_dev;
    const std::vector<TensorRequest> requests = model.tensor_requests();
    std::string header = "{";
    size_t offset = 0;
    for (size_t i = 0; i < requests.size(); ++i) {
        size_t n = 1;
        for (long long s : requests[i].shapes[0]) n *= (size_t)s;
        header += (i ? "," : "") + std::string("\"") + requests[i].name + "\":{\"dtype\":\"BF16\",\"shape\":" + shape_list(requests[i].shapes[0]) +
                  ",\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + 2 * n) + "]}";
        offset += 2 * n;
    }
    header += "}";
    while (header.size() % 8) header += ' ';
    {
        std::ofstream cfg(folder + "/config.json");
        if (!cfg) throw std::runtime_error("cannot write into " + folder);
        cfg << config_text;
    }
    std::ofstream out(folder + "/model.safetensors", std::ios::binary);
    if (!out) throw std::runtime_error("cannot write " + folder + "/model.safetensors");
    const uint64_t hlen = header.size();
    unsigned char len[8];
    for (int i = 0; i < 8; ++i) len[i] = (unsigned char)(hlen >> (8 * i));
    out.write((const char*)len, 8);
    out.write(header.data(), (std::streamsize)header.size());
    std::vector<uint16_t> values;
    for (auto& r : requests) {
        size_t n = 1;
        for (long long s : r.shapes[0]) n *= (size_t)s;
        values.resize(n);
        NormalStream g(seed, r.name);
        const bool vector = r.shapes[0].size() == 1;
        const bool gain = vector && ends_with(r.name, "norm.weight");
        for (size_t i = 0; i < n; ++i) {
            float v;
            if (gain) v = 1.0f + (gain_std > 0 ? (float)(g.next() * gain_std) : 0.0f);
            else v = (float)(g.next() * (vector ? bias_std : std_dev));
            values[i] = float_to_bf16(v);
        }
        out.write((const char*)values.data(), (std::streamsize)(n * 2));
    }
    if (!out) throw std::runtime_error("writing " + folder + "/model.safetensors failed");
}

}  // namespace easygpt::engine
