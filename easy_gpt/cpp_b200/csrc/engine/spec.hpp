// What a model is made of, as data: a list of layers, each naming its sub-layers (mixer, feed-forward,
// their norms and where these stand) and its position encoding by *kind* with every size and constant as a
// parameter, and a run order that may name a layer twice or let a layer read another layer's cache.
// An architecture's builder turns its typed configuration into a ModelSpec; nothing below knows which
// model it is in.
#pragma once
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace easygpt::engine {

// One parameter of a part: an integer, a real number, a switch, a string, or nothing (null).
struct Param {
    enum Type { Null, Int, Real, Bool, Str } type = Null;
    int64_t i = 0;
    double r = 0.0;
    bool b = false;
    std::string s;
    Param() = default;
    Param(int v) : type(Int), i(v), r((double)v) {}
    Param(long long v) : type(Int), i(v), r((double)v) {}
    Param(double v) : type(Real), r(v) {}
    Param(bool v) : type(Bool), b(v) {}
    Param(const char* v) : type(Str), s(v) {}
    Param(const std::string& v) : type(Str), s(v) {}
    static Param null() { return Param(); }
};

class Params {
public:
    Params() = default;
    Params(std::initializer_list<std::pair<const std::string, Param>> init) : map_(init) {}
    void set(const std::string& key, Param value) { map_[key] = std::move(value); }
    bool has(const std::string& key) const {
        auto it = map_.find(key);
        return it != map_.end() && it->second.type != Param::Null;
    }
    long long integer(const std::string& key) const {
        const Param& p = need(key);
        if (p.type != Param::Int) throw std::invalid_argument("parameter '" + key + "' must be an integer");
        return p.i;
    }
    long long integer(const std::string& key, long long fallback) const { return has(key) ? integer(key) : fallback; }
    double real(const std::string& key) const {
        const Param& p = need(key);
        if (p.type != Param::Int && p.type != Param::Real) throw std::invalid_argument("parameter '" + key + "' must be a number");
        return p.r;
    }
    bool flag(const std::string& key, bool fallback) const {
        if (!has(key)) return fallback;
        const Param& p = map_.at(key);
        if (p.type != Param::Bool) throw std::invalid_argument("parameter '" + key + "' must be true or false");
        return p.b;
    }
    std::string text(const std::string& key, const std::string& fallback = "") const {
        if (!has(key)) return fallback;
        const Param& p = map_.at(key);
        if (p.type != Param::Str) throw std::invalid_argument("parameter '" + key + "' must be a string");
        return p.s;
    }

private:
    const Param& need(const std::string& key) const {
        auto it = map_.find(key);
        if (it == map_.end() || it->second.type == Param::Null) throw std::invalid_argument("a part lacks its parameter '" + key + "'");
        return it->second;
    }
    std::map<std::string, Param> map_;
};

// One part: `kind` selects the factory from the part registry, `params` are its sizes, constants and
// switches, `prefix` is the tensor-name prefix its weights live under.
struct PartSpec {
    std::string kind;
    Params params;
    std::string prefix;
    bool present = true;
    static PartSpec none() {
        PartSpec p;
        p.present = false;
        return p;
    }
};

// One residual sub-layer.  With x the residual stream and f the part:
//   norm present, placement "pre":   x = x + f(norm(x))
//   norm present, placement "post":  x = norm(x + f(x))
//   no norm:                         x = x + f(x)
//   output_norm present as well:     x = x + output_norm(f(norm(x)))
struct SubLayerSpec {
    std::string role;                   // "mixer" or "feed_forward"
    PartSpec part;
    PartSpec norm = PartSpec::none();
    std::string norm_placement = "pre";
    PartSpec output_norm = PartSpec::none();
};

struct LayerSpec {
    std::vector<SubLayerSpec> sublayers;
    PartSpec position = PartSpec::none();     // handed to the layer's mixer

    // the common block x += mixer(norm1(x)); x += feed_forward(norm2(x))
    static LayerSpec pre_norm(PartSpec mixer, PartSpec feed_forward, PartSpec mixer_norm, PartSpec feed_forward_norm, PartSpec position) {
        LayerSpec l;
        l.sublayers.push_back({"mixer", std::move(mixer), std::move(mixer_norm), "pre", PartSpec::none()});
        l.sublayers.push_back({"feed_forward", std::move(feed_forward), std::move(feed_forward_norm), "pre", PartSpec::none()});
        l.position = std::move(position);
        return l;
    }
};

// One line of the run order: `layer` indexes ModelSpec::layers (a layer may be named more than once: its
// weights are shared); entries with the same `cache` share it and only the one with writes_cache appends.
struct RunEntry {
    int layer;
    int cache;
    bool writes_cache = true;
};

struct ModelSpec {
    std::string architecture;
    long long vocab_size = 0, hidden_size = 0, max_positions = 0;
    std::vector<LayerSpec> layers;
    std::vector<RunEntry> run_order;
    PartSpec embedding, final_norm, lm_head;
    PartSpec embedding_position = PartSpec::none();
    long long bos_token_id = -1, eos_token_id = -1;

    void validate() const {
        std::map<int, int> owner;
        for (size_t i = 0; i < run_order.size(); ++i) {
            const RunEntry& e = run_order[i];
            if (e.layer < 0 || e.layer >= (int)layers.size())
                throw std::invalid_argument("run order entry " + std::to_string(i) + " names layer " + std::to_string(e.layer) + ", but there are " +
                                            std::to_string(layers.size()) + " layers");
            if (e.writes_cache) {
                if (owner.count(e.cache))
                    throw std::invalid_argument("cache " + std::to_string(e.cache) + " is written by run entries " + std::to_string(owner[e.cache]) +
                                                " and " + std::to_string(i));
                owner[e.cache] = (int)i;
            }
        }
        for (size_t i = 0; i < run_order.size(); ++i) {
            const RunEntry& e = run_order[i];
            if (!owner.count(e.cache)) throw std::invalid_argument("run entry " + std::to_string(i) + " reads cache " + std::to_string(e.cache) + ", which no entry writes");
            if (owner[e.cache] > (int)i)
                throw std::invalid_argument("run entry " + std::to_string(i) + " reads cache " + std::to_string(e.cache) + " before entry " +
                                            std::to_string(owner[e.cache]) + " has written it");
        }
        for (auto& l : layers) {
            int mixers = 0;
            if (l.sublayers.empty()) throw std::invalid_argument("a layer needs at least one sub-layer");
            for (auto& s : l.sublayers) {
                if (s.role != "mixer" && s.role != "feed_forward") throw std::invalid_argument("a sub-layer's role is 'mixer' or 'feed_forward', not '" + s.role + "'");
                if (s.norm_placement != "pre" && s.norm_placement != "post") throw std::invalid_argument("norm_placement is 'pre' or 'post'");
                mixers += s.role == "mixer";
            }
            if (mixers > 1) throw std::invalid_argument("a layer has at most one mixer");
        }
    }
};

}  // namespace easygpt::engine
