// Architectures: the registry from an architecture's name to its model, and the one architecture the engine
// ships, the Qwen2 / Qwen2.5 dense decoder.
//
// The lookup rule is the reference's (src/models/layer_key_prefix.cpp:24-28, 92-105): lower-case
// architectures[0] and model_type; an entry matches if its key occurs in the architecture string or equals the
// model type; no match raises an error naming both strings.  An entry turns the config.json object into a
// ModelSpec; loader, cache manager, step function, scheduler and replay need nothing else.
#pragma once
#include <algorithm>
#include <cctype>
#include <functional>
#include <map>

#include "json.hpp"
#include "spec.hpp"

namespace easygpt::engine {

struct ConfigError : std::invalid_argument {
    using std::invalid_argument::invalid_argument;
};

struct ArchitectureRegistry {
    using Builder = std::function<ModelSpec(const json::Value&)>;
    std::vector<std::pair<std::string, Builder>> entries;      // in the order of registration
    static ArchitectureRegistry& instance() {
        static ArchitectureRegistry r;
        return r;
    }
    void add(std::string key, Builder b) {
        std::transform(key.begin(), key.end(), key.begin(), [](unsigned char c) { return (char)std::tolower(c); });
        for (auto& e : entries)
            if (e.first == key) { e.second = std::move(b); return; }
        entries.emplace_back(std::move(key), std::move(b));
    }
    ModelSpec build(const json::Value& config) const {
        std::string arch, model_type;
        if (const json::Value* a = config.find("architectures"))
            if (a->is_array() && !a->array.empty() && a->array[0].is_string()) arch = a->array[0].string;
        if (const json::Value* m = config.find("model_type"))
            if (m->is_string()) model_type = m->string;
        auto lower = [](std::string s) {
            std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
            return s;
        };
        const std::string la = lower(arch), lm = lower(model_type);
        for (auto& e : entries)
            if (la.find(e.first) != std::string::npos || lm == e.first) {
                ModelSpec spec = e.second(config);
                spec.validate();
                return spec;
            }
        throw std::invalid_argument("Unsupported model architecture/model_type: architecture='" + arch + "', model_type='" + model_type + "'");
    }
};

// ---- Qwen2 / Qwen2.5 -------------------------------------------------------------------------------------------------
// Typed configuration read from the keys of its own config.json.  The reference reads eleven keys
// (src/config.cpp:16-31) and takes the rest from the shapes of the weights or from constants in its code (eps 1e-6 at
// src/models/norm.cpp:41, head size at src/models/self_attn.cpp:169-174, intermediate size at
// src/models/model_param_validation.cpp:167-194).  Here every one of those is a key with the default the reference's
// constant implies.
struct Qwen2Config {
    long long vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, head_dim,
        max_position_embeddings, max_window_layers, sliding_window = -1, bos_token_id = -1, eos_token_id = -1;
    double rope_theta, rms_norm_eps;
    bool tie_word_embeddings, attention_bias, attention_out_bias, mlp_bias, use_sliding_window;
    std::string hidden_act, architecture, model_type;

    static long long integer(const json::Value& d, const std::string& key) {
        const json::Value* v = d.find(key);
        if (!v || !v->is_number() || !v->is_integer) throw ConfigError(key + " must be an integer");
        return v->integer;
    }
    static bool boolean(const json::Value& d, const std::string& key, bool fallback) {
        const json::Value* v = d.find(key);
        if (!v || v->is_null()) return fallback;
        if (v->is_bool()) return v->boolean;
        if (v->is_number()) return v->number != 0;
        throw ConfigError(key + " must be true or false");
    }
    static Qwen2Config from_json(const json::Value& d) {
        if (!d.is_object()) throw ConfigError("config.json is not a JSON object");
        std::string missing;
        for (const char* k : {"vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                              "rope_theta", "max_position_embeddings"}) {
            const json::Value* v = d.find(k);
            if (!v || v->is_null()) missing += (missing.empty() ? "" : ", ") + std::string(k);
        }
        if (!missing.empty()) throw ConfigError("config.json lacks: " + missing);
        Qwen2Config c;
        c.num_attention_heads = integer(d, "num_attention_heads");
        c.hidden_size = integer(d, "hidden_size");
        if (c.num_attention_heads <= 0 || c.hidden_size <= 0) throw ConfigError("hidden_size and num_attention_heads must be > 0");
        const json::Value* hd = d.find("head_dim");
        if (hd && !hd->is_null()) c.head_dim = integer(d, "head_dim");
        else {
            if (c.hidden_size % c.num_attention_heads)      // src/models/model_param_validation.cpp:94-97
                throw ConfigError("hidden_size must be divisible by num_attention_heads when head_dim is not given");
            c.head_dim = c.hidden_size / c.num_attention_heads;
        }
        c.vocab_size = integer(d, "vocab_size");
        c.intermediate_size = integer(d, "intermediate_size");
        c.num_hidden_layers = integer(d, "num_hidden_layers");
        c.num_key_value_heads = integer(d, "num_key_value_heads");
        c.max_position_embeddings = integer(d, "max_position_embeddings");
        const json::Value* theta = d.find("rope_theta");
        if (!theta->is_number()) throw ConfigError("rope_theta must be a number");
        c.rope_theta = theta->number;
        const json::Value* eps = d.find("rms_norm_eps");
        c.rms_norm_eps = (eps && eps->is_number()) ? eps->number : 1e-6;
        c.tie_word_embeddings = boolean(d, "tie_word_embeddings", false);
        c.attention_bias = boolean(d, "attention_bias", true);
        c.attention_out_bias = boolean(d, "attention_out_bias", false);
        c.mlp_bias = boolean(d, "mlp_bias", false);
        const json::Value* act = d.find("hidden_act");
        c.hidden_act = (act && act->is_string()) ? act->string : "silu";
        c.use_sliding_window = boolean(d, "use_sliding_window", false);
        const json::Value* sw = d.find("sliding_window");
        bool window_ok = false;
        if (sw && sw->is_number() && sw->is_integer && sw->integer > 0) { c.sliding_window = sw->integer; window_ok = true; }
        const json::Value* mwl = d.find("max_window_layers");
        c.max_window_layers = (mwl && !mwl->is_null()) ? integer(d, "max_window_layers") : c.num_hidden_layers;
        const json::Value* bos = d.find("bos_token_id");
        c.bos_token_id = (bos && !bos->is_null()) ? integer(d, "bos_token_id") : -1;
        const json::Value* eos = d.find("eos_token_id");
        if (eos && eos->is_array()) c.eos_token_id = (!eos->array.empty() && eos->array[0].is_integer) ? eos->array[0].integer : -1;
        else c.eos_token_id = (eos && !eos->is_null()) ? integer(d, "eos_token_id") : -1;
        if (const json::Value* a = d.find("architectures"))
            if (a->is_array() && !a->array.empty() && a->array[0].is_string()) c.architecture = a->array[0].string;      // src/config.cpp:26-31
        if (const json::Value* m = d.find("model_type"))
            if (m->is_string()) c.model_type = m->string;
        // what cannot run is refused
        auto positive = [](long long v, const char* key) {
            if (v <= 0) throw ConfigError(std::string(key) + " must be > 0, got " + std::to_string(v));
        };
        positive(c.vocab_size, "vocab_size");
        positive(c.intermediate_size, "intermediate_size");
        positive(c.num_hidden_layers, "num_hidden_layers");
        positive(c.num_key_value_heads, "num_key_value_heads");
        positive(c.head_dim, "head_dim");
        positive(c.max_position_embeddings, "max_position_embeddings");
        if (c.num_attention_heads % c.num_key_value_heads)       // src/cuda/ops/self_attn.cu:216-218
            throw ConfigError("num_attention_heads (" + std::to_string(c.num_attention_heads) + ") must be a multiple of num_key_value_heads (" +
                              std::to_string(c.num_key_value_heads) + ")");
        if (c.head_dim % 2) throw ConfigError("head_dim must be even for the half rotation");       // src/ops.cpp:155-157
        if (c.rope_theta <= 0.0) throw ConfigError("rope_theta must be > 0");                        // src/ops.cpp:158-160
        if (c.rms_norm_eps <= 0.0) throw ConfigError("rms_norm_eps must be > 0");
        if (c.hidden_act != "silu") throw ConfigError("hidden_act '" + c.hidden_act + "' is not supported (silu only)");
        if (const json::Value* rs = d.find("rope_scaling"))
            if (!rs->is_null() && !(rs->is_object() && rs->object.empty())) throw ConfigError("rope_scaling is not supported");
        if (c.use_sliding_window) {
            if (!window_ok) throw ConfigError("use_sliding_window needs a positive integer sliding_window");
            if (c.max_window_layers < 0) throw ConfigError("max_window_layers must be >= 0");
        }
        return c;
    }
    // layers from max_window_layers on see only the last sliding_window positions when use_sliding_window is set
    long long layer_window(long long layer) const { return (use_sliding_window && layer >= max_window_layers) ? sliding_window : -1; }
};

// Tensor names are the reference's (src/models/layer_key_prefix.cpp:77-87, src/models/embedding.cpp:30) plus
// lm_head.weight for an untied head, which the reference never consumes (src/models/gpt_model.cpp:324-328).
inline ModelSpec qwen2_spec(const json::Value& config) {
    const Qwen2Config c = Qwen2Config::from_json(config);
    ModelSpec spec;
    spec.architecture = "qwen2";
    spec.vocab_size = c.vocab_size;
    spec.hidden_size = c.hidden_size;
    spec.max_positions = c.max_position_embeddings;
    spec.bos_token_id = c.bos_token_id;
    spec.eos_token_id = c.eos_token_id;
    auto norm = [&](const std::string& prefix) { return PartSpec{"rmsnorm", Params{{"size", c.hidden_size}, {"eps", c.rms_norm_eps}}, prefix, true}; };
    for (long long i = 0; i < c.num_hidden_layers; ++i) {
        const std::string prefix = "model.layers." + std::to_string(i);
        Params attention{{"hidden_size", c.hidden_size}, {"num_heads", c.num_attention_heads}, {"num_kv_heads", c.num_key_value_heads},
                         {"head_dim", c.head_dim}, {"qkv_bias", c.attention_bias}, {"out_bias", c.attention_out_bias}};
        if (c.layer_window(i) > 0) attention.set("window", c.layer_window(i));
        spec.layers.push_back(LayerSpec::pre_norm(
            PartSpec{"attention", attention, prefix + ".self_attn", true},
            PartSpec{"swiglu", Params{{"hidden_size", c.hidden_size}, {"intermediate_size", c.intermediate_size}, {"bias", c.mlp_bias}}, prefix + ".mlp", true},
            norm(prefix + ".input_layernorm"), norm(prefix + ".post_attention_layernorm"),
            PartSpec{"rope", Params{{"head_dim", c.head_dim}, {"rotary_dim", c.head_dim}, {"theta", c.rope_theta}}, "", true}));
        spec.run_order.push_back(RunEntry{(int)i, (int)i, true});
    }
    spec.embedding = PartSpec{"embedding", Params{{"vocab_size", c.vocab_size}, {"hidden_size", c.hidden_size}}, "model.embed_tokens", true};
    spec.final_norm = norm("model.norm");
    Params head{{"vocab_size", c.vocab_size}, {"hidden_size", c.hidden_size}};
    if (c.tie_word_embeddings) head.set("tied_to", "model.embed_tokens");
    spec.lm_head = PartSpec{"lm_head", head, "lm_head", true};
    return spec;
}

inline void register_builtin_architectures() {
    ArchitectureRegistry& r = ArchitectureRegistry::instance();
    for (auto& e : r.entries)
        if (e.first == "qwen2") return;
    r.add("qwen2", qwen2_spec);
}

}  // namespace easygpt::engine
