// The native engine's host-only parts from C++ alone (no GPU, no CUDA headers): the JSON reader, the safetensors
// reader with every malformed file refused, the one error that lists missing / unexpected / wrongly shaped tensors, the
// typed Qwen2 configuration with what cannot run refused, the architecture registry's rule, and the run order's checks.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>

#include "architectures.hpp"
#include "weights.hpp"

using namespace easygpt;
using namespace easygpt::engine;

static int failures = 0;
#define CHECK(cond)                                                                 \
    do {                                                                            \
        if (!(cond)) {                                                              \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);           \
            ++failures;                                                             \
        }                                                                           \
    } while (0)

template <class E> static bool throws(const std::function<void()>& f, const std::string& part) {
    try {
        f();
    } catch (const E& e) {
        if (std::string(e.what()).find(part) != std::string::npos) return true;
        std::printf("  message was: %s\n", e.what());
        return false;
    } catch (...) {
        return false;
    }
    return false;
}

static std::string safetensors_bytes(const std::string& header, const std::string& data) {
    std::string out(8, '\0');
    const uint64_t n = header.size();
    for (int i = 0; i < 8; ++i) out[i] = (char)(n >> (8 * i));
    return out + header + data;
}
static std::string write_file(const std::string& dir, const std::string& name, const std::string& bytes) {
    const std::string path = dir + "/" + name;
    std::ofstream(path, std::ios::binary).write(bytes.data(), (std::streamsize)bytes.size());
    return path;
}

static const char* kConfig = R"({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 3, "hidden_size": 80,
  "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 208, "vocab_size": 391, "rope_theta": 1000000.0,
  "rms_norm_eps": 1e-5, "tie_word_embeddings": false, "max_position_embeddings": 2048, "bos_token_id": null, "eos_token_id": [7, 9],
  "use_sliding_window": true, "sliding_window": 24, "max_window_layers": 1})";

// The configuration text with `key` dropped (value empty) or set to `value`.
static std::string with(const std::string& config, const std::string& key, const std::string& value) {
    std::string text = config;
    const std::string needle = "\"" + key + "\":";
    size_t at = text.find(needle);
    if (at != std::string::npos) {
        size_t end = at + needle.size();
        int depth = 0;
        while (end < text.size() && !((text[end] == ',' || text[end] == '}') && depth == 0)) {
            if (text[end] == '[') ++depth;
            if (text[end] == ']') --depth;
            ++end;
        }
        if (text[end] == ',') ++end;
        text.erase(at, end - at);
    }
    if (!value.empty()) {
        const size_t brace = text.rfind('}');
        std::string head = text.substr(0, brace);
        while (!head.empty() && (head.back() == ' ' || head.back() == '\n' || head.back() == ',')) head.pop_back();
        text = head + ", \"" + key + "\": " + value + "}";
    } else {
        const size_t brace = text.rfind('}');
        std::string head = text.substr(0, brace);
        while (!head.empty() && (head.back() == ' ' || head.back() == '\n' || head.back() == ',')) head.pop_back();
        text = head + "}";
    }
    return text;
}

int main(int argc, char** argv) {
    const std::string dir = argc > 1 ? argv[1] : ".";

    // ---- JSON ----------------------------------------------------------------------------------------------------
    {
        const json::Value v = json::parse(R"({"a": [1, 2.5, -3e2, true, null], "s": "x\né😀\"", "o": {"k": 12345678901234}})");
        CHECK(v.find("a")->array.size() == 5 && v.find("a")->array[0].is_integer && v.find("a")->array[0].integer == 1);
        CHECK(!v.find("a")->array[1].is_integer && v.find("a")->array[1].number == 2.5 && v.find("a")->array[2].number == -300.0);
        CHECK(v.find("a")->array[3].boolean && v.find("a")->array[4].is_null());
        CHECK(v.find("s")->string == "x\n\xc3\xa9\xf0\x9f\x98\x80\"");
        CHECK(v.find("o")->find("k")->integer == 12345678901234LL && v.object[0].first == "a" && !v.contains("missing"));
        CHECK(throws<json::ParseError>([] { json::parse("{\"a\": }"); }, "byte"));
        CHECK(throws<json::ParseError>([] { json::parse("[1, 2] x"); }, "after the JSON value"));
        CHECK(throws<json::ParseError>([] { json::parse("\"abc"); }, "unterminated"));
    }

    // ---- safetensors: what is malformed is refused (src/models/loader.cpp:79-140, 214-252) ------------------------------
    {
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(dir + "/nowhere.safetensors"); }, "cannot open"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "short", "abc")); }, "smaller than the 8-byte"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "long", std::string("\xff\xff\0\0\0\0\0\0", 8) + "{}")); }, "exceeds the file size"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "nojson", safetensors_bytes("{not json", ""))); }, "not JSON"));
        CHECK(throws<SafetensorsError>([&] { SafetensorsFile f(write_file(dir, "array", safetensors_bytes("[1]", ""))); }, "not a JSON object"));
        auto one = [&](const std::string& meta, const std::string& data = std::string(8, '\0')) {
            return [=] { SafetensorsFile f(write_file(dir, "one", safetensors_bytes("{\"t\": " + meta + "}", data))); };
        };
        CHECK(throws<SafetensorsError>(one(R"({"shape": [2], "data_offsets": [0, 8]})"), "missing dtype"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F64", "shape": [1], "data_offsets": [0, 8]})"), "Unsupported dtype F64"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [], "data_offsets": [0, 8]})"), "empty shape"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2, 0], "data_offsets": [0, 8]})"), "bad dimension"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2.5], "data_offsets": [0, 8]})"), "bad dimension"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2], "data_offsets": [8, 0]})"), "bad data_offsets"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [2], "data_offsets": [0, 16]})"), "past the end"));
        CHECK(throws<SafetensorsError>(one(R"({"dtype": "F32", "shape": [3], "data_offsets": [0, 8]})"), "8 bytes stored"));
        // a good file: F32, BF16 and F16 values read as float32; __metadata__ skipped
        const float f32[2] = {1.5f, -2.0f};
        const uint16_t bf[2] = {0x3fc0, 0xc000}, fh[3] = {0x3e00, 0xc000, 0x0001};
        std::string data((const char*)f32, 8);
        data += std::string((const char*)bf, 4) + std::string((const char*)fh, 6);
        SafetensorsFile good(write_file(dir, "good", safetensors_bytes(
            R"({"__metadata__": {"format": "pt"}, "a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},)"
            R"( "b": {"dtype": "BF16", "shape": [2, 1], "data_offsets": [8, 12]}, "c": {"dtype": "F16", "shape": [3], "data_offsets": [12, 18]}})", data)));
        CHECK(good.entries().size() == 3 && !good.find("__metadata__"));
        float out[3];
        good.find("a")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f);
        good.find("b")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f && good.find("b")->shape.size() == 2);
        good.find("c")->to_float(out);
        CHECK(out[0] == 1.5f && out[1] == -2.0f && out[2] > 0 && out[2] < 1e-7f);
        CHECK(float_to_bf16(1.5f) == 0x3fc0 && float_to_bf16(1.00390625f) == 0x3f80 && float_to_bf16(1.01171875f) == 0x3f82);      // ties to even
        // one error for everything: missing, unexpected, wrong shape; [n, 1] accepted like [n]
        std::vector<TensorRequest> wanted = {TensorRequest::vector("a", 2), TensorRequest::vector("b", 2), TensorRequest::matrix("c", 3, 1),
                                             TensorRequest::matrix("d", 4, 4), TensorRequest::vector("e", 4)};
        CHECK(throws<WeightError>([&] { check_manifest(wanted, good); }, "Missing required model weights: d, e"));
        CHECK(throws<WeightError>([&] { check_manifest(wanted, good); }, "Invalid tensor shape for key 'c': expected [3, 1], got [3]"));
        CHECK(throws<WeightError>([&] { check_manifest({TensorRequest::vector("a", 2)}, good); }, "Unexpected tensors in the file: b, c"));
        check_manifest({TensorRequest::vector("a", 2), TensorRequest::vector("b", 2), TensorRequest::vector("c", 3)}, good);
    }

    // ---- the typed configuration and the registry ------------------------------------------------------------------------
    {
        register_builtin_architectures();
        const ModelSpec spec = ArchitectureRegistry::instance().build(json::parse(kConfig));
        CHECK(spec.architecture == "qwen2" && spec.layers.size() == 3 && spec.run_order.size() == 3 && spec.vocab_size == 391);
        CHECK(spec.eos_token_id == 7 && spec.bos_token_id == -1 && spec.max_positions == 2048);
        const SubLayerSpec& mixer = spec.layers[1].sublayers[0];
        CHECK(mixer.role == "mixer" && mixer.part.kind == "attention" && mixer.part.params.integer("window") == 24 &&
              mixer.part.params.integer("head_dim") == 32 && mixer.part.prefix == "model.layers.1.self_attn");       // src/models/layer_key_prefix.cpp:77-87
        CHECK(!spec.layers[0].sublayers[0].part.params.has("window"));                                                // windows from layer 1 on
        CHECK(spec.layers[1].sublayers[1].part.kind == "swiglu" && spec.layers[1].sublayers[1].part.params.integer("intermediate_size") == 208);
        CHECK(mixer.norm.params.real("eps") == 1e-5 && spec.layers[1].position.params.real("theta") == 1e6);
        CHECK(!spec.lm_head.params.has("tied_to") && spec.lm_head.prefix == "lm_head");
        const ModelSpec tied = ArchitectureRegistry::instance().build(json::parse(with(kConfig, "tie_word_embeddings", "true")));
        CHECK(tied.lm_head.params.text("tied_to") == "model.embed_tokens");
        // the reference's rule: the key occurs in architectures[0], or equals model_type (src/models/layer_key_prefix.cpp:92-105)
        ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", "[\"MyQwen2Thing\"]"), "model_type", "\"other\"")));
        ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", ""), "model_type", "\"QWEN2\"")));
        CHECK(throws<std::invalid_argument>([&] {
            ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "architectures", "[\"LlamaForCausalLM\"]"), "model_type", "\"llama\"")));
        }, "Unsupported model architecture/model_type: architecture='LlamaForCausalLM', model_type='llama'"));
        auto refuse = [&](const std::string& key, const std::string& value, const std::string& message) {
            const bool ok = throws<ConfigError>([&] { ArchitectureRegistry::instance().build(json::parse(with(kConfig, key, value))); }, message);
            if (!ok) std::printf("  (%s = %s)\n", key.c_str(), value.c_str());
            return ok;
        };
        CHECK(refuse("vocab_size", "", "config.json lacks: vocab_size"));
        CHECK(refuse("hidden_size", "\"80\"", "hidden_size must be an integer"));
        CHECK(refuse("num_key_value_heads", "4", "must be a multiple of num_key_value_heads"));
        CHECK(refuse("head_dim", "31", "head_dim must be even"));
        CHECK(refuse("rope_theta", "0", "rope_theta must be > 0"));
        CHECK(refuse("rms_norm_eps", "0", "rms_norm_eps must be > 0"));
        CHECK(refuse("hidden_act", "\"gelu\"", "is not supported (silu only)"));
        CHECK(refuse("rope_scaling", "{\"type\": \"yarn\"}", "rope_scaling is not supported"));
        CHECK(refuse("sliding_window", "null", "needs a positive integer sliding_window"));
        CHECK(refuse("num_hidden_layers", "0", "num_hidden_layers must be > 0"));
        const ModelSpec derived = ArchitectureRegistry::instance().build(json::parse(with(with(kConfig, "head_dim", ""), "num_attention_heads", "4")));
        CHECK(derived.layers[0].sublayers[0].part.params.integer("head_dim") == 20);                               // hidden / heads when no key
        CHECK(refuse("head_dim", "", "hidden_size must be divisible by num_attention_heads"));                       // 80 / 6
        // the run order is data and is checked
        ModelSpec bad = spec;
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{5, 1, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "names layer 5"));
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{1, 0, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "is written by run entries 0 and 1"));
        bad.run_order = {RunEntry{0, 1, false}, RunEntry{1, 1, true}};
        CHECK(throws<std::invalid_argument>([&] { bad.validate(); }, "before entry 1 has written it"));
        bad.run_order = {RunEntry{0, 0, true}, RunEntry{1, 1, true}, RunEntry{0, 2, true}, RunEntry{1, 1, false}};
        bad.validate();                                                                                             // a layer twice, a shared cache: fine
    }

    if (failures) {
        std::printf("%d checks failed\n", failures);
        return 1;
    }
    std::printf("native engine, host side: all checks passed\n");
    return 0;
}
