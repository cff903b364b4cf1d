// Drives the reference's own CPU model code (MarsPain/easy_gpt.cpp, compiled in
// true 32-bit with -DUSE_FP32) through its public classes and dumps logits.
// Built and run only by tests/golden/make_golden.py; nothing in the product or
// in the test suite compiles it.
//
// usage: ref_harness <model.safetensors> <script.txt> <out.f32> L NH NKV H V theta
// script: one call per line:  n  (id offset ntok tok...){n}
//   - every sample of a call has the same ntok (the reference's batches are rectangular)
// The sequence of calls mirrors GptModel::forward_logits (src/models/gpt_model.cpp:310-333).
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "spdlog/spdlog.h"
#include "config.hpp"
#include "models/block.hpp"
#include "models/embedding.hpp"
#include "models/layer_key_prefix.hpp"
#include "models/loader.hpp"
#include "models/model_param_validation.hpp"
#include "models/norm.hpp"

using namespace easy_llm;

int main(int argc, char** argv) {
    if (argc != 10) {
        std::fprintf(stderr, "bad arguments\n");
        return 2;
    }
    spdlog::set_level(spdlog::level::warn);
    Config cfg;
    cfg.num_layers = std::atoi(argv[4]);
    cfg.num_heads = std::atoi(argv[5]);
    cfg.num_heads_kv = std::atoi(argv[6]);
    cfg.hidden_size = std::atoi(argv[7]);
    cfg.vocab_size = std::atoi(argv[8]);
    cfg.rope_theta = static_cast<float>(std::atof(argv[9]));
    cfg.architecture = "Qwen2ForCausalLM";
    cfg.model_type = "qwen2";

    auto params = ModelParam::load(argv[1]);
    auto names = create_layer_key_prefix(cfg);
    validate_model_params_before_load(cfg, *names, *params);
    Embedding embedding;
    embedding.load_param(*params);
    std::vector<std::unique_ptr<Block>> blocks;
    for (int i = 0; i < cfg.num_layers; ++i) {
        blocks.emplace_back(std::make_unique<Block>(cfg));
        blocks.back()->load_param(*names, names->layer(i), *params);
    }
    RMSNorm final_norm;
    final_norm.load_param(names->model_norm(), *params);
    for (auto& b : blocks) {
        b->init_kv_cache(8);
    }

    std::ifstream script(argv[2]);
    std::ofstream out(argv[3], std::ios::binary);
    std::string line;
    while (std::getline(script, line)) {
        if (line.empty()) continue;
        std::istringstream in(line);
        int n = 0;
        in >> n;
        std::vector<int> ids(n), offsets(n);
        std::vector<std::vector<int>> tokens(n);
        for (int s = 0; s < n; ++s) {
            int ntok = 0;
            in >> ids[s] >> offsets[s] >> ntok;
            tokens[s].resize(ntok);
            for (int t = 0; t < ntok; ++t) in >> tokens[s][t];
        }
        Tensor x = embedding.forward(tokens);
        for (auto& b : blocks) x = b->forward(x, ids, &offsets);
        x = final_norm.forward(x);
        x = embedding.forward(x);
        std::vector<float> row(x.size());
        for (int i = 0; i < x.size(); ++i) row[i] = static_cast<float>(x[i]);
        out.write(reinterpret_cast<const char*>(row.data()), static_cast<std::streamsize>(row.size() * sizeof(float)));
    }
    return 0;
}
