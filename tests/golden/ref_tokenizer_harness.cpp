// Drives the reference's own tokenizer (MarsPain/easy_gpt.cpp: Tokenizer over Bpe, src/tokenizer.cpp,
// src/bpe.cpp) and writes what it makes of given texts.  Built and run only by
// tests/golden/make_golden.py; nothing in the product or in the test suite compiles it.
//
// usage: ref_tokenizer_harness <tokenizer.json> <tokenizer_config.json> <texts.json> <out.json>
// texts.json: a JSON array of strings.  out.json: for each text {"tokens": [...], "ids": [...]}.
#include <fstream>
#include <string>
#include <vector>

#include "spdlog/spdlog.h"
#include "json.hpp"
#include "config.hpp"
#include "tokenizer.hpp"

using namespace easy_llm;

int main(int argc, char** argv) {
    if (argc != 5) return 2;
    spdlog::set_level(spdlog::level::err);
    Config cfg;
    cfg.tokenizer_path = argv[1];
    cfg.tokenizer_config_path = argv[2];
    cfg.bos_token_id = -1;
    auto tokenizer = Tokenizer::create(cfg);
    nlohmann::json texts;
    std::ifstream(argv[3]) >> texts;
    nlohmann::json out = nlohmann::json::array();
    for (const auto& t : texts) {
        const std::string text = t.get<std::string>();
        const std::vector<std::string> tokens = tokenizer->tokenize(text);
        out.push_back({{"tokens", tokens}, {"ids", tokenizer->tokens_to_ids(tokens)}});
    }
    std::ofstream(argv[4]) << out.dump();
    return 0;
}
