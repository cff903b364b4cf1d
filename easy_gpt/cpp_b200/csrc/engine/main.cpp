// easy_llm: generate from the command line, in the reference's manner (src/main.cpp:24-125, src/cli_options.cpp): the same
// option names, meanings, defaults, checks and error texts where the reference has them, plus the options this engine
// adds (a model folder instead of a fixed path, token-id prompts, cache and batch sizes).  --serve and its options are
// not provided: no server is built here.  Text prompts go through the reference's whitespace-split byte-level BPE
// (csrc/host/bpe_tokenizer.hpp) and the fixed Qwen chat template.  Everything between the model folder and the
// generated tokens is this program and the kernel library; no interpreter is involved.
#include <sys/stat.h>

#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>

#include "../host/bpe_tokenizer.hpp"
#include "engine.hpp"
#include "random_init.hpp"

using namespace easygpt::engine;
namespace host = easygpt::host;

namespace {

const char* kUsage =
    "Usage: easy_llm [--model <dir>] [--prompt-file <path>] [--max-steps <n>]\n"
    "                [--temperature <float>] [--top-p <float>] [--top-k <int>] [--seed <int>] [--greedy]\n"
    "                [--token-ids] [--dtype <bfloat16|float32>] [\"prompt\"]\n"
    "  -f, --prompt-file <path>  Read prompts from file (one per line, ignore empty lines)\n"
    "  -m, --max-steps <n>        Maximum generation steps per request (default: 100)\n"
    "      --temperature <float> Sampling temperature (default: 0.8)\n"
    "      --top-p <float>        Nucleus sampling cutoff in (0,1] (default: 0.95)\n"
    "      --top-k <int>          Top-K sampling cutoff, 0 disables (default: 20)\n"
    "      --seed <int>           RNG seed for sampling (default: 42)\n"
    "      --greedy               Use greedy decoding (override sampling)\n"
    "      --model <dir>          Folder with config.json and model.safetensors (default: data/model)\n"
    "      --dtype <name>         bfloat16 (default) or float32 (true 32-bit everywhere)\n"
    "      --token-ids            Prompts are lists of token ids (\"5 17 3\" or \"5,17,3\"); outputs are ids too\n"
    "      --random-weights <seed> Write random weights for --config into --model first\n"
    "      --config <path>        config.json to use with --random-weights\n"
    "      --page-size <n>        Tokens per cache page (default: 16)\n"
    "      --cache-tokens <n>     Tokens the cache pool holds (default: max-active x 4096)\n"
    "      --max-active <n>       Max concurrent requests (default: 16)\n"
    "      --prefill-batch <n>    Max requests admitted per step (default: 4)\n"
    "      --max-batch-tokens <n> Token budget of one step (default: 2048)\n"
    "      --chunk-size <n>       Longest portion of a prompt in one step (default: 512)\n"
    "      --no-chat-template     Do not wrap text prompts in the chat template\n"
    "  -h, --help                Show this help message\n"
    "Examples:\n"
    "  easy_llm --model data/model --max-steps 128 \"Hello\"\n"
    "  easy_llm --model m --token-ids --greedy \"5 17 3\"\n"
    "  easy_llm --model m -f prompts.txt\n";

struct CliOptions {
    std::string prompt_file, prompt, model = "data/model", dtype = "bfloat16", config;
    long long max_steps = 100, top_k = 20, seed = 42, random_weights = -1, page_size = 16, cache_tokens = 0, max_active = 16, prefill_batch = 4,
              max_batch_tokens = 2048, chunk_size = 512;
    double temperature = 0.8, top_p = 0.95;
    bool use_greedy = false, show_help = false, token_ids = false, chat_template = true;
};

bool whole_integer(const std::string& text, long long* out) {
    try {
        size_t used = 0;
        *out = std::stoll(text, &used);
        return used == text.size();
    } catch (...) {
        return false;
    }
}
bool whole_real(const std::string& text, double* out) {
    try {
        size_t used = 0;
        *out = std::stod(text, &used);
        return used == text.size();
    } catch (...) {
        return false;
    }
}

// Returns "" or the error text; error texts of the options the reference has are its own (src/cli_options.cpp:86-286).
std::string parse_args(int argc, char** argv, CliOptions* o) {
    struct IntOption { const char* flag; long long CliOptions::*field; const char* label; long long least; const char* complaint; };
    const IntOption ints[] = {
        {"--max-steps", &CliOptions::max_steps, "max steps", 1, "Max steps must be greater than 0"},
        {"-m", &CliOptions::max_steps, "max steps", 1, "Max steps must be greater than 0"},
        {"--top-k", &CliOptions::top_k, "top-k", 0, "Top-k must be >= 0"},
        {"--seed", &CliOptions::seed, "seed", 0, "Seed must be >= 0"},
        {"--random-weights", &CliOptions::random_weights, "random weights seed", 0, "random-weights seed must be >= 0"},
        {"--page-size", &CliOptions::page_size, "page size", 1, "page-size must be greater than 0"},
        {"--cache-tokens", &CliOptions::cache_tokens, "cache tokens", 1, "cache-tokens must be greater than 0"},
        {"--max-active", &CliOptions::max_active, "max active", 1, "max-active must be greater than 0"},
        {"--prefill-batch", &CliOptions::prefill_batch, "prefill batch", 1, "prefill-batch must be greater than 0"},
        {"--max-batch-tokens", &CliOptions::max_batch_tokens, "max batch tokens", 1, "max-batch-tokens must be greater than 0"},
        {"--chunk-size", &CliOptions::chunk_size, "chunk size", 1, "chunk-size must be greater than 0"},
    };
    for (int i = 1; i < argc; ++i) {
        const std::string arg = argv[i];
        auto value = [&](const char* what, std::string* out) -> std::string {
            if (i + 1 >= argc) return std::string("Missing ") + what + " after " + arg;
            *out = argv[++i];
            return "";
        };
        if (arg == "-h" || arg == "--help") {
            o->show_help = true;
            return "";
        }
        if (arg == "-f" || arg == "--prompt-file") {
            std::string v;
            const std::string err = value("path", &v);
            if (!err.empty()) return err;
            if (!o->prompt_file.empty()) return "Prompt file option specified multiple times";
            o->prompt_file = v;
            continue;
        }
        bool handled = false;
        for (const IntOption& opt : ints)
            if (arg == opt.flag) {
                std::string v;
                const std::string err = value("number", &v);
                if (!err.empty()) return err;
                long long num;
                if (!whole_integer(v, &num)) return std::string("Invalid number for ") + opt.label + ": " + v;
                if (num < opt.least) return opt.complaint;
                o->*(opt.field) = num;
                handled = true;
                break;
            }
        if (handled) continue;
        if (arg == "--temperature" || arg == "--top-p") {
            std::string v;
            const std::string err = value("number", &v);
            if (!err.empty()) return err;
            double num;
            if (!whole_real(v, &num)) return std::string("Invalid number for ") + (arg == "--top-p" ? "top-p" : "temperature") + ": " + v;
            if (arg == "--temperature") {
                if (!(num > 0.0)) return "Temperature must be greater than 0";
                o->temperature = num;
            } else {
                if (!(num > 0.0 && num <= 1.0)) return "Top-p must be in (0, 1]";
                o->top_p = num;
            }
            continue;
        }
        if (arg == "--greedy") { o->use_greedy = true; continue; }
        if (arg == "--token-ids") { o->token_ids = true; continue; }
        if (arg == "--no-chat-template") { o->chat_template = false; continue; }
        if (arg == "--model" || arg == "--config" || arg == "--dtype") {
            std::string v;
            const std::string err = value("value", &v);
            if (!err.empty()) return err;
            if (arg == "--dtype" && v != "bfloat16" && v != "float32") return "dtype must be bfloat16 or float32";
            (arg == "--model" ? o->model : arg == "--config" ? o->config : o->dtype) = v;
            continue;
        }
        if (arg.rfind("--serve", 0) == 0) return arg + ": the serving mode is not provided by this engine";
        if (arg.size() > 1 && arg[0] == '-') {
            bool numeric = true;                // "-5 3" is a prompt of token ids, not an option
            for (size_t k = 1; k < arg.size(); ++k)
                if (!(std::isdigit((unsigned char)arg[k]) || arg[k] == ',' || arg[k] == ' ')) numeric = false;
            if (!numeric) return "Unknown option: " + arg;
        }
        if (!o->prompt.empty()) return "Multiple prompts provided; use a single prompt or --prompt-file";
        o->prompt = arg;
    }
    return "";
}

std::string strip(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && std::isspace((unsigned char)s[a])) ++a;
    while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}
// one prompt per non-empty trimmed line (src/cli_options.cpp:66-84)
bool read_prompts_file(const std::string& path, std::vector<std::string>* prompts) {
    std::ifstream in(path);
    if (!in.is_open()) return false;
    std::string line;
    while (std::getline(in, line)) {
        line = strip(line);
        if (!line.empty()) prompts->push_back(line);
    }
    return true;
}
// <stem>_output<ext> beside the prompt file (src/main.cpp:113-120)
std::string output_path_for(const std::string& prompt_file) {
    const size_t slash = prompt_file.find_last_of('/');
    const std::string dir = slash == std::string::npos ? "" : prompt_file.substr(0, slash + 1);
    const std::string name = slash == std::string::npos ? prompt_file : prompt_file.substr(slash + 1);
    const size_t dot = name.find_last_of('.');
    if (dot == std::string::npos || dot == 0) return dir + name + "_output";
    return dir + name.substr(0, dot) + "_output" + name.substr(dot);
}
// the fixed Qwen template (src/cli_options.cpp:49-64)
std::string apply_chat_template(const std::string& user_query) {
    return "<|im_start|>system\nYou are Qwen, created by Alibaba Cloud. You are a helpful assistant.<|im_end|>\n<|im_start|>user\n" + user_query +
           "<|im_end|>\n<|im_start|>assistant\n";
}
bool parse_token_ids(std::string text, std::vector<int64_t>* out) {
    for (char& c : text)
        if (c == ',') c = ' ';
    std::istringstream in(text);
    std::string word;
    while (in >> word) {
        long long v;
        if (!whole_integer(word, &v)) return false;
        out->push_back(v);
    }
    return true;
}
std::string escape_single_line(const std::string& text) {
    std::string out;
    for (char c : text) {
        if (c == '\\') out += "\\\\";
        else if (c == '\n') out += "\\n";
        else if (c == '\r') out += "\\r";
        else out += c;
    }
    return out;
}
bool file_exists(const std::string& path) {
    struct stat st;
    return stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

// tokenizer.json (vocabulary and merges) and, for special tokens, tokenizer_config.json
std::unique_ptr<host::BpeTokenizer> load_tokenizer(const std::string& dir, int bos_token_id) {
    const std::string path = dir + "/tokenizer.json";
    if (!file_exists(path)) throw std::runtime_error("no tokenizer.json in " + dir);
    const easygpt::json::Value data = easygpt::json::parse(read_text_file(path));
    const easygpt::json::Value* model = data.find("model");
    if (!model || !model->find("vocab") || !model->find("merges")) throw std::runtime_error(path + " has no model.vocab / model.merges");
    std::unique_ptr<host::BpeTokenizer> tok(new host::BpeTokenizer());
    std::map<std::string, int> vocab;
    std::set<int> ids;
    for (auto& kv : model->find("vocab")->object) {
        vocab[kv.first] = (int)kv.second.integer;
        ids.insert((int)kv.second.integer);
    }
    std::vector<std::string> specials;
    const std::string cfg = dir + "/tokenizer_config.json";
    if (file_exists(cfg)) {
        const easygpt::json::Value c = easygpt::json::parse(read_text_file(cfg));
        if (const easygpt::json::Value* added = c.find("added_tokens_decoder"))
            for (auto& kv : added->object) {
                const easygpt::json::Value* content = kv.second.find("content");
                const easygpt::json::Value* special = kv.second.find("special");
                if (!content || !content->is_string() || content->string.empty() || !special || !special->is_bool() || !special->boolean) continue;
                specials.push_back(content->string);
                const int id = std::atoi(kv.first.c_str());
                if (!vocab.count(content->string) && !ids.count(id)) {
                    vocab[content->string] = id;
                    ids.insert(id);
                }
            }
    }
    for (auto& kv : vocab) tok->add_token(kv.first, kv.second);
    for (auto& m : model->find("merges")->array) {
        if (m.is_string()) {
            const size_t space = m.string.find(' ');
            if (space != std::string::npos) tok->add_merge(m.string.substr(0, space), m.string.substr(space + 1));
        } else if (m.is_array() && m.array.size() == 2) {
            tok->add_merge(m.array[0].string, m.array[1].string);
        }
    }
    std::sort(specials.begin(), specials.end(), [](const std::string& a, const std::string& b) { return a.size() != b.size() ? a.size() > b.size() : a < b; });
    for (auto& s : specials) tok->add_special(s);       // longest first
    tok->set_bos(bos_token_id);
    return tok;
}

}  // namespace

int main(int argc, char** argv) {
    CliOptions opts;
    const std::string err = parse_args(argc, argv, &opts);
    if (!err.empty()) {
        std::cerr << err << "\n" << kUsage;
        return 1;
    }
    if (opts.show_help) {
        std::cout << kUsage;
        return 0;
    }
    std::vector<std::string> prompts;
    if (!opts.prompt_file.empty() && !read_prompts_file(opts.prompt_file, &prompts)) {
        std::cerr << "Failed to open prompt file: " << opts.prompt_file << "\n";
        return 1;
    }
    if (!opts.prompt.empty()) prompts.push_back(opts.prompt);
    if (prompts.empty()) {
        std::cerr << "No prompts provided\n" << kUsage;
        return 1;
    }
    try {
        if (opts.random_weights >= 0) {
            if (opts.config.empty()) {
                std::cerr << "--random-weights needs --config <config.json>\n";
                return 1;
            }
            mkdir(opts.model.c_str(), 0777);
            write_random_model(opts.model, read_text_file(opts.config), (uint64_t)opts.random_weights);
        }
        std::unique_ptr<host::BpeTokenizer> tokenizer;
        std::vector<std::vector<int64_t>> token_prompts;
        if (opts.token_ids) {
            for (auto& p : prompts) {
                token_prompts.emplace_back();
                if (!parse_token_ids(p, &token_prompts.back())) {
                    std::cerr << "--token-ids prompts must be lists of integers\n";
                    return 1;
                }
            }
        } else {
            try {
                int bos = -1;
                const easygpt::json::Value config = easygpt::json::parse(read_text_file(opts.model + "/config.json"));
                if (const easygpt::json::Value* b = config.find("bos_token_id"))
                    if (b->is_number()) bos = (int)b->integer;
                tokenizer = load_tokenizer(opts.model, bos);
            } catch (const std::exception& e) {
                std::cerr << e.what() << "; text prompts need tokenizer.json (or pass --token-ids)\n";
                return 1;
            }
            for (auto& p : prompts) {
                const std::vector<int32_t> ids = tokenizer->encode(opts.chat_template ? apply_chat_template(p) : p);
                token_prompts.emplace_back(ids.begin(), ids.end());
            }
        }
        EngineOptions eo;
        eo.page_size = (int)opts.page_size;
        eo.cache_tokens = opts.cache_tokens;
        eo.max_active = (int)opts.max_active;
        eo.prefill_batch = (int)opts.prefill_batch;
        eo.max_batch_tokens = opts.max_batch_tokens;
        eo.chunk_size = opts.chunk_size;
        GptEngine engine(opts.model, opts.dtype == "float32" ? DType::F32 : DType::BF16, eo);
        SamplingParams params;
        params.temperature = (float)opts.temperature;
        params.top_p = (float)opts.top_p;
        params.top_k = (int)opts.top_k;
        params.seed = opts.seed;
        params.greedy = opts.use_greedy;
        const std::vector<std::vector<int64_t>> outputs = engine.generate(token_prompts, params, /*max_new_tokens=*/0, opts.max_steps);
        std::vector<std::string> lines;
        for (auto& out : outputs) {
            if (!tokenizer) {
                std::string line;
                for (size_t i = 0; i < out.size(); ++i) line += (i ? " " : "") + std::to_string(out[i]);
                lines.push_back(line);
            } else {
                const std::vector<int32_t> ids(out.begin(), out.end());
                lines.push_back(escape_single_line(tokenizer->decode(ids.data(), ids.size())));
            }
        }
        if (!opts.prompt_file.empty()) {
            std::ofstream file(output_path_for(opts.prompt_file));
            for (auto& line : lines) file << line << "\n";
        }
        for (auto& line : lines) std::cout << line << "\n";
    } catch (const std::exception& e) {
        std::cerr << "easy_llm: " << e.what() << "\n";
        return 1;
    }
    return 0;
}
