// spbitnet_infer for the sm_100a library: the command line of the reference's src/main.cpp over the C-ABI.
//
//   spbitnet_infer --model <dir> [--prompt <text>] [--max-tokens N] [--dump-tokens <file>] [--benchmark [N]]
//
// Flags and flow as the reference (src/main.cpp:43-68, 97-124, 266-340): the model directory is loaded, the
// tokenizer (<dir>/tokenizer.json) if present, the input is BOS + the prompt's ids, the prompt is fed token by
// token, then greedy decoding until --max-tokens or EOS; --dump-tokens writes the JSON object
// {"prompt", "prompt_ids", "input_ids", "generated_ids"} that python/baseline_pytorch.py --compare reads
// (src/main.cpp:315-340); --benchmark N times N generated tokens (1 warm-up + 3 runs, median, :161-245).
// --profile is accepted and ignored (the per-kernel profiler of the reference has no counterpart: a token is one
// CUDA graph here).  The arg-max runs on the device; tokens are the ones the host loop would pick (first maximum).
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "../../include/spbitnet_b200.h"

static void usage(const char* argv0) {
    std::printf("Usage: %s --model <dir> [--prompt <text>] [--max-tokens N] [--dump-tokens <file>] [--benchmark [N]] [--profile]\n", argv0);
}

static std::string json_escape(const std::string& s) {
    std::string o;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { o += '\\'; o += static_cast<char>(c); }
        else if (c == '\n') o += "\\n";
        else if (c == '\r') o += "\\r";
        else if (c == '\t') o += "\\t";
        else if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += static_cast<char>(c);
    }
    return o;
}

int main(int argc, char** argv) {
    std::string model_dir, prompt = "Hello", dump_path;
    int max_tokens = 32, bench_tokens = 128;
    bool bench = false;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--model" && i + 1 < argc) model_dir = argv[++i];
        else if (a == "--prompt" && i + 1 < argc) prompt = argv[++i];
        else if (a == "--max-tokens" && i + 1 < argc) max_tokens = std::atoi(argv[++i]);
        else if (a == "--dump-tokens" && i + 1 < argc) dump_path = argv[++i];
        else if (a == "--benchmark") {
            bench = true;
            if (i + 1 < argc && argv[i + 1][0] != '-') {
                bench_tokens = std::atoi(argv[++i]);
                if (bench_tokens <= 0) bench_tokens = 128;
            }
        } else if (a == "--profile") {
        } else if (a == "--help") {
            usage(argv[0]);
            return 0;
        } else {
            std::fprintf(stderr, "Unknown option: %s\n", a.c_str());
            usage(argv[0]);
            return 1;
        }
    }
    std::printf("spbitnet_infer (%s)\n", spb_version());
    if (model_dir.empty()) {
        std::printf("No model specified. Use --model <dir> to load a model.\n");
        return 0;
    }
    auto die = [](const char* what) {
        std::fprintf(stderr, "Error: %s: %s\n", what, spb_last_error_string());
        return 1;
    };
    spb_model* model = spb_model_load(model_dir.c_str());
    if (!model) return die("model");
    spb_model_config cfg;
    int bos = 0, eos = 0;
    spb_model_get_config(model, &cfg, &bos, &eos);
    std::printf("Model: %d layers, hidden %d, vocab %d, %.1f MB on the device\n", cfg.num_hidden_layers, cfg.hidden_size,
                cfg.vocab_size, spb_model_device_bytes(model) / 1e6);
    spb_engine* engine = spb_engine_create(&cfg);
    if (!engine || spb_model_attach(model, engine) != SPB_OK) return die("engine");
    spb_tokenizer* tok = spb_tokenizer_load((model_dir + "/tokenizer.json").c_str());
    if (tok) std::printf("Tokenizer loaded (%d tokens)\n", spb_tokenizer_vocab_size(tok));
    else std::printf("Warning: tokenizer not available (%s)\n", spb_last_error_string());

    std::vector<int> prompt_ids;
    if (tok) {
        const int n = spb_tokenizer_encode(tok, prompt.data(), prompt.size(), nullptr, 0);
        prompt_ids.resize(static_cast<size_t>(std::max(n, 0)));
        spb_tokenizer_encode(tok, prompt.data(), prompt.size(), prompt_ids.data(), n);
        std::printf("Prompt: \"%s\" -> %d tokens [", prompt.c_str(), n);
        for (size_t i = 0; i < prompt_ids.size(); ++i) std::printf("%s%d", i ? ", " : "", prompt_ids[i]);
        std::printf("]\n");
    }
    std::vector<int> input_ids;
    input_ids.push_back(bos);
    input_ids.insert(input_ids.end(), prompt_ids.begin(), prompt_ids.end());

    if (bench) {
        std::vector<int> out(static_cast<size_t>(bench_tokens));
        std::vector<double> secs;
        for (int run = 0; run < 4; ++run) {  // one warm-up, three timed
            spb_engine_reset(engine);
            const auto t0 = std::chrono::steady_clock::now();
            const int n = spb_engine_generate(engine, input_ids.data(), static_cast<int>(input_ids.size()), bench_tokens, -1, out.data());
            const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
            if (n < 0) return die("generate");
            if (run > 0) secs.push_back(dt);
        }
        std::sort(secs.begin(), secs.end());
        const int steps = static_cast<int>(input_ids.size()) - 1 + bench_tokens;
        std::printf("Benchmark: %d prompt + %d generated tokens, median %.2f ms, %.1f tok/s\n", static_cast<int>(input_ids.size()),
                    bench_tokens, secs[1] * 1e3, steps / secs[1]);
    }

    std::printf("Max tokens: %d\n\n--- Generation ---\n", max_tokens);
    if (tok) std::printf("%s", prompt.c_str());
    spb_engine_reset(engine);
    std::vector<int> generated(static_cast<size_t>(std::max(max_tokens, 1)));
    const int n_gen = spb_engine_generate(engine, input_ids.data(), static_cast<int>(input_ids.size()), max_tokens, eos, generated.data());
    if (n_gen < 0) return die("generate");
    generated.resize(static_cast<size_t>(n_gen));
    for (int t = 0; t < n_gen; ++t) {
        if (tok) {
            char piece[256];
            spb_tokenizer_decode(tok, &generated[static_cast<size_t>(t)], 1, piece, sizeof piece);
            std::printf("%s", piece);
        } else {
            std::printf("token[%d] = %d\n", t, generated[static_cast<size_t>(t)]);
        }
    }
    std::printf("\n\n--- %d tokens generated ---\n", n_gen);

    if (!dump_path.empty()) {
        std::ofstream ofs(dump_path);
        if (!ofs) {
            std::fprintf(stderr, "Error: cannot open %s\n", dump_path.c_str());
            return 1;
        }
        auto list = [&](const char* name, const std::vector<int>& v, bool last) {
            ofs << "  \"" << name << "\": [";
            for (size_t i = 0; i < v.size(); ++i) ofs << (i ? ", " : "") << v[i];
            ofs << (last ? "]\n" : "],\n");
        };
        ofs << "{\n  \"prompt\": \"" << json_escape(prompt) << "\",\n";
        list("prompt_ids", prompt_ids, false);
        list("input_ids", input_ids, false);
        list("generated_ids", generated, true);
        ofs << "}\n";
        std::printf("Token IDs saved to %s\n", dump_path.c_str());
    }
    if (tok) spb_tokenizer_destroy(tok);
    spb_engine_destroy(engine);
    spb_model_destroy(model);
    return 0;
}
