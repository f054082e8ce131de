// gguf_generate: text generation from a GGUF file as a native program (C++ reader, tokenizer, chat templates, CUDA decode
// engine).  The flags are those of the reference's test_gguf_inference (examples/gguf/test_gguf_inference.cpp:76-120):
//
//   gguf_generate MODEL [PROMPT] [--device cuda|cpu] [--greedy] [--max-tokens N] [--temp T] [--top-k K] [--top-p P]
//                 [--repeat-penalty R] [--seed S] [--chat | --raw] [--info] [--tensors] [--profile]
//
// MODEL is a .gguf path, an Ollama model name or (with --device cpu, --info or --tensors) a Hugging Face directory.
// --info prints the metadata and the parsed configuration, --tensors the tensor directory (neither touches the GPU),
// --chat wraps the prompt in the model's chat template, --profile prints per-kernel phase times of the last token.
// --fp16-weights and --llama-gemv select kernels that have no counterpart here and are accepted and ignored.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>

#include "promethorch/gguf_backend.h"
#include "promethorch/gguf_cpu.h"

namespace pio = promethorch::io;
namespace ps = promethorch::serve;

static const char* type_name(uint32_t t) {
    switch (t) {
        case pio::gguf::F32: return "F32";
        case pio::gguf::F16: return "F16";
        case pio::gguf::BF16: return "BF16";
        case pio::gguf::Q4_0: return "Q4_0";
        case pio::gguf::Q8_0: return "Q8_0";
        case pio::gguf::Q2_K: return "Q2_K";
        case pio::gguf::Q3_K: return "Q3_K";
        case pio::gguf::Q4_K: return "Q4_K";
        case pio::gguf::Q5_K: return "Q5_K";
        case pio::gguf::Q6_K: return "Q6_K";
        default: return "?";
    }
}
static std::string show(const pio::gguf::Value& v) {
    switch (v.type) {
        case 8: return "'" + v.s + "'";
        case 7: return v.b ? "true" : "false";
        case 6: case 12: { char b[48]; std::snprintf(b, sizeof b, "%g", v.f); return b; }
        case 9: {
            std::string s = "[";
            for (size_t i = 0; i < v.arr.size() && i < 6; ++i) s += (i ? ", " : "") + show(v.arr[i]);
            if (v.arr.size() > 6) s += ", ... (" + std::to_string(v.arr.size()) + " items)";
            return s + "]";
        }
        default: return std::to_string(v.as_int());
    }
}

int main(int argc, char** argv) {
    std::string model, prompt = "Hello, how are you?", device = "cuda";
    bool have_prompt = false, info = false, tensors = false, greedy = false, chat = false, raw = false, profile = false;
    ps::GenerateOptions opt;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto val = [&]() -> std::string {
            if (i + 1 >= argc) { std::fprintf(stderr, "gguf_generate: %s needs a value\n", a.c_str()); std::exit(2); }
            return argv[++i];
        };
        if (a == "--info") info = true;
        else if (a == "--tensors") tensors = true;
        else if (a == "--greedy") greedy = true;
        else if (a == "--chat") chat = true;
        else if (a == "--raw") raw = true;
        else if (a == "--profile") profile = true;
        else if (a == "--cuda") device = "cuda";
        else if (a == "--device") device = val();
        else if (a == "--fp16-weights" || a == "--fp16_weights" || a == "--llama-gemv" || a == "--llama_gemv") {}
        else if (a == "--max-tokens" || a == "--max_tokens") opt.num_predict = std::atoi(val().c_str());
        else if (a == "--temp" || a == "--temperature") opt.temperature = std::atof(val().c_str());
        else if (a == "--top-k") opt.top_k = std::atoi(val().c_str());
        else if (a == "--top-p") opt.top_p = std::atof(val().c_str());
        else if (a == "--repeat-penalty") opt.repeat_penalty = std::atof(val().c_str());
        else if (a == "--seed") opt.seed = std::atoll(val().c_str());
        else if (a.size() > 2 && a[0] == '-' && a[1] == '-') { std::fprintf(stderr, "gguf_generate: unknown flag %s\n", a.c_str()); return 2; }
        else if (model.empty()) model = a;
        else if (!have_prompt) { prompt = a; have_prompt = true; }
    }
    if (model.empty()) { std::fprintf(stderr, "usage: gguf_generate MODEL [PROMPT] [flags]  (see the top of apps/gguf_generate.cpp)\n"); return 2; }
    try {
        const bool is_path = model.find('/') != std::string::npos || (model.size() > 5 && model.compare(model.size() - 5, 5, ".gguf") == 0);
        const std::string path = is_path ? model : ps::store::resolve_ollama(model);
        if ((info || tensors) && ps::store::is_dir(path)) {            // a Hugging Face directory: what the model loader sees
            const pio::loader::ModelWeights mw = pio::loader::load_model(path);
            const auto& m = mw.config;
            if (info)
                std::printf("architecture %s (%s), %lld layers, hidden %lld, %lld heads (%lld kv), ffn %lld, context %lld, %lld parameters in %zu file(s)\n",
                            mw.architecture.c_str(), mw.format.c_str(), (long long)m.num_layers, (long long)m.hidden_size, (long long)m.num_heads, (long long)m.num_kv_heads,
                            (long long)m.intermediate_size, (long long)m.context_length, (long long)mw.total_parameters(), mw.files.size());
            if (tensors)
                for (const auto& name : mw.order) {
                    const auto& t = mw.tensors.at(name);
                    std::string shape = "(";
                    for (size_t d = 0; d < t.shape.size(); ++d) shape += (d ? ", " : "") + std::to_string(t.shape[d]);
                    shape += ")";
                    std::printf("%-48s %-24s %-6s %llu B\n", name.c_str(), shape.c_str(), t.dtype.c_str(), (unsigned long long)t.nbytes);
                }
            return 0;
        }
        if (info || tensors) {
            pio::gguf::GGUFReader r(path);
            if (info) {
                for (const auto& kv : r.metadata()) {
                    std::string s = show(kv.second);
                    if (s.size() > 120) s = s.substr(0, 117) + "...";
                    std::printf("%s = %s\n", kv.first.c_str(), s.c_str());
                }
                std::printf("architecture %s, %lld layers, hidden %lld, %lld heads (%lld kv), ffn %lld, context %lld\n", r.arch().c_str(),
                            (long long)r.arch_int("block_count", 0), (long long)r.arch_int("embedding_length", 0), (long long)r.arch_int("attention.head_count", 0),
                            (long long)r.arch_int("attention.head_count_kv", r.arch_int("attention.head_count", 0)), (long long)r.arch_int("feed_forward_length", 0),
                            (long long)r.arch_int("context_length", 8192));
            }
            if (tensors)
                for (const auto& kv : r.tensors()) {
                    std::string shape = "(";
                    for (size_t d = 0; d < kv.second.shape.size(); ++d) shape += (d ? ", " : "") + std::to_string(kv.second.shape[d]);
                    shape += ")";
                    std::printf("%-48s %-24s %-6s %llu B\n", kv.first.c_str(), shape.c_str(), type_name(kv.second.type), (unsigned long long)kv.second.nbytes);
                }
            return 0;
        }
        if (device != "cuda" && device != "gpu" && device != "cpu") { std::fprintf(stderr, "gguf_generate: --device is cuda or cpu\n"); return 2; }
        const bool on_cpu = device == "cpu";
        if (greedy) { opt.temperature = 0.0; opt.repeat_penalty = 1.0; }
        if (profile && !on_cpu) ::setenv("PTB_TRACE", "1", 1);
        using clock = std::chrono::steady_clock;
        const auto t0 = clock::now();
        const int max_seq = std::min(4096, opt.num_predict + 2048);
        std::unique_ptr<ps::GGUFBackend> gpu;
        std::unique_ptr<ps::CpuBackend> cpu;
        if (on_cpu) cpu.reset(new ps::CpuBackend(path, "cli", max_seq));
        else gpu.reset(new ps::GGUFBackend(path, "cli", max_seq));
        ps::ModelBackend& backend = on_cpu ? static_cast<ps::ModelBackend&>(*cpu) : static_cast<ps::ModelBackend&>(*gpu);
        const pio::TransformerConfig& c = on_cpu ? cpu->model().config : gpu->model().config;
        std::printf("[Model] %s %d layers, hidden %d, loaded in %.1f s on %s\n", c.architecture.c_str(), c.num_layers, c.hidden_size,
                    std::chrono::duration<double>(clock::now() - t0).count(), on_cpu ? "CPU" : "CUDA");
        const std::string text = (chat && !raw) ? pio::chat::apply_chat_template(prompt, backend.architecture, backend.model_name) : prompt;
        std::vector<int> ids = backend.encode(text);
        if (ids.empty()) ids.push_back(0);
        std::printf("[Generate] Prompt tokens: %zu\n", ids.size());
        int n = 0;
        std::vector<int> out;
        const auto t1 = clock::now();
        backend.generate(ids, opt, [&](int id) {
            ++n;
            out.push_back(id);
            std::fputs(backend.decode_token(id).c_str(), stdout);
            std::fflush(stdout);
            return true;
        });
        const double dt = std::chrono::duration<double>(clock::now() - t1).count();
        std::printf("\n\n[Generate] %d tokens in %.2fs (%.1f tok/s, prompt included)\n", n, dt, n / std::max(dt, 1e-9));
        std::printf("[Ids]");
        for (int id : out) std::printf(" %d", id);
        std::printf("\n");
        if (profile && !on_cpu) {
            const int n_k = 5 * c.num_layers + 2;
            std::vector<unsigned long long> buf((size_t)8 * n_k);
            const int got = gpu->model().read_trace(buf.data(), n_k);
            static const char* per_layer[5] = {"qkv", "attention", "o", "gate/up", "down"};
            std::map<std::string, std::pair<double, int>> tot;
            std::vector<std::string> order;
            for (int k = 0; k < got; ++k) {
                const std::string name = k == 0 ? "embed" : (k == n_k - 1 ? "lm_head" : per_layer[(k - 1) % 5]);
                const unsigned long long* s = &buf[(size_t)8 * k];
                if (!s[0] || !s[5]) continue;
                if (!tot.count(name)) order.push_back(name);
                tot[name].first += (double)(s[5] - s[0]) / 1e3;
                tot[name].second += 1;
            }
            for (const auto& nm : order) std::printf("[Profile] %-10s %4d launches, %7.2f us each (CTA 0, start to end)\n", nm.c_str(), tot[nm].second, tot[nm].first / tot[nm].second);
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "gguf_generate: %s\n", e.what());
        return 1;
    }
    return 0;
}
