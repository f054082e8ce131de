// promethorch C++ API: the GGUF model behind PromeServe (serve.h) on the CUDA decode engine.
//
// One GGUFBackend = one GGUFModel (gguf.h) + the tokenizer its file describes (tokenizer.h).  The prompt runs as one
// scripted pass on the device; greedy requests (temperature <= 0 and no repetition penalty) then step with the arg-max the
// engine computes, sampled requests draw on the device from the logits of each step; one id per token crosses to the host
// either way.  Link with libptb200.so and the CUDA runtime.
#pragma once
#include <chrono>
#include <set>

#include "gguf.h"
#include "serve.h"
#include "tokenizer.h"

namespace promethorch {
namespace serve {

class GGUFBackend : public ModelBackend {
 public:
    GGUFBackend(const std::string& path, const std::string& name_, int max_seq = 4096) {
        model_.load(path, max_seq, /*want_logits=*/true);
        tok_ = io::GGUFTokenizer::from_reader(model_.reader());
        name = name_;
        architecture = model_.config.architecture;
        model_name = model_.reader().has("general.name") ? model_.reader().get("general.name").s : "";
        size = store::file_size(path);
        unsigned long long bytes = 0;
        for (const auto& kv : model_.reader().tensors()) bytes += kv.second.nbytes;
        char buf[32];
        std::snprintf(buf, sizeof buf, "%.1fB", (double)bytes / 0.5625 / 1e9);          // 4.5 bits per weight
        parameter_size = buf;
        if (tok_.eos_id() >= 0) stop_.insert(tok_.eos_id());
        for (const char* t : {"<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>"})
            if (tok_.token_id(t) >= 0) stop_.insert(tok_.token_id(t));
    }
    std::vector<int> encode(const std::string& text) override { return tok_.encode(text); }
    std::string decode_token(int id) override { return tok_.decode_token(id); }
    std::pair<double, double> generate(const std::vector<int>& prompt, const GenerateOptions& opt, const std::function<bool(int)>& on_token) override {
        using clock = std::chrono::steady_clock;
        const int n = (int)prompt.size();
        if (n + 2 > model_.max_seq()) throw std::runtime_error("the prompt does not fit the context of " + std::to_string(model_.max_seq()) + " tokens");
        const int n_new = std::max(0, std::min(opt.num_predict, model_.max_seq() - n - 1));
        const bool greedy = opt.temperature <= 0.0 && opt.repeat_penalty == 1.0;
        const auto t0 = clock::now();
        if (n > 1) model_.run_prompt(std::vector<int>(prompt.begin(), prompt.end() - 1));
        const auto t1 = clock::now();
        if (!greedy) model_.sampler_reset(prompt, (uint64_t)opt.seed);
        int tok = prompt.back(), pos = n - 1;
        for (int i = 0; i < n_new; ++i) {
            int next = model_.forward_decode(tok, pos);
            if (!greedy) next = model_.sample(opt.temperature, opt.top_k, opt.top_p, opt.repeat_penalty);
            if (!on_token(next) || stop_.count(next)) break;
            tok = next;
            if (++pos + 1 >= model_.max_seq()) break;
        }
        const auto t2 = clock::now();
        return {std::chrono::duration<double>(t1 - t0).count(), std::chrono::duration<double>(t2 - t1).count()};
    }
    io::GGUFModel& model() { return model_; }
    const io::GGUFTokenizer& tokenizer() const { return tok_; }

 private:
    io::GGUFModel model_;
    io::GGUFTokenizer tok_;
    std::set<int> stop_;
};

// The loader PromeServe uses for names it has not seen: <model dir>/<name>.gguf, else the Ollama store.
inline ApiHandlers::Loader gguf_loader(const ServerConfig& cfg) {
    return [cfg](const std::string& name) -> std::shared_ptr<ModelBackend> {
        return std::make_shared<GGUFBackend>(store::resolve(name, cfg.model_dirs), name, cfg.max_seq);
    };
}

}  // namespace serve
}  // namespace promethorch
