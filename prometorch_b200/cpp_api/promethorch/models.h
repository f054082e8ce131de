// promethorch C++ API: a Llama-family decoder over libtorch, loaded from a Hugging Face directory.
//
//   LlamaConfig::from_json(dir + "/config.json")
//   models::Llama model(cfg);  model->load_hf(dir);               // config.json + *.safetensors (sharded or not)
//   logits = model->forward(ids [B, T]);                           // full causal pass
//   ids    = model->generate(prompt, n, temperature = 0);          // greedy or sampled decoding with a key / value cache
//
// The layer structure is the one the Python engine of this package runs (serve/llm.py) and the reference's torch::serve
// engine loads (torch/serve/llm.h): RMSNorm -> q/k/v projections -> rotary embedding on pairs (j, j + D/2) -> grouped-query
// causal attention -> output projection, then RMSNorm -> SiLU-gated MLP, pre-norm residuals, tied or separate output head.
// This model is tensor code (runs wherever libtorch runs, CPU included); the hand-written decode kernels are reached through
// io::GGUFModel (gguf.h) and the Python engine.
#pragma once
#include <torch/torch.h>

#include <cmath>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "json.h"
#include "serialization.h"

namespace promethorch {
namespace models {
using Tensor = at::Tensor;

struct LlamaConfig {
    int64_t vocab_size = 32000, hidden_size = 4096, intermediate_size = 11008, num_hidden_layers = 32, num_attention_heads = 32,
            num_key_value_heads = 32, max_position_embeddings = 4096, bos_token_id = 1, eos_token_id = 2;
    double rms_norm_eps = 1e-5, rope_theta = 10000.0;
    bool tie_word_embeddings = false;
    int64_t head_dim() const { return hidden_size / num_attention_heads; }
    static LlamaConfig from_json(const std::string& path) {
        std::ifstream f(path);
        if (!f) throw std::runtime_error("LlamaConfig: cannot open " + path);
        std::stringstream ss;
        ss << f.rdbuf();
        const json::Value d = json::parse(ss.str());
        LlamaConfig c;
        auto geti = [&](const char* k, int64_t& v) { if (d[k].is_number()) v = d[k].as_int(); };
        geti("vocab_size", c.vocab_size);
        geti("hidden_size", c.hidden_size);
        geti("intermediate_size", c.intermediate_size);
        geti("num_hidden_layers", c.num_hidden_layers);
        geti("num_attention_heads", c.num_attention_heads);
        c.num_key_value_heads = c.num_attention_heads;
        geti("num_key_value_heads", c.num_key_value_heads);
        geti("max_position_embeddings", c.max_position_embeddings);
        geti("bos_token_id", c.bos_token_id);
        if (d["eos_token_id"].is_array() && d["eos_token_id"].size()) c.eos_token_id = d["eos_token_id"].at(0).as_int();
        else geti("eos_token_id", c.eos_token_id);
        if (d["rms_norm_eps"].is_number()) c.rms_norm_eps = d["rms_norm_eps"].as_double();
        if (d["rope_theta"].is_number()) c.rope_theta = d["rope_theta"].as_double();
        if (d["tie_word_embeddings"].is_bool()) c.tie_word_embeddings = d["tie_word_embeddings"].as_bool();
        return c;
    }
};

class LlamaImpl : public torch::nn::Module {
 public:
    explicit LlamaImpl(const LlamaConfig& cfg) : cfg_(cfg) {
        const int64_t D = cfg.hidden_size, H = cfg.num_attention_heads, Hk = cfg.num_key_value_heads, Dh = cfg.head_dim(), I = cfg.intermediate_size;
        embed = reg("model.embed_tokens.weight", torch::randn({cfg.vocab_size, D}) * 0.02);
        for (int64_t l = 0; l < cfg.num_hidden_layers; ++l) {
            const std::string p = "model.layers." + std::to_string(l) + ".";
            Layer L;
            auto lin = [&](const std::string& n, int64_t out, int64_t in) { return reg(p + n, torch::randn({out, in}) * std::pow((double)in, -0.5)); };
            L.attn_norm = reg(p + "input_layernorm.weight", torch::ones({D}));
            L.q = lin("self_attn.q_proj.weight", H * Dh, D);
            L.k = lin("self_attn.k_proj.weight", Hk * Dh, D);
            L.v = lin("self_attn.v_proj.weight", Hk * Dh, D);
            L.o = lin("self_attn.o_proj.weight", D, H * Dh);
            L.ffn_norm = reg(p + "post_attention_layernorm.weight", torch::ones({D}));
            L.gate = lin("mlp.gate_proj.weight", I, D);
            L.up = lin("mlp.up_proj.weight", I, D);
            L.down = lin("mlp.down_proj.weight", D, I);
            layers_.push_back(L);
        }
        norm = reg("model.norm.weight", torch::ones({D}));
        if (!cfg.tie_word_embeddings) lm_head = reg("lm_head.weight", torch::randn({cfg.vocab_size, D}) * std::pow((double)D, -0.5));
        rope_tables();
    }
    const LlamaConfig& config() const { return cfg_; }

    // Reads every *.safetensors of the directory (or a single file) into the parameters; names are Hugging Face's.
    void load_hf(const std::string& path) {
        torch::NoGradGuard ng;
        std::map<std::string, Tensor> sd;
        for (auto& kv : load_safetensors_sharded(path)) sd[kv.first] = kv.second;
        if (sd.count("embed_tokens.weight") && !sd.count("model.embed_tokens.weight")) {          // a bare decoder checkpoint
            std::map<std::string, Tensor> fixed;
            for (auto& kv : sd) fixed[kv.first.rfind("lm_head", 0) == 0 ? kv.first : "model." + kv.first] = kv.second;
            sd.swap(fixed);
        }
        for (auto& item : hf_) {
            auto it = sd.find(item.first);
            if (it == sd.end()) {
                if (item.first == "lm_head.weight" && sd.count("model.embed_tokens.weight")) { item.second.copy_(sd["model.embed_tokens.weight"]); continue; }
                throw std::runtime_error("Llama::load_hf: the checkpoint has no tensor " + item.first);
            }
            if (it->second.sizes() != item.second.sizes()) throw std::runtime_error("Llama::load_hf: shape mismatch for " + item.first);
            item.second.copy_(it->second);
        }
    }
    // The parameters under their Hugging Face names, in checkpoint order (what save_safetensors / save_pytorch take).
    OrderedStateDict hf_state_dict() const { return hf_; }

    // ids [B, T] -> logits [B, T, vocab] (fp32 math in the dtype of the parameters); pos0: position of the first column.
    Tensor forward(const Tensor& ids, int64_t pos0 = 0) { return run(ids, pos0, nullptr); }

    // Decoding with a key / value cache: the prompt in one pass, then one token per pass.  temperature <= 0: greedy.
    std::vector<int64_t> generate(const std::vector<int64_t>& prompt, int64_t max_new_tokens, double temperature = 0.0, int64_t top_k = 0, bool stop_at_eos = true) {
        torch::NoGradGuard ng;
        std::vector<Cache> cache((size_t)cfg_.num_hidden_layers);
        std::vector<int64_t> out;
        Tensor ids = torch::tensor(prompt, torch::kLong).unsqueeze(0).to(embed.device());
        int64_t pos = 0;
        for (int64_t i = 0; i < max_new_tokens; ++i) {
            Tensor logits = run(ids, pos, &cache).select(1, ids.size(1) - 1).squeeze(0).to(torch::kFloat);
            pos += ids.size(1);
            int64_t next;
            if (temperature <= 0.0) {
                next = logits.argmax().item<int64_t>();
            } else {
                Tensor l = logits / temperature;
                if (top_k > 0 && top_k < l.numel()) l = l.masked_fill(l < std::get<0>(l.topk(top_k)).min(), -INFINITY);
                next = torch::multinomial(torch::softmax(l, 0), 1).item<int64_t>();
            }
            out.push_back(next);
            if ((stop_at_eos && next == cfg_.eos_token_id) || pos + 1 >= cfg_.max_position_embeddings) break;
            ids = torch::tensor({next}, torch::kLong).unsqueeze(0).to(embed.device());
        }
        return out;
    }

    Tensor embed, norm, lm_head;

 private:
    struct Layer { Tensor attn_norm, q, k, v, o, ffn_norm, gate, up, down; };
    struct Cache { Tensor k, v; };

    // libtorch parameter names cannot hold dots: registered with '_' instead, the Hugging Face name kept beside the tensor
    Tensor reg(const std::string& hf_name, Tensor init) {
        std::string flat = hf_name;
        for (auto& c : flat)
            if (c == '.') c = '_';
        Tensor t = register_parameter(flat, std::move(init), false);
        hf_.emplace_back(hf_name, t);
        return t;
    }
    void rope_tables() {
        const int64_t Dh = cfg_.head_dim();
        Tensor inv = 1.0 / torch::pow(cfg_.rope_theta, torch::arange(0, Dh, 2, torch::kDouble) / (double)Dh);
        Tensor ang = torch::arange(cfg_.max_position_embeddings, torch::kDouble).unsqueeze(1) * inv.unsqueeze(0);
        cos_ = register_buffer("rope_cos", ang.cos().to(torch::kFloat));
        sin_ = register_buffer("rope_sin", ang.sin().to(torch::kFloat));
    }
    Tensor rms(const Tensor& x, const Tensor& w) const {
        Tensor v = x.to(torch::kFloat);
        return (v * torch::rsqrt(v.pow(2).mean(-1, true) + cfg_.rms_norm_eps) * w.to(torch::kFloat)).to(x.dtype());
    }
    // x [B, T, heads, Dh]: pairs (j, j + Dh/2) rotate by the angle of the token's position.
    Tensor rope(const Tensor& x, int64_t pos0) const {
        const int64_t T = x.size(1), half = x.size(3) / 2;
        Tensor c = cos_.slice(0, pos0, pos0 + T).unsqueeze(0).unsqueeze(2), s = sin_.slice(0, pos0, pos0 + T).unsqueeze(0).unsqueeze(2);
        Tensor a = x.slice(3, 0, half).to(torch::kFloat), b = x.slice(3, half, 2 * half).to(torch::kFloat);
        return torch::cat({a * c - b * s, b * c + a * s}, 3).to(x.dtype());
    }
    Tensor run(const Tensor& ids, int64_t pos0, std::vector<Cache>* cache) {
        const int64_t B = ids.size(0), T = ids.size(1), H = cfg_.num_attention_heads, Hk = cfg_.num_key_value_heads, Dh = cfg_.head_dim();
        TORCH_CHECK(pos0 + T <= cfg_.max_position_embeddings, "Llama: the sequence runs past max_position_embeddings");
        Tensor h = torch::embedding(embed, ids);
        for (size_t l = 0; l < layers_.size(); ++l) {
            const Layer& L = layers_[l];
            Tensor x = rms(h, L.attn_norm);
            Tensor q = rope(torch::nn::functional::linear(x, L.q).view({B, T, H, Dh}), pos0);
            Tensor k = rope(torch::nn::functional::linear(x, L.k).view({B, T, Hk, Dh}), pos0);
            Tensor v = torch::nn::functional::linear(x, L.v).view({B, T, Hk, Dh});
            if (cache) {
                Cache& c = (*cache)[l];
                c.k = c.k.defined() ? torch::cat({c.k, k}, 1) : k;
                c.v = c.v.defined() ? torch::cat({c.v, v}, 1) : v;
                k = c.k;
                v = c.v;
            }
            const int64_t Tk = k.size(1);
            Tensor qh = q.permute({0, 2, 1, 3}).to(torch::kFloat);
            Tensor kh = k.permute({0, 2, 1, 3}).repeat_interleave(H / Hk, 1).to(torch::kFloat);
            Tensor vh = v.permute({0, 2, 1, 3}).repeat_interleave(H / Hk, 1).to(torch::kFloat);
            Tensor s = torch::matmul(qh, kh.transpose(-1, -2)) / std::sqrt((double)Dh);
            Tensor qi = torch::arange(T, ids.device()).unsqueeze(1) + (Tk - T), ki = torch::arange(Tk, ids.device()).unsqueeze(0);
            s = s.masked_fill(ki > qi, -INFINITY);
            Tensor a = torch::matmul(torch::softmax(s, -1), vh).permute({0, 2, 1, 3}).reshape({B, T, H * Dh}).to(h.dtype());
            h = h + torch::nn::functional::linear(a, L.o);
            x = rms(h, L.ffn_norm);
            h = h + torch::nn::functional::linear(torch::silu(torch::nn::functional::linear(x, L.gate)) * torch::nn::functional::linear(x, L.up), L.down);
        }
        return torch::nn::functional::linear(rms(h, norm), lm_head.defined() ? lm_head : embed);
    }

    LlamaConfig cfg_;
    OrderedStateDict hf_;
    std::vector<Layer> layers_;
    Tensor cos_, sin_;
};
TORCH_MODULE(Llama);

}  // namespace models
}  // namespace promethorch
