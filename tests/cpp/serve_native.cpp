// Test program for the native serving stack (json.h, tokenizer.h, chat.h, serve.h): no GPU, no libtorch.
//   serve_native tokenize SPEC.json        ids / decoded text / pre-tokeniser pieces for every text of the spec
//   serve_native gguf-tokenize FILE.gguf TEXTS.json
//   serve_native chat SPEC.json            rendered prompts
//   serve_native json FILE.json            parse and dump again
//   serve_native serve [--workers N] [--queue-depth N] [--timeout-ms MS] [--model-dir DIR] [--max-body N]
//                                          serves fake backends on a free port, prints "PORT n", runs until stdin closes
#include <fstream>
#include <iostream>
#include <sstream>
#include <thread>

#include "promethorch/gguf_cpu.h"
#include "promethorch/model_loader.h"
#include "promethorch/serve.h"
#include "promethorch/tokenizer.h"

namespace pj = promethorch::json;
namespace ps = promethorch::serve;
namespace pio = promethorch::io;

static std::string slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}
static pj::Value ids_json(const std::vector<int>& ids) {
    pj::Value a = pj::Value::array();
    for (int i : ids) a.push_back(i);
    return a;
}
static pj::Value run_texts(const pio::GGUFTokenizer& tok, const pj::Value& texts) {
    pj::Value out = pj::Value::object(), all_ids = pj::Value::array(), decoded = pj::Value::array(), pieces = pj::Value::array(), single = pj::Value::array();
    for (const auto& t : texts.items()) {
        const std::vector<int> ids = tok.encode(t.as_string());
        all_ids.push_back(ids_json(ids));
        decoded.push_back(tok.decode(ids));
        pj::Value p = pj::Value::array(), s = pj::Value::array();
        for (const auto& x : pio::GGUFTokenizer::gpt2_pieces(t.as_string())) p.push_back(x);
        for (int id : ids) s.push_back(tok.decode_token(id));
        pieces.push_back(p);
        single.push_back(s);
    }
    out.set("ids", all_ids);
    out.set("decoded", decoded);
    out.set("pieces", pieces);
    out.set("single", single);
    return out;
}

// Token = one byte.  "echo" spells a fixed answer, "mirror" answers with the prompt it was given, "slow" takes 30 ms a token.
class FakeBackend : public ps::ModelBackend {
 public:
    explicit FakeBackend(std::string kind) : kind_(std::move(kind)) {
        architecture = "qwen3";
        model_name = kind_;
        size = 1234;
        parameter_size = "1B";
    }
    std::vector<int> encode(const std::string& text) override {
        std::vector<int> ids;
        for (unsigned char c : text) ids.push_back(c);
        return ids;
    }
    std::string decode_token(int id) override { return std::string(1, (char)id); }
    std::pair<double, double> generate(const std::vector<int>& prompt, const ps::GenerateOptions& opt, const std::function<bool(int)>& on_token) override {
        std::string answer = "hello world";
        if (kind_ == "mirror") {
            answer.clear();
            for (int t : prompt) answer.push_back((char)t);
            answer += "|" + std::to_string(opt.top_k) + "|" + std::to_string((int)(opt.temperature * 100));
        }
        if (kind_ == "slow") answer = std::string(200, 'z');
        if (kind_ == "tool") answer = "sure {\"tool_call\": {\"name\": \"add\", \"arguments\": {\"a\": 1, \"b\": 2}}} done";
        int n = 0;
        for (char c : answer) {
            if (n++ >= opt.num_predict) break;
            if (kind_ == "slow") std::this_thread::sleep_for(std::chrono::milliseconds(30));
            if (!on_token((unsigned char)c)) break;
        }
        return {0.001, 0.002};
    }

 private:
    std::string kind_;
};

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    const std::string mode = argv[1];
    try {
        if (mode == "json") {
            std::cout << pj::parse(slurp(argv[2])).dump() << "\n";
            return 0;
        }
        if (mode == "tokenize") {
            const pj::Value spec = pj::parse(slurp(argv[2]));
            std::vector<std::string> tokens, merges;
            std::vector<float> scores;
            std::vector<int> types;
            for (const auto& v : spec["tokens"].items()) tokens.push_back(v.as_string());
            for (const auto& v : spec["merges"].items()) merges.push_back(v.as_string());
            for (const auto& v : spec["scores"].items()) scores.push_back((float)v.as_double());
            for (const auto& v : spec["types"].items()) types.push_back((int)v.as_int());
            pio::GGUFTokenizer tok(tokens, spec["model"].as_string(), scores, merges, types, (int)spec["bos"].as_int(-1), (int)spec["eos"].as_int(-1),
                                   spec["add_bos"].as_bool(), spec["pre"].as_string());
            pj::Value out = run_texts(tok, spec["texts"]);
            if (spec["pre"].is_string()) {                               // the pieces of the named pattern too
                pj::Value styled = pj::Value::array();
                for (const auto& t : spec["texts"].items()) {
                    pj::Value p = pj::Value::array();
                    for (const auto& x : pio::GGUFTokenizer::pieces(t.as_string(), pio::GGUFTokenizer::style_of(spec["pre"].as_string()))) p.push_back(x);
                    styled.push_back(p);
                }
                out.set("styled_pieces", styled);
            }
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "gguf-tokenize") {
            pio::gguf::GGUFReader reader(argv[2]);
            const pio::GGUFTokenizer tok = pio::GGUFTokenizer::from_reader(reader);
            std::cout << run_texts(tok, pj::parse(slurp(argv[3]))).dump() << "\n";
            return 0;
        }
        if (mode == "hf-tokenize") {                 // DIR TEXTS.json
            pio::GGUFTokenizer tok;
            if (!pio::load_hf_tokenizer(argv[2], tok)) { std::cout << "null\n"; return 0; }
            std::cout << run_texts(tok, pj::parse(slurp(argv[3]))).dump() << "\n";
            return 0;
        }
        if (mode == "chat") {
            const pj::Value spec = pj::parse(slurp(argv[2]));
            pj::Value out = pj::Value::array();
            for (const auto& c : spec.items()) {
                if (c["messages"].is_array()) {
                    std::vector<pio::chat::Message> ms;
                    for (const auto& m : c["messages"].items()) ms.push_back({m["role"].as_string(), m["content"].as_string()});
                    out.push_back(pio::chat::render_messages(ms, c["arch"].as_string(), c["name"].as_string()));
                } else if (c["strip"].is_string()) {
                    out.push_back(pio::chat::strip_think(c["strip"].as_string()));
                } else {
                    const std::string sys = c["system"].as_string();
                    out.push_back(pio::chat::apply_chat_template(c["prompt"].as_string(), c["arch"].as_string(), c["name"].as_string(),
                                                                 c["system"].is_string() ? &sys : nullptr, c["no_think"].is_null() ? -1 : (int)c["no_think"].as_bool()));
                }
            }
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "dequant") {                     // TYPE FILE: the file's bytes as consecutive blocks of that GGML type, dequantised
            const uint32_t type = (uint32_t)std::atoi(argv[2]);
            std::ifstream f(argv[3], std::ios::binary);
            std::vector<uint8_t> raw((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
            int be, bb;
            pio::gguf::block_geometry(type, be, bb);
            pj::Value out = pj::Value::array();
            float y[256];
            for (size_t o = 0; o + (size_t)bb <= raw.size(); o += (size_t)bb) {
                const int n = pio::cpu_detail::dequant_block(type, raw.data() + o, y);
                for (int i = 0; i < n; ++i) out.push_back((double)y[i]);
            }
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "cpu-generate") {                // FILE|DIR N id id id ...: greedy ids and a few logits of the CPU decoder
            pio::GGUFCpuModel m;
            m.load(argv[2], 256);
            const int n_new = std::atoi(argv[3]);
            std::vector<int> prompt;
            for (int i = 4; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
            pj::Value out = pj::Value::object(), first = pj::Value::array();
            int pos = 0;
            for (int t : prompt) m.forward(t, pos++);
            const auto& lg = m.forward(prompt.back(), pos);          // one more step so that the probe is not the prompt's last
            for (int i = 0; i < 24; ++i) first.push_back((double)lg[(size_t)i]);
            out.set("probe_logits", first);
            out.set("probe_argmax", m.argmax());
            pio::GGUFCpuModel fresh;
            fresh.load(argv[2], 256);
            out.set("ids", ids_json(fresh.generate(prompt, n_new)));
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "model") {                       // model_loader.h: what a path holds
            namespace L = pio::loader;
            pj::Value out = pj::Value::object();
            out.set("detected", L::detect_format(argv[2]));
            const L::ModelWeights mw = L::load_model(argv[2]);
            out.set("format", mw.format);
            out.set("architecture", mw.architecture);
            pj::Value cfg = pj::Value::object(), tensors = pj::Value::object(), files = pj::Value::array();
            const auto& c = mw.config;
            cfg.set("hidden_size", (long long)c.hidden_size);
            cfg.set("num_layers", (long long)c.num_layers);
            cfg.set("num_heads", (long long)c.num_heads);
            cfg.set("num_kv_heads", (long long)c.num_kv_heads);
            cfg.set("intermediate_size", (long long)c.intermediate_size);
            cfg.set("vocab_size", (long long)c.vocab_size);
            cfg.set("head_dim", (long long)c.head_dim);
            cfg.set("context_length", (long long)c.context_length);
            cfg.set("rms_norm_eps", c.rms_norm_eps);
            cfg.set("rope_freq_base", c.rope_freq_base);
            cfg.set("tie_word_embeddings", c.tie_word_embeddings);
            out.set("config", cfg);
            for (const auto& name : mw.order) {
                const auto& t = mw.tensors.at(name);
                pj::Value e = pj::Value::object(), shape = pj::Value::array();
                for (auto d : t.shape) shape.push_back((long long)d);
                e.set("dtype", t.dtype);
                e.set("shape", shape);
                e.set("file", t.file);
                if (argc > 3) {                      // byte sums on request
                    unsigned long long sum = 0;
                    const auto bytes = L::read_tensor_bytes(mw, name);
                    for (uint8_t b : bytes) sum += b;
                    e.set("nbytes", (long long)bytes.size());
                    e.set("byte_sum", (long long)sum);
                }
                tensors.set(name, e);
            }
            out.set("tensors", tensors);
            for (const auto& f : mw.files) files.push_back(f);
            out.set("files", files);
            out.set("total_parameters", (long long)mw.total_parameters());
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "engine") {                      // the request queue over a fake backend
            ps::LLMEngine eng(std::make_shared<FakeBackend>("echo"));
            const int a = eng.submit_request("one", 3), b = eng.submit_request(std::vector<int>{'t', 'w', 'o'}, 5);
            pj::Value out = pj::Value::object();
            out.set("pending", (long long)eng.num_pending());
            out.set("first_step", eng.step());
            pj::Value polled = pj::Value::object();
            for (auto& kv : eng.poll_responses()) polled.set(std::to_string(kv.first), ids_json(kv.second));
            out.set("after_first", polled);
            out.set("second_step", eng.step());
            pj::Value polled2 = pj::Value::object();
            for (auto& kv : eng.poll_responses()) polled2.set(std::to_string(kv.first), ids_json(kv.second));
            out.set("after_second", polled2);
            out.set("empty_step", eng.step());
            out.set("ids", ids_json({a, b}));
            pj::Value texts = pj::Value::array();
            for (const auto& t : eng.generate({"x", "y"}, 4)) texts.push_back(t);
            out.set("generate", texts);
            std::cout << out.dump() << "\n";
            return 0;
        }
        if (mode == "serve") {
            ps::ServerConfig cfg;
            cfg.port = 0;
            cfg.worker_threads = 2;
            std::string gguf_file;
            for (int i = 2; i + 1 < argc; i += 2) {
                const std::string a = argv[i];
                if (a == "--workers") cfg.worker_threads = std::atoi(argv[i + 1]);
                if (a == "--queue-depth") cfg.max_queue_depth = std::atoi(argv[i + 1]);
                if (a == "--timeout-ms") cfg.server_timeout_ms = std::atoi(argv[i + 1]);
                if (a == "--model-dir") cfg.model_dirs.push_back(argv[i + 1]);
                if (a == "--max-body") cfg.max_body_bytes = (size_t)std::atol(argv[i + 1]);
                if (a == "--max-models") cfg.max_loaded_models = std::atoi(argv[i + 1]);
                if (a == "--gguf") gguf_file = argv[i + 1];
            }
            int loads = 0;
            // names found on disk load as fakes that remember how many loads there were (no GPU in this program)
            ps::PromeServe srv(cfg, [&cfg, &loads](const std::string& name) -> std::shared_ptr<ps::ModelBackend> {
                const std::string path = ps::store::resolve(name, cfg.model_dirs);
                auto b = std::make_shared<FakeBackend>("echo");
                b->size = ps::store::file_size(path);
                b->parameter_size = "load#" + std::to_string(++loads);
                return b;
            });
            for (const char* k : {"echo", "mirror", "slow", "tool"}) srv.handlers().add_backend(std::string(k) + ":1b", std::make_shared<FakeBackend>(k));
            if (!gguf_file.empty()) srv.handlers().add_backend("cpu-model", std::make_shared<ps::CpuBackend>(gguf_file, "cpu-model", 256));   // a real file on the CPU decoder
            srv.start();
            std::cout << "PORT " << srv.port() << std::endl;
            std::string line;
            while (std::getline(std::cin, line)) {
                if (line == "loaded") std::cout << "LOADED " << srv.handlers().loaded_models() << std::endl;
            }
            srv.stop();
            return 0;
        }
    } catch (const std::exception& e) {
        std::cerr << "error: " << e.what() << "\n";
        return 1;
    }
    return 2;
}
