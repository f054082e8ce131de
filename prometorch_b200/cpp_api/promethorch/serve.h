// promethorch C++ API: PromeServe, an Ollama-compatible HTTP server (native counterpart of the reference's
// promeserve/{http_server,api_handlers,model_manager}.h).
//
// Routes: GET / (the chat page of web_root for a browser, liveness text otherwise), GET /api/version, GET /api/tags, GET /api/ps (loaded models and counters), POST /api/show,
// POST /api/generate, POST /api/chat, POST /api/embeddings (501), HEAD, OPTIONS with CORS.  Streaming answers are chunked application/x-ndjson: one object
// per token ({"model","created_at","response","done":false}, or "message":{"role","content"} for chat) and a final
// object with total_duration, load_duration, prompt_eval_count, prompt_eval_duration, eval_count, eval_duration in
// nanoseconds.  Back-pressure: a bounded queue in front of a fixed pool of workers; a full queue answers 503 with
// Retry-After: 1.  A request that outlives the server timeout ends with an in-stream {"error":"timeout","done":true}.
// One generation runs on a backend at a time unless the backend says it batches (concurrent()).
//
// The server knows models only through ModelBackend; gguf_backend.h binds the CUDA decode engine, tests bind a fake.
// Model names resolve inside the configured model directories and the Ollama store only: a request cannot name a path.
#pragma once
#include <arpa/inet.h>
#include <dirent.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/time.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <ctime>
#include <deque>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "chat.h"
#include "json.h"

namespace promethorch {
namespace serve {

inline const char* version() { return "0.1.0-promeserve"; }

struct GenerateOptions {
    int num_predict = 128;
    double temperature = 0.7;
    int top_k = 40;
    double top_p = 0.9;
    double repeat_penalty = 1.05;
    long long seed = 42;
    static GenerateOptions from_body(const json::Value& body) {
        GenerateOptions o;
        const json::Value& b = body["options"];
        if (b["num_predict"].is_number()) o.num_predict = (int)b["num_predict"].as_int();
        if (b["temperature"].is_number()) o.temperature = b["temperature"].as_double();
        if (b["top_k"].is_number()) o.top_k = (int)b["top_k"].as_int();
        if (b["top_p"].is_number()) o.top_p = b["top_p"].as_double();
        if (b["repeat_penalty"].is_number()) o.repeat_penalty = b["repeat_penalty"].as_double();
        if (b["seed"].is_number()) o.seed = b["seed"].as_int();
        return o;
    }
};

// What the handlers need from a model.
class ModelBackend {
 public:
    virtual ~ModelBackend() = default;
    std::string name = "model", architecture = "llama", format = "gguf", model_name, parameter_size;
    long long size = 0;
    virtual std::vector<int> encode(const std::string& text) = 0;
    virtual std::string decode_token(int id) = 0;
    // Prefill + decode; on_token(id) per generated token, false stops.  Returns {prompt seconds, decode seconds}.
    virtual std::pair<double, double> generate(const std::vector<int>& prompt, const GenerateOptions& opt, const std::function<bool(int)>& on_token) = 0;
    virtual bool concurrent() const { return false; }
};

struct ServerConfig {
    std::string host = "127.0.0.1";          // loopback by default; 0.0.0.0 serves other machines
    int port = 11434;                        // 0 = any free port (read it back from PromeServe::port())
    int worker_threads = 4;
    int max_queue_depth = 128;
    int server_timeout_ms = 60000;
    std::string device = "cuda";
    std::vector<std::string> model_dirs;
    int max_seq = 4096;
    int max_loaded_models = 2;               // resident at once; the least recently used one is dropped
    size_t max_body_bytes = 8u << 20;        // larger request bodies are answered 413
    std::string web_root;                    // folder whose index.html answers a browser's GET /; empty = liveness text only
};

class NotFound : public std::runtime_error {
 public:
    using std::runtime_error::runtime_error;
};

inline std::string now_iso() {
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    struct tm tmv;
    gmtime_r(&tv.tv_sec, &tmv);
    char buf[64];
    std::snprintf(buf, sizeof buf, "%04d-%02d-%02dT%02d:%02d:%02d.%06ldZ", tmv.tm_year + 1900, tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min,
                  tmv.tm_sec, (long)tv.tv_usec);
    return buf;
}

// ---------------------------------------------------------------------------------------------- model lookup on disk
namespace store {
inline bool is_file(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode); }
inline bool is_dir(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode); }
inline long long file_size(const std::string& p) { struct stat st; return ::stat(p.c_str(), &st) == 0 ? (long long)st.st_size : 0; }
inline std::vector<std::string> listdir(const std::string& d) {
    std::vector<std::string> out;
    if (DIR* dir = ::opendir(d.c_str())) {
        while (struct dirent* e = ::readdir(dir)) {
            const std::string n = e->d_name;
            if (n != "." && n != "..") out.push_back(n);
        }
        ::closedir(dir);
    }
    std::sort(out.begin(), out.end());
    return out;
}
inline std::string models_root() {
    if (const char* r = std::getenv("OLLAMA_MODELS")) return r;
    const char* home = std::getenv("HOME");
    return std::string(home ? home : "") + "/.ollama/models";
}
// The blob behind an Ollama name ("model" or "model:tag"): the manifest's layer of media type ...image.model.
inline std::string resolve_ollama(const std::string& name, const std::string& root = models_root()) {
    const size_t c = name.find(':');
    const std::string model = name.substr(0, c), tag = c == std::string::npos || c + 1 == name.size() ? "latest" : name.substr(c + 1);
    const std::string manifest = root + "/manifests/registry.ollama.ai/library/" + model + "/" + tag;
    if (!is_file(manifest)) throw NotFound("model '" + name + "' not found (looked for " + manifest + ")");
    std::ifstream f(manifest);
    std::stringstream ss;
    ss << f.rdbuf();
    const json::Value m = json::parse(ss.str());
    for (const auto& layer : m["layers"].items()) {
        const std::string& mt = layer["mediaType"].as_string();
        if (mt.size() >= 11 && mt.compare(mt.size() - 11, 11, "image.model") == 0) {
            std::string digest = layer["digest"].as_string();
            std::replace(digest.begin(), digest.end(), ':', '-');
            const std::string blob = root + "/blobs/" + digest;
            if (is_file(blob)) return blob;
            throw NotFound("blob for '" + name + "' is missing: " + blob);
        }
    }
    throw NotFound("manifest of '" + name + "' has no model layer");
}
// A request names models, not files: a name with a path separator or ".." is refused.
inline bool is_plain_name(const std::string& name) {
    return !name.empty() && name[0] != '/' && name.find('/') == std::string::npos && name.find('\\') == std::string::npos && name.find("..") == std::string::npos;
}
// <dir>/<name without tag>.gguf in one of `dirs`, else the Ollama store.
inline std::string resolve(const std::string& name, const std::vector<std::string>& dirs) {
    if (!is_plain_name(name)) throw NotFound("model '" + name + "' not found (paths are not accepted as model names)");
    const std::string stem = name.substr(0, name.find(':'));
    for (const auto& d : dirs)
        if (is_file(d + "/" + stem + ".gguf")) return d + "/" + stem + ".gguf";
    return resolve_ollama(name);
}
struct Listed { std::string name, path; long long size; };
inline std::vector<Listed> list_models(const std::vector<std::string>& dirs) {
    std::vector<Listed> out;
    const std::string root = models_root(), lib = root + "/manifests/registry.ollama.ai/library";
    for (const auto& model : listdir(lib))
        for (const auto& tag : listdir(lib + "/" + model)) {
            try {
                const std::string p = resolve_ollama(model + ":" + tag, root);
                out.push_back({model + ":" + tag, p, file_size(p)});
            } catch (const std::exception&) {
            }
        }
    for (const auto& d : dirs)
        for (const auto& fn : listdir(d))
            if (fn.size() > 5 && fn.compare(fn.size() - 5, 5, ".gguf") == 0) out.push_back({fn.substr(0, fn.size() - 5), d + "/" + fn, file_size(d + "/" + fn)});
    return out;
}
}  // namespace store

// ---------------------------------------------------------------------------------------------- socket helpers
namespace net {
inline bool send_all(int fd, const char* p, size_t n) {
    while (n) {
        const ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
        if (w <= 0) return false;
        p += w;
        n -= (size_t)w;
    }
    return true;
}
inline bool send_all(int fd, const std::string& s) { return send_all(fd, s.data(), s.size()); }
inline const char* reason(int status) {
    switch (status) {
        case 200: return "OK";
        case 204: return "No Content";
        case 400: return "Bad Request";
        case 404: return "Not Found";
        case 413: return "Request Entity Too Large";
        case 500: return "Internal Server Error";
        case 501: return "Not Implemented";
        case 503: return "Service Unavailable";
        default: return "Status";
    }
}
inline const char* cors() {
    return "Access-Control-Allow-Origin: *\r\nAccess-Control-Allow-Methods: POST, GET, OPTIONS\r\nAccess-Control-Allow-Headers: Content-Type, Authorization\r\n";
}
inline bool send_response(int fd, int status, const std::string& body, const char* ctype = "application/json", const char* extra = "") {
    std::string h = "HTTP/1.1 " + std::to_string(status) + " " + reason(status) + "\r\nContent-Type: " + ctype + "\r\nContent-Length: " +
                    std::to_string(body.size()) + "\r\nConnection: close\r\n" + cors() + extra + "\r\n";
    return send_all(fd, h + body);
}
}  // namespace net

// Chunked-transfer NDJSON writer over a socket.
class StreamWriter {
 public:
    explicit StreamWriter(int fd) : fd_(fd) {}
    bool write(const json::Value& obj) {
        if (!open_) return false;
        const std::string data = obj.dump() + "\n";
        char len[32];
        std::snprintf(len, sizeof len, "%zx\r\n", data.size());
        open_ = net::send_all(fd_, std::string(len) + data + "\r\n");
        return open_;
    }
    void finish() {
        if (open_) net::send_all(fd_, "0\r\n\r\n");
        open_ = false;
    }
    bool is_open() const { return open_; }

 private:
    int fd_;
    bool open_ = true;
};

// ---------------------------------------------------------------------------------------------- handlers
class ApiHandlers {
 public:
    using Loader = std::function<std::shared_ptr<ModelBackend>(const std::string&)>;
    ApiHandlers(const ServerConfig& cfg, Loader loader) : cfg_(cfg), loader_(std::move(loader)) {}

    // A backend handed in by the host program; never evicted.
    void add_backend(const std::string& name, std::shared_ptr<ModelBackend> b) {
        std::lock_guard<std::mutex> g(table_mutex_);
        b->name = name;
        backends_.push_back({name, std::move(b)});
        pinned_.insert(name);
    }
    std::shared_ptr<ModelBackend> ensure_model(const std::string& name) {
        if (auto b = lookup(name)) return b;
        if (!loader_) throw NotFound("model '" + name + "' not found");
        std::lock_guard<std::mutex> load(load_mutex_);            // one load at a time; a second request for the same name finds it cached
        if (auto b = lookup(name)) return b;
        for (;;) {
            std::shared_ptr<ModelBackend> victim;
            {
                std::lock_guard<std::mutex> g(table_mutex_);
                size_t loaded = 0, first = backends_.size();
                for (size_t i = 0; i < backends_.size(); ++i)
                    if (!pinned_.count(backends_[i].first)) { if (first == backends_.size()) first = i; ++loaded; }
                if (loaded < (size_t)std::max(1, cfg_.max_loaded_models)) break;
                victim = backends_[first].second;
                backends_.erase(backends_.begin() + (long)first);
            }
            std::lock_guard<std::mutex> gen(generate_mutex_);     // never drop a model in the middle of its generation
            victim.reset();
        }
        std::shared_ptr<ModelBackend> b = loader_(name);
        if (!b) throw NotFound("model '" + name + "' not found");
        b->name = name;
        std::lock_guard<std::mutex> g(table_mutex_);
        backends_.push_back({name, b});
        return b;
    }
    size_t loaded_models() { std::lock_guard<std::mutex> g(table_mutex_); return backends_.size(); }

    json::Value tags() {
        json::Value models = json::Value::array();
        std::set<std::string> seen;
        {
            std::lock_guard<std::mutex> g(table_mutex_);
            for (const auto& kv : backends_) {
                seen.insert(kv.first);
                models.push_back(model_entry(kv.first, kv.second->size, kv.second->architecture, kv.second->format, kv.second->parameter_size));
            }
        }
        try {
            for (const auto& m : store::list_models(cfg_.model_dirs))
                if (!seen.count(m.name)) models.push_back(model_entry(m.name, m.size, "", "gguf", ""));
        } catch (const std::exception&) {
        }
        json::Value out = json::Value::object();
        out.set("models", models);
        return out;
    }
    // Loaded models and the server's counters (the shape of Ollama's /api/ps, plus "stats").
    json::Value ps() {
        json::Value models = json::Value::array();
        std::lock_guard<std::mutex> g(table_mutex_);
        for (const auto& kv : backends_) {
            json::Value m = model_entry(kv.first, kv.second->size, kv.second->architecture, kv.second->format, kv.second->parameter_size);
            m.set("expires_at", "");
            m.set("size_vram", kv.second->size);
            models.push_back(m);
        }
        json::Value out = json::Value::object(), st = json::Value::object();
        st.set("requests", (long long)requests_.load());
        st.set("tokens_generated", (long long)tokens_generated_.load());
        st.set("prompt_tokens", (long long)prompt_tokens_.load());
        st.set("timeouts", (long long)timeouts_.load());
        out.set("models", models);
        out.set("stats", st);
        return out;
    }
    json::Value show(const json::Value& body) {
        const std::string name = body["model"].is_string() ? body["model"].as_string() : body["name"].as_string();
        auto b = ensure_model(name);
        json::Value out = json::Value::object(), details = json::Value::object(), info = json::Value::object();
        details.set("family", b->architecture);
        details.set("format", b->format);
        details.set("parameter_size", b->parameter_size);
        info.set("general.architecture", b->architecture);
        info.set("general.name", b->model_name);
        out.set("modelfile", "");
        out.set("parameters", "");
        out.set("template", "");
        out.set("details", details);
        out.set("model_info", info);
        return out;
    }
    // writer == nullptr: the whole answer comes back as one object.
    json::Value generate(const json::Value& body, StreamWriter* writer) {
        const std::string model = body["model"].as_string();
        auto backend = ensure_model(model);
        std::string prompt = body["prompt"].as_string();
        const bool templated = prompt.find("<|im_start|>") != std::string::npos || prompt.find("[INST]") != std::string::npos ||
                               prompt.find("<|start_header_id|>") != std::string::npos;
        if (!body["raw"].as_bool(false) && !templated) {
            const std::string sys = body["system"].as_string();
            prompt = io::chat::apply_chat_template(prompt, backend->architecture, backend->model_name, body["system"].is_string() ? &sys : nullptr);
        }
        auto emit = [&](const std::string& piece) {
            if (!writer) return true;
            json::Value o = json::Value::object();
            o.set("model", model);
            o.set("created_at", now_iso());
            o.set("response", piece);
            o.set("done", false);
            return writer->write(o);
        };
        Run r = run(*backend, prompt, GenerateOptions::from_body(body), emit);
        json::Value fin = json::Value::object();
        if (r.timed_out) {
            fin.set("error", "timeout");
            fin.set("done", true);
        } else {
            fin.set("model", model);
            fin.set("created_at", now_iso());
            fin.set("response", writer ? std::string() : r.text);
            fin.set("done", true);
            add_stats(fin, r);
        }
        if (writer) { writer->write(fin); writer->finish(); }
        return fin;
    }
    json::Value chat(const json::Value& body, StreamWriter* writer) {
        const std::string model = body["model"].as_string();
        auto backend = ensure_model(model);
        std::vector<io::chat::Message> messages;
        const bool tools = body["tools"].is_array() && body["tools"].size() > 0;
        if (tools)
            messages.push_back({"system", "You may call a tool by answering with a JSON object {\"tool_call\": {\"name\": ..., \"arguments\": {...}}}. Tools: " +
                                              body["tools"].dump()});
        for (const auto& m : body["messages"].items()) messages.push_back({m["role"].as_string(), m["content"].as_string()});
        auto emit = [&](const std::string& piece) {
            if (!writer) return true;
            json::Value o = json::Value::object(), msg = json::Value::object();
            msg.set("role", "assistant");
            msg.set("content", piece);
            o.set("model", model);
            o.set("created_at", now_iso());
            o.set("message", msg);
            o.set("done", false);
            return writer->write(o);
        };
        Run r = run(*backend, io::chat::render_messages(messages, backend->architecture, backend->model_name), GenerateOptions::from_body(body), emit);
        json::Value fin = json::Value::object();
        if (r.timed_out) {
            fin.set("error", "timeout");
            fin.set("done", true);
        } else {
            json::Value msg = json::Value::object();
            msg.set("role", "assistant");
            msg.set("content", writer ? std::string() : r.text);
            if (tools) {
                json::Value call = parse_tool_call(r.text);
                if (!call.is_null()) {
                    json::Value fn = json::Value::object(), calls = json::Value::array();
                    fn.set("function", call);
                    calls.push_back(fn);
                    msg.set("tool_calls", calls);
                }
            }
            fin.set("model", model);
            fin.set("created_at", now_iso());
            fin.set("message", msg);
            fin.set("done", true);
            add_stats(fin, r);
        }
        if (writer) { writer->write(fin); writer->finish(); }
        return fin;
    }
    // The object after {"tool_call": in the model's answer, or null.
    static json::Value parse_tool_call(const std::string& text) {
        const size_t i = text.find("{\"tool_call\"");
        if (i == std::string::npos) return json::Value();
        int depth = 0;
        for (size_t j = i; j < text.size(); ++j) {
            depth += text[j] == '{';
            depth -= text[j] == '}';
            if (depth == 0) {
                try {
                    const json::Value v = json::parse(text.substr(i, j + 1 - i));
                    return v["tool_call"];
                } catch (const std::exception&) {
                    return json::Value();
                }
            }
        }
        return json::Value();
    }

 private:
    struct Run {
        std::string text;
        bool timed_out = false;
        int n_prompt = 0, n_eval = 0;
        double prompt_s = 0, eval_s = 0;
    };
    static json::Value model_entry(const std::string& name, long long size, const std::string& family, const std::string& format, const std::string& psize) {
        json::Value m = json::Value::object(), d = json::Value::object();
        d.set("family", family);
        d.set("format", format);
        d.set("parameter_size", psize);
        m.set("name", name);
        m.set("model", name);
        m.set("modified_at", now_iso());
        m.set("size", size);
        m.set("digest", "");
        m.set("details", d);
        return m;
    }
    static void add_stats(json::Value& fin, const Run& r) {
        fin.set("total_duration", (long long)((r.prompt_s + r.eval_s) * 1e9));
        fin.set("load_duration", 0);
        fin.set("prompt_eval_count", r.n_prompt);
        fin.set("prompt_eval_duration", (long long)(r.prompt_s * 1e9));
        fin.set("eval_count", r.n_eval);
        fin.set("eval_duration", (long long)(r.eval_s * 1e9));
    }
    std::shared_ptr<ModelBackend> lookup(const std::string& name) {
        std::lock_guard<std::mutex> g(table_mutex_);
        for (size_t i = 0; i < backends_.size(); ++i)
            if (backends_[i].first == name) {
                auto kv = backends_[i];
                backends_.erase(backends_.begin() + (long)i);
                backends_.push_back(kv);                           // most recently used goes last
                return kv.second;
            }
        const std::string base = name.substr(0, name.find(':'));
        for (const auto& kv : backends_)
            if (kv.first.substr(0, kv.first.find(':')) == base) return kv.second;
        return nullptr;
    }
    Run run(ModelBackend& backend, const std::string& prompt, const GenerateOptions& opt, const std::function<bool(const std::string&)>& emit) {
        Run r;
        std::vector<int> ids = backend.encode(prompt);
        if (ids.empty()) ids.push_back(0);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(cfg_.server_timeout_ms);
        auto on_token = [&](int id) {
            if (std::chrono::steady_clock::now() > deadline) { r.timed_out = true; return false; }
            ++r.n_eval;
            const std::string piece = backend.decode_token(id);
            r.text += piece;
            return emit(piece);
        };
        std::unique_lock<std::mutex> gen(generate_mutex_, std::defer_lock);
        if (!backend.concurrent()) gen.lock();
        const auto t = backend.generate(ids, opt, on_token);
        r.n_prompt = (int)ids.size();
        r.prompt_s = t.first;
        r.eval_s = t.second;
        ++requests_;
        tokens_generated_ += r.n_eval;
        prompt_tokens_ += r.n_prompt;
        timeouts_ += r.timed_out ? 1 : 0;
        return r;
    }

    ServerConfig cfg_;
    Loader loader_;
    std::vector<std::pair<std::string, std::shared_ptr<ModelBackend>>> backends_;      // least recently used first
    std::set<std::string> pinned_;
    std::mutex table_mutex_, load_mutex_, generate_mutex_;
    std::atomic<long long> requests_{0}, tokens_generated_{0}, prompt_tokens_{0}, timeouts_{0};
};

// ---------------------------------------------------------------------------------------------- request queue
// submit_request / step / poll_responses / generate over one backend (the call names of the reference's
// torch::serve::LLMEngine, torch/serve/llm.h:299-420).  Requests are served in arrival order, one per step().
class LLMEngine {
 public:
    struct Request {
        int id = 0;
        std::vector<int> prompt, output;
        GenerateOptions options;
        bool done = false;
    };
    explicit LLMEngine(std::shared_ptr<ModelBackend> backend) : backend_(std::move(backend)) {}

    int submit_request(const std::vector<int>& prompt_ids, int max_tokens = 32, double temperature = 0.0, int top_k = 0) {
        Request r;
        r.id = next_++;
        r.prompt = prompt_ids;
        r.options.num_predict = max_tokens;
        r.options.temperature = temperature;
        r.options.top_k = top_k > 0 ? top_k : 40;
        r.options.repeat_penalty = 1.0;
        std::lock_guard<std::mutex> g(m_);
        queue_.push_back(std::move(r));
        return queue_.back().id;
    }
    int submit_request(const std::string& prompt, int max_tokens = 32, double temperature = 0.0, int top_k = 0) {
        return submit_request(backend_->encode(prompt), max_tokens, temperature, top_k);
    }
    size_t num_pending() { std::lock_guard<std::mutex> g(m_); return queue_.size(); }
    // Serves the oldest request; returns how many tokens it produced (0 when the queue is empty).
    int step() {
        Request r;
        {
            std::lock_guard<std::mutex> g(m_);
            if (queue_.empty()) return 0;
            r = std::move(queue_.front());
            queue_.pop_front();
        }
        backend_->generate(r.prompt, r.options, [&r](int id) {
            r.output.push_back(id);
            return (int)r.output.size() < r.options.num_predict;
        });
        r.done = true;
        const int n = (int)r.output.size();
        std::lock_guard<std::mutex> g(m_);
        finished_[r.id] = std::move(r);
        return n;
    }
    // Finished requests since the last call: id -> generated ids.
    std::map<int, std::vector<int>> poll_responses() {
        std::map<int, std::vector<int>> out;
        std::lock_guard<std::mutex> g(m_);
        for (auto& kv : finished_) out[kv.first] = std::move(kv.second.output);
        finished_.clear();
        return out;
    }
    std::vector<std::string> generate(const std::vector<std::string>& prompts, int max_tokens = 32, double temperature = 0.0, int top_k = 0) {
        std::vector<int> ids;
        for (const auto& p : prompts) ids.push_back(submit_request(p, max_tokens, temperature, top_k));
        std::map<int, std::vector<int>> res;
        while (num_pending()) {
            step();
            for (auto& kv : poll_responses()) res[kv.first] = std::move(kv.second);
        }
        std::vector<std::string> out;
        for (int id : ids) {
            std::string text;
            for (int t : res[id]) text += backend_->decode_token(t);
            out.push_back(text);
        }
        return out;
    }

 private:
    std::shared_ptr<ModelBackend> backend_;
    std::deque<Request> queue_;
    std::map<int, Request> finished_;
    std::mutex m_;
    int next_ = 0;
};

// ---------------------------------------------------------------------------------------------- HTTP
// Blocking accept loop + fixed worker pool + bounded queue (503 when full).
class HttpServer {
 public:
    HttpServer(const ServerConfig& cfg, ApiHandlers& handlers) : cfg_(cfg), h_(handlers) {}
    ~HttpServer() { stop(); }
    int port() const { return port_; }

    void start() {
        listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
        if (listen_fd_ < 0) throw std::runtime_error("PromeServe: socket() failed");
        int one = 1;
        ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
        sockaddr_in addr{};
        addr.sin_family = AF_INET;
        addr.sin_port = htons((uint16_t)cfg_.port);
        if (::inet_pton(AF_INET, cfg_.host.c_str(), &addr.sin_addr) != 1) throw std::runtime_error("PromeServe: bad bind address " + cfg_.host);
        if (::bind(listen_fd_, (sockaddr*)&addr, sizeof addr) != 0) throw std::runtime_error("PromeServe: cannot bind " + cfg_.host + ":" + std::to_string(cfg_.port));
        socklen_t len = sizeof addr;
        ::getsockname(listen_fd_, (sockaddr*)&addr, &len);
        port_ = ntohs(addr.sin_port);
        if (::listen(listen_fd_, 128) != 0) throw std::runtime_error("PromeServe: listen() failed");
        running_ = true;
        for (int i = 0; i < std::max(1, cfg_.worker_threads); ++i) threads_.emplace_back([this] { worker(); });
        threads_.emplace_back([this] { accept_loop(); });
    }
    void stop() {
        if (!running_.exchange(false)) return;
        ::shutdown(listen_fd_, SHUT_RDWR);
        ::close(listen_fd_);
        {
            std::lock_guard<std::mutex> g(m_);
            stopping_ = true;
        }
        cv_.notify_all();
        for (auto& t : threads_)
            if (t.joinable()) t.join();
        threads_.clear();
        for (int fd : q_) ::close(fd);
        q_.clear();
    }

 private:
    void accept_loop() {
        while (running_) {
            const int fd = ::accept(listen_fd_, nullptr, nullptr);
            if (fd < 0) {
                if (!running_) return;
                continue;
            }
            bool queued = false;
            {
                std::lock_guard<std::mutex> g(m_);
                if ((int)q_.size() < cfg_.max_queue_depth) { q_.push_back(fd); queued = true; }
            }
            if (queued) cv_.notify_one();
            else {
                net::send_all(fd, "HTTP/1.1 503 Service Unavailable\r\nRetry-After: 1\r\nContent-Length: 0\r\nConnection: close\r\n\r\n");
                ::close(fd);
            }
        }
    }
    void worker() {
        for (;;) {
            int fd;
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [this] { return stopping_ || !q_.empty(); });
                if (stopping_) return;
                fd = q_.front();
                q_.pop_front();
            }
            struct timeval tv;
            tv.tv_sec = cfg_.server_timeout_ms / 1000;
            tv.tv_usec = (cfg_.server_timeout_ms % 1000) * 1000;
            ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
            ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);
            int one = 1;
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
            try {
                handle(fd);
            } catch (const std::exception&) {
            }
            ::shutdown(fd, SHUT_WR);
            ::close(fd);
        }
    }
    struct Request {
        std::string method, path, body;
        std::map<std::string, std::string> headers;
        bool too_large = false;
    };
    static std::string lower(std::string s) { for (auto& c : s) c = (char)std::tolower((unsigned char)c); return s; }
    static bool read_file(const std::string& path, std::string& out) {
        std::FILE* f = std::fopen(path.c_str(), "rb");
        if (!f) return false;
        char buf[16384];
        size_t n;
        while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) out.append(buf, n);
        std::fclose(f);
        return true;
    }
    static std::string trim(const std::string& s) {
        size_t a = 0, b = s.size();
        while (a < b && std::isspace((unsigned char)s[a])) ++a;
        while (b > a && std::isspace((unsigned char)s[b - 1])) --b;
        return s.substr(a, b - a);
    }
    bool read_request(int fd, Request& r) const {
        std::string buf;
        size_t end = std::string::npos;
        char tmp[4096];
        while ((end = buf.find("\r\n\r\n")) == std::string::npos) {
            if (buf.size() > 65536) return false;
            const ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
            if (n <= 0) return false;
            buf.append(tmp, (size_t)n);
        }
        std::istringstream head(buf.substr(0, end));
        std::string line;
        if (!std::getline(head, line)) return false;
        std::istringstream first(line);
        std::string target;
        first >> r.method >> target;
        for (auto& c : r.method) c = (char)std::toupper((unsigned char)c);
        r.path = target.substr(0, target.find('?'));
        while (std::getline(head, line)) {
            const size_t c = line.find(':');
            if (c != std::string::npos) r.headers[lower(trim(line.substr(0, c)))] = trim(line.substr(c + 1));
        }
        long long n = 0;
        if (r.headers.count("content-length")) {
            char* e = nullptr;
            n = std::strtoll(r.headers["content-length"].c_str(), &e, 10);
            if (e == r.headers["content-length"].c_str() || *e != 0) n = -1;
        }
        if (n < 0 || (size_t)n > cfg_.max_body_bytes) { r.too_large = true; return true; }
        r.body = buf.substr(end + 4);
        while (r.body.size() < (size_t)n) {
            const ssize_t k = ::recv(fd, tmp, std::min(sizeof tmp, (size_t)n - r.body.size()), 0);
            if (k <= 0) return false;
            r.body.append(tmp, (size_t)k);
        }
        r.body.resize((size_t)n);
        return true;
    }
    static std::string error_json(const std::string& what) {
        json::Value o = json::Value::object();
        o.set("error", what);
        return o.dump();
    }
    void handle(int fd) {
        Request r;
        if (!read_request(fd, r)) return;
        if (r.too_large) { net::send_response(fd, 413, error_json("request body too large")); return; }
        if (lower(r.headers["transfer-encoding"]).find("chunked") != std::string::npos) {
            net::send_response(fd, 400, error_json("chunked request bodies are not supported: send Content-Length"));
            return;
        }
        if (r.method == "OPTIONS") { net::send_response(fd, 204, ""); return; }
        if (r.method == "HEAD") { net::send_response(fd, (r.path == "/" || r.path == "/api/version" || r.path == "/api/tags") ? 200 : 404, ""); return; }
        if (r.method == "GET" && (r.path == "/" || r.path == "/index.html")) {
            // a browser gets the chat page (the reference serves promeserve/web/index.html, api_handlers.h:400-430); other clients the liveness text
            const bool wants_page = r.path != "/" || r.headers["accept"].find("text/html") != std::string::npos;
            std::string page;
            if (wants_page && !cfg_.web_root.empty() && read_file(cfg_.web_root + "/index.html", page)) net::send_response(fd, 200, page, "text/html; charset=utf-8");
            else if (r.path != "/") net::send_response(fd, 404, error_json("not found"));
            else net::send_response(fd, 200, "PromeServe is running", "text/plain");
            return;
        }
        if (r.method == "GET" && r.path == "/api/version") {
            json::Value o = json::Value::object();
            o.set("version", version());
            net::send_response(fd, 200, o.dump());
            return;
        }
        if (r.method == "GET" && r.path == "/api/tags") { net::send_response(fd, 200, h_.tags().dump()); return; }
        if (r.method == "GET" && r.path == "/api/ps") { net::send_response(fd, 200, h_.ps().dump()); return; }
        if (r.method == "POST" && (r.path == "/api/embeddings" || r.path == "/api/embed")) {
            net::send_response(fd, 501, error_json("embeddings are not implemented"));
            return;
        }
        if (r.method == "POST" && (r.path == "/api/generate" || r.path == "/api/chat" || r.path == "/api/show")) {
            json::Value body;
            try {
                body = json::parse(r.body.empty() ? "{}" : r.body);
            } catch (const std::exception&) {
                net::send_response(fd, 400, error_json("invalid JSON"));
                return;
            }
            try {
                if (r.path == "/api/show") { net::send_response(fd, 200, h_.show(body).dump()); return; }
                h_.ensure_model(body["model"].as_string());
            } catch (const NotFound& e) {
                net::send_response(fd, 404, error_json(e.what()));
                return;
            } catch (const std::exception& e) {
                net::send_response(fd, 500, error_json(e.what()));
                return;
            }
            const bool is_generate = r.path == "/api/generate";
            const bool stream = body["stream"].is_null() ? true : body["stream"].as_bool(true);
            if (stream) {
                net::send_all(fd, std::string("HTTP/1.1 200 OK\r\nContent-Type: application/x-ndjson\r\nTransfer-Encoding: chunked\r\nConnection: close\r\n") +
                                      net::cors() + "\r\n");
                StreamWriter w(fd);
                try {
                    if (is_generate) h_.generate(body, &w);
                    else h_.chat(body, &w);
                } catch (const std::exception& e) {          // errors travel in-stream
                    json::Value o = json::Value::object();
                    o.set("error", e.what());
                    o.set("done", true);
                    w.write(o);
                    w.finish();
                }
                return;
            }
            try {
                net::send_response(fd, 200, (is_generate ? h_.generate(body, nullptr) : h_.chat(body, nullptr)).dump());
            } catch (const std::exception& e) {
                net::send_response(fd, 500, error_json(e.what()));
            }
            return;
        }
        net::send_response(fd, 404, error_json("not found"));
    }

    ServerConfig cfg_;
    ApiHandlers& h_;
    int listen_fd_ = -1, port_ = 0;
    std::atomic<bool> running_{false};
    bool stopping_ = false;
    std::mutex m_;
    std::condition_variable cv_;
    std::deque<int> q_;
    std::vector<std::thread> threads_;
};

class PromeServe {
 public:
    explicit PromeServe(ServerConfig cfg = {}, ApiHandlers::Loader loader = nullptr)
        : cfg_(std::move(cfg)), handlers_(cfg_, std::move(loader)), http_(cfg_, handlers_) {}
    ApiHandlers& handlers() { return handlers_; }
    const ServerConfig& config() const { return cfg_; }
    void start() { http_.start(); }
    void stop() { http_.stop(); }
    int port() const { return http_.port(); }

 private:
    ServerConfig cfg_;
    ApiHandlers handlers_;
    HttpServer http_;
};

}  // namespace serve
}  // namespace promethorch
