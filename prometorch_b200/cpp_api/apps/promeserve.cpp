// promeserve: the Ollama-compatible server as a native program.
//
//   promeserve --port 11434 --device cuda|cpu --model NAME --workers N --queue-depth N --timeout-ms MS --model-dir DIR
//
// The flags are the reference's (promeserve/main.cpp:40-105) plus --host, --model-dir (repeatable), --max-seq,
// --max-models and --web-root (the folder whose index.html a browser gets at /; by default web/ beside the program,
// else ../serve/web, which is where the page sits in the source tree).  --model is loaded before the port opens and stays
// resident; it may be a path to a .gguf file or, with --device cpu, to a Hugging Face directory (config.json, safetensors,
// tokenizer files); requests may only use names.
// Build: g++ -std=c++17 -O3 promeserve.cpp -I<cpp_api> -I<cuda>/include -L<lib> -lptb200 -lcudart -lpthread
#include <csignal>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unistd.h>

#include "promethorch/gguf_backend.h"
#include "promethorch/gguf_cpu.h"

namespace ps = promethorch::serve;

static volatile std::sig_atomic_t g_stop = 0;
static void on_signal(int) { g_stop = 1; }

int main(int argc, char** argv) {
    ps::ServerConfig cfg;
    std::string model;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto val = [&]() -> std::string {
            if (i + 1 >= argc) { std::fprintf(stderr, "promeserve: %s needs a value\n", a.c_str()); std::exit(2); }
            return argv[++i];
        };
        if (a == "--host") cfg.host = val();
        else if (a == "--port") cfg.port = std::atoi(val().c_str());
        else if (a == "--device") cfg.device = val();
        else if (a == "--model") model = val();
        else if (a == "--workers") cfg.worker_threads = std::atoi(val().c_str());
        else if (a == "--queue-depth") cfg.max_queue_depth = std::atoi(val().c_str());
        else if (a == "--timeout-ms") cfg.server_timeout_ms = std::atoi(val().c_str());
        else if (a == "--model-dir") cfg.model_dirs.push_back(val());
        else if (a == "--max-seq") cfg.max_seq = std::atoi(val().c_str());
        else if (a == "--max-models") cfg.max_loaded_models = std::atoi(val().c_str());
        else if (a == "--web-root") cfg.web_root = val();
        else if (a == "--fp16-weights") {}                       // accepted for compatibility: weights stay in their file format
        else if (a == "--help" || a == "-h") {
            std::printf("usage: promeserve [--host A] [--port N] [--device cuda|cpu] [--model NAME|FILE.gguf] [--workers N] [--queue-depth N]\n"
                        "                  [--timeout-ms MS] [--model-dir DIR]... [--max-seq N] [--max-models N] [--web-root DIR]\n");
            return 0;
        } else { std::fprintf(stderr, "promeserve: unknown flag %s\n", a.c_str()); return 2; }
    }
    if (cfg.web_root.empty()) {
        char exe[4096];
        const ssize_t n = ::readlink("/proc/self/exe", exe, sizeof exe - 1);
        if (n > 0) {
            std::string dir(exe, (size_t)n);
            dir.resize(dir.find_last_of('/'));
            for (const char* rel : {"/web", "/../serve/web"})
                if (ps::store::is_file(dir + rel + "/index.html")) { cfg.web_root = dir + rel; break; }
        }
    }
    if (cfg.device != "cuda" && cfg.device != "cpu") { std::fprintf(stderr, "promeserve: --device is cuda or cpu\n"); return 2; }
    const bool on_cpu = cfg.device == "cpu";                  // the fp32 reference decoder: for checking and for machines without a GPU
    auto make = [&](const std::string& path, const std::string& name) -> std::shared_ptr<ps::ModelBackend> {
        if (on_cpu) return std::make_shared<ps::CpuBackend>(path, name, cfg.max_seq);
        if (ps::store::is_dir(path))
            throw std::runtime_error(path + " is a Hugging Face directory: this program serves those with --device cpu (on a GPU, python -m prometorch_b200.serve does)");
        return std::make_shared<ps::GGUFBackend>(path, name, cfg.max_seq);
    };
    try {
        ps::PromeServe srv(cfg, [&](const std::string& name) { return make(ps::store::resolve(name, cfg.model_dirs), name); });
        if (!model.empty()) {
            if (ps::store::is_file(model) || ps::store::is_file(model + "/config.json")) {     // a .gguf file, or a Hugging Face directory
                while (model.size() > 1 && model.back() == '/') model.pop_back();
                std::string name = model.substr(model.find_last_of('/') + 1);
                if (name.size() > 5 && name.compare(name.size() - 5, 5, ".gguf") == 0) name.resize(name.size() - 5);
                srv.handlers().add_backend(name, make(model, name));
                std::printf("[PromeServe] loaded %s as '%s'\n", model.c_str(), name.c_str());
            } else {
                srv.handlers().add_backend(model, make(ps::store::resolve(model, cfg.model_dirs), model));
                std::printf("[PromeServe] loaded '%s'\n", model.c_str());
            }
        }
        srv.start();
        std::printf("[PromeServe] listening on %s:%d (%s)\n", cfg.host.c_str(), srv.port(), on_cpu ? "cpu" : "cuda");
        std::fflush(stdout);
        std::signal(SIGINT, on_signal);
        std::signal(SIGTERM, on_signal);
        while (!g_stop) ::usleep(100000);
        srv.stop();
    } catch (const std::exception& e) {
        std::fprintf(stderr, "promeserve: %s\n", e.what());
        return 1;
    }
    return 0;
}
