// The serving-side headers need no libtorch and no CUDA: this program opens a GGUF file, prints what the model loader sees,
// tokenises a prompt with the file's own tokenizer, wraps it in the model's chat template and, with --generate N, continues
// it on the CPU reference decoder.
//
//   make -C examples/cpp tokenize && examples/cpp/tokenize MODEL.gguf "a prompt" [--generate N]
#include <cstdio>
#include <cstdlib>
#include <string>

#include <promethorch/chat.h>
#include <promethorch/gguf_cpu.h>
#include <promethorch/model_loader.h>
#include <promethorch/tokenizer.h>

namespace pio = promethorch::io;

int main(int argc, char** argv) {
    if (argc < 3) { std::fprintf(stderr, "usage: tokenize MODEL.gguf PROMPT [--generate N]\n"); return 2; }
    const std::string path = argv[1], prompt = argv[2];
    const int n_new = argc > 4 && std::string(argv[3]) == "--generate" ? std::atoi(argv[4]) : 0;
    try {
        const auto mw = pio::loader::load_model(path);
        std::printf("%s: format %s, architecture %s, %zu tensors, %lld parameters, %lld layers, hidden %lld\n", path.c_str(), mw.format.c_str(),
                    mw.architecture.c_str(), mw.tensors.size(), (long long)mw.total_parameters(), (long long)mw.config.num_layers, (long long)mw.config.hidden_size);
        pio::gguf::GGUFReader reader(path);
        const auto tok = pio::GGUFTokenizer::from_reader(reader);
        const std::string text = pio::chat::apply_chat_template(prompt, mw.architecture);
        const auto ids = tok.encode(text);
        std::printf("prompt in the chat template: %zu tokens:", ids.size());
        for (size_t i = 0; i < ids.size() && i < 24; ++i) std::printf(" %d", ids[i]);
        std::printf("%s\nround trip: %s\n", ids.size() > 24 ? " ..." : "", tok.decode(tok.encode(prompt)).c_str());
        if (n_new > 0) {
            pio::GGUFCpuModel model;
            model.load(path, 512);
            std::printf("greedy continuation on the CPU decoder: %s\n", tok.decode(model.generate(tok.encode(prompt), n_new), true, false).c_str());
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "tokenize: %s\n", e.what());
        return 1;
    }
    return 0;
}
