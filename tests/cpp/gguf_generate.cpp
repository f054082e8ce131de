// Generates tokens from a GGUF file through the C++ GGUFModel (promethorch/gguf.h) and prints their ids:
//   gguf_generate <file.gguf> <n_new> <prompt id> [<prompt id> ...]
#include <promethorch/gguf.h>

#include <cstdio>
#include <cstdlib>

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: %s file.gguf n_new id [id ...]\n", argv[0]);
        return 2;
    }
    try {
        promethorch::io::GGUFModel model;
        model.load(argv[1], 256);
        std::vector<int> prompt;
        for (int i = 3; i < argc; ++i) prompt.push_back(std::atoi(argv[i]));
        const std::vector<int> out = model.generate(prompt, std::atoi(argv[2]));
        std::printf("IDS");
        for (int t : out) std::printf(" %d", t);
        std::printf("\n");
        // the stepwise entry point must agree with the scripted run on the first token
        int next = -1;
        for (size_t p = 0; p < prompt.size(); ++p) next = model.forward_decode(prompt[p], (int)p);
        std::printf("STEP %d\n", next);
        std::printf("ARCH %s layers %d hidden %d weights %zu\n", model.config.architecture.c_str(), model.config.num_layers,
                    model.config.hidden_size, model.weight_bytes());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
