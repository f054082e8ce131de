// Every element-wise optimizer of the C++ API run for a few steps on a fixed, formula-made sequence of gradients; the final
// parameters are printed so that the Python optimizers can be run on the same sequence and compared (the two are separate
// implementations of the same rules).  Output: one line per optimizer, "NAME v v v ...".
#include <cmath>
#include <cstdio>

#include <promethorch/torch.h>

namespace pt = promethorch;

static pt::Tensor start(std::vector<int64_t> shape, double phase) {
    const int64_t n = c10::multiply_integers(shape);
    auto i = pt::arange(n, pt::kDouble);
    return (pt::sin(i * 0.37 + phase) + 0.1 * i / (double)n).to(pt::kFloat).reshape(shape);
}
static pt::Tensor gradient(std::vector<int64_t> shape, int step, double phase) {
    const int64_t n = c10::multiply_integers(shape);
    auto i = pt::arange(n, pt::kDouble);
    return (pt::cos(i * 0.21 + 0.9 * step + phase) * (1.0 + 0.1 * step)).to(pt::kFloat).reshape(shape);
}

template <typename Opt, typename Options>
static void run(const char* name, Options o, int steps = 6) {
    auto w = start({6, 5}, 0.0).requires_grad_(true);
    auto b = start({5}, 1.0).requires_grad_(true);
    Opt opt({w, b}, o);
    for (int s = 0; s < steps; ++s) {
        w.mutable_grad() = gradient({6, 5}, s, 0.0);
        b.mutable_grad() = gradient({5}, s, 2.0);
        opt.step();
    }
    std::printf("%s", name);
    for (const auto& t : {w, b}) {
        auto f = t.detach().reshape(-1).to(pt::kDouble);
        for (int64_t i = 0; i < f.numel(); ++i) std::printf(" %.9g", f[i].template item<double>());
    }
    std::printf("\n");
}

int main() {
    using namespace pt::optim;
    run<SGD>("SGD", SGDOptions(0.05).momentum_(0.9).nesterov_(true).weight_decay_(0.01));
    run<SGD>("SGD_plain", SGDOptions(0.05));
    run<Adam>("Adam", AdamOptions(1e-2));
    run<Adam>("Adam_amsgrad", AdamOptions(1e-2).amsgrad_(true).weight_decay_(0.1));
    run<AdamW>("AdamW", AdamWOptions(1e-2));
    run<RMSprop>("RMSprop", RMSpropOptions().learning_rate(1e-2));
    run<RMSprop>("RMSprop_centered", RMSpropOptions().learning_rate(1e-2).centered_(true).momentum_(0.5));
    run<Lion>("Lion", LionOptions().learning_rate(3e-3).weight_decay_(0.1));
    run<SophiaG>("SophiaG", SophiaGOptions().learning_rate(1e-2));
    run<LAMB>("LAMB", LAMBOptions().learning_rate(1e-2));
    run<Adafactor>("Adafactor", AdafactorOptions());
    run<Adafactor>("Adafactor_fixed", AdafactorOptions().learning_rate(1e-2).relative_step_(false).scale_parameter_(false).beta1_(0.9));
    run<NAdam>("NAdam", NAdamOptions().learning_rate(1e-2));
    run<RAdam>("RAdam", RAdamOptions().learning_rate(2e-2), 9);
    run<Adagrad>("Adagrad", AdagradOptions().learning_rate(0.1));
    run<Adadelta>("Adadelta", AdadeltaOptions());
    run<Adamax>("Adamax", AdamaxOptions().learning_rate(2e-2));
    run<AdamKiller>("AdamKiller", AdamKillerOptions().learning_rate(1e-2));
    run<ASGD>("ASGD", ASGDOptions().learning_rate(0.05));
    return 0;
}
