// A first program against the C++ API: the MNIST-shaped MLP of the reference's examples/mnist/train_mnist_mlp.cpp on a synthetic
// set, with this package's Adam, a warm-up + cosine schedule, gradient clipping and a PTOR checkpoint at the end.
//
//   make -C examples/cpp mlp && examples/cpp/mlp [epochs]
#include <cstdio>
#include <cstdlib>

#include <promethorch/torch.h>

namespace pt = promethorch;

struct NetImpl : pt::nn::Module {
    NetImpl() {
        fc1 = register_module("fc1", pt::nn::Linear(784, 512));
        fc2 = register_module("fc2", pt::nn::Linear(512, 256));
        fc3 = register_module("fc3", pt::nn::Linear(256, 10));
    }
    pt::Tensor forward(const pt::Tensor& x) { return fc3(pt::relu(fc2(pt::relu(fc1(x))))); }
    pt::nn::Linear fc1{nullptr}, fc2{nullptr}, fc3{nullptr};
};
TORCH_MODULE(Net);

int main(int argc, char** argv) {
    const int epochs = argc > 1 ? std::atoi(argv[1]) : 2;
    pt::manual_seed(0);
    // ten noisy class prototypes stand in for the digits (no dataset ships with the package)
    auto protos = pt::rand({10, 784});
    auto make = [&](int64_t n) {
        auto y = pt::randint(0, 10, {n});
        return std::make_pair((protos.index_select(0, y) + 0.8 * pt::randn({n, 784})).clamp(0, 1), y);
    };
    auto train = make(8192), test = make(2048);
    auto dataset = std::make_shared<pt::data::TensorDataset>(train.first, train.second);
    pt::data::DataLoader loader(dataset, pt::data::DataLoaderOptions(64).shuffle(true).seed(1));

    Net net;
    pt::optim::Adam opt(net->parameters(), pt::optim::AdamOptions(1e-3));
    const int64_t total = epochs * (int64_t)((dataset->size() + 63) / 64);
    pt::optim::WarmupCosineAnnealingLR sched(opt, total / 10, total);
    for (int e = 0; e < epochs; ++e) {
        double last = 0;
        for (auto& batch : loader) {
            opt.zero_grad();
            auto loss = pt::nn::functional::cross_entropy(net(batch.data), batch.target);
            loss.backward();
            pt::nn::utils::clip_grad_norm_(net->parameters(), 1.0);
            opt.step();
            sched.step();
            last = loss.item<double>();
        }
        pt::NoGradGuard ng;
        const double acc = (net(test.first).argmax(-1) == test.second).to(pt::kFloat).mean().item<double>();
        std::printf("epoch %d: loss %.4f  test accuracy %.2f %%  lr %.2e\n", e + 1, last, 100 * acc, opt.get_lr(0));
    }
    pt::save(*net, "mlp.ptor");
    std::printf("saved mlp.ptor (%lld parameters)\n", (long long)pt::nn::num_parameters(*net));
    return 0;
}
