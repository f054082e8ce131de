// Exercises the C++ API on the CPU: the 784-512-256-10 MLP of the training benchmark for a few steps with Adam and a
// warm-up/cosine schedule, every optimizer on a small problem, schedulers against their closed forms, PTOR and .pt
// round trips, optimizer state export, and DistributedDataParallel over two forked ranks with no_sync accumulation.
#include <promethorch/torch.h>

#include <cstdio>
#include <iostream>

namespace pt = promethorch;

struct NetImpl : pt::nn::Module {
    NetImpl() {
        l1 = register_module("l1", pt::nn::Linear(784, 512));
        l2 = register_module("l2", pt::nn::Linear(512, 256));
        l3 = register_module("l3", pt::nn::Linear(256, 10));
    }
    pt::Tensor forward(const pt::Tensor& x) { return l3(pt::relu(l2(pt::relu(l1(x))))); }
    pt::nn::Linear l1{nullptr}, l2{nullptr}, l3{nullptr};
};
TORCH_MODULE(Net);

#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); return 1; } \
    } while (0)

static int train_mlp() {
    pt::manual_seed(0);
    Net net;
    pt::optim::Adam opt(net->parameters(), pt::optim::AdamOptions(1e-3));
    pt::optim::WarmupCosineAnnealingLR sched(opt, 2, 20);
    auto x = pt::rand({256, 784});
    auto w = pt::randn({784, 10});
    auto y = x.matmul(w).argmax(1);                      // a learnable labelling
    double first = 0, last = 0;
    for (int step = 0; step < 12; ++step) {
        opt.zero_grad();
        auto loss = pt::nn::functional::cross_entropy(net->forward(x), y);
        loss.backward();
        pt::clip_grad_norm_(net->parameters(), 10.0);
        opt.step();
        sched.step();
        if (step == 0) first = loss.item<double>();
        last = loss.item<double>();
    }
    CHECK(last < 0.7 * first);
    // optimizer state: "state.<i>.<key>", resumable
    auto sd = opt.state_dict();
    CHECK(sd.count("state.0.exp_avg") && sd.count("state.0.step") && sd.at("state.0.step").item<float>() == 12.f);
    // PTOR round trip of the module
    const std::string path = "/tmp/promethorch_cpp_test.ptor";
    pt::save(*net, path);
    Net net2;
    pt::load(*net2, path);
    CHECK(pt::allclose(net2->forward(x), net->forward(x)));
    // .pt round trip
    pt::save_pytorch(pt::state_dict(*net), path + ".pt");
    auto back = pt::load_pytorch(path + ".pt");
    CHECK(back.size() == 6 && pt::equal(back[0].second, net->l1->weight));
    std::remove(path.c_str());
    std::remove((path + ".pt").c_str());
    return 0;
}

template <typename Opt, typename Options>
static int descends(const char* name, Options o, double factor = 0.9, int steps = 60) {
    pt::manual_seed(1);
    auto w = pt::randn({16, 8}).requires_grad_(true);
    auto b = pt::zeros({8}).requires_grad_(true);
    auto x = pt::randn({64, 16}), t = pt::randn({64, 8});
    Opt opt({w, b}, o);
    double first = 0, last = 0;
    for (int i = 0; i < steps; ++i) {
        opt.zero_grad();
        auto loss = (x.matmul(w) + b - t).pow(2).mean();
        loss.backward();
        opt.step();
        if (i == 0) first = loss.template item<double>();
        last = loss.template item<double>();
    }
    if (!(last < factor * first)) { std::printf("FAIL %s did not descend: %f -> %f\n", name, first, last); return 1; }
    return 0;
}

static int optimizers() {
    using namespace pt::optim;
    int rc = 0;
    rc |= descends<SGD>("SGD", SGDOptions(0.05).momentum_(0.9).nesterov_(true));
    rc |= descends<Adam>("Adam", AdamOptions(1e-2).amsgrad_(true));
    rc |= descends<AdamW>("AdamW", AdamWOptions(1e-2));
    rc |= descends<RMSprop>("RMSprop", RMSpropOptions().learning_rate(1e-2).centered_(true).momentum_(0.5));
    rc |= descends<Lion>("Lion", LionOptions().learning_rate(3e-3));
    rc |= descends<SophiaG>("SophiaG", SophiaGOptions().learning_rate(0.3));
    rc |= descends<LAMB>("LAMB", LAMBOptions().learning_rate(1e-2));
    rc |= descends<Adafactor>("Adafactor", AdafactorOptions());
    rc |= descends<NAdam>("NAdam", NAdamOptions().learning_rate(1e-2));
    rc |= descends<RAdam>("RAdam", RAdamOptions().learning_rate(2e-2));
    rc |= descends<Adagrad>("Adagrad", AdagradOptions().learning_rate(0.1));
    rc |= descends<Adadelta>("Adadelta", AdadeltaOptions(), 0.98, 120);
    rc |= descends<Adamax>("Adamax", AdamaxOptions().learning_rate(2e-2));
    rc |= descends<AdamKiller>("AdamKiller", AdamKillerOptions().learning_rate(1e-2));
    rc |= descends<ASGD>("ASGD", ASGDOptions().learning_rate(0.05));
    {   // LBFGS with a closure
        pt::manual_seed(1);
        auto w = pt::randn({16, 8}).requires_grad_(true);
        auto x = pt::randn({64, 16}), t = pt::randn({64, 8});
        LBFGS opt({w}, LBFGSOptions().learning_rate(0.5));
        auto closure = [&] { opt.zero_grad(); auto l = (x.matmul(w) - t).pow(2).mean(); l.backward(); return l; };
        const double first = closure().item<double>();
        opt.step(closure);
        rc |= !(closure().item<double>() < 0.7 * first);
    }
    {   // parameter groups: per-group override, inherit otherwise; resume of the flat state continues the run
        pt::manual_seed(2);
        auto a = pt::randn({4}).requires_grad_(true), b = pt::randn({4}).requires_grad_(true);
        Adam opt(std::vector<ParamGroup>{ParamGroup({a}).learning_rate(0.1), ParamGroup({b})}, AdamOptions(0.01));
        rc |= !(opt.get_lr(0) == 0.1 && opt.get_lr(1) == 0.01);
        for (int i = 0; i < 3; ++i) { opt.zero_grad(); (a.pow(2).sum() + b.pow(2).sum()).backward(); opt.step(); }
        auto a2 = a.detach().clone().requires_grad_(true), b2 = b.detach().clone().requires_grad_(true);
        Adam opt2(std::vector<ParamGroup>{ParamGroup({a2}).learning_rate(0.1), ParamGroup({b2})}, AdamOptions(0.01));
        opt2.load_state_dict(opt.state_dict());
        opt.zero_grad(); (a.pow(2).sum() + b.pow(2).sum()).backward(); opt.step();
        opt2.zero_grad(); (a2.pow(2).sum() + b2.pow(2).sum()).backward(); opt2.step();
        rc |= !(pt::allclose(a, a2) && pt::allclose(b, b2));
    }
    {   // EMA
        auto p = pt::ones({2});
        EMA ema({p}, 0.9);
        p.fill_(2.0);
        ema.update();
        rc |= !pt::allclose(ema.shadow()[0], pt::full({2}, 1.1));
    }
    if (rc) std::printf("FAIL optimizers\n");
    return rc;
}

static int schedulers() {
    using namespace pt::optim;
    auto p = pt::zeros({1}).requires_grad_(true);
    int line = 0;
    auto near = [&](double a, double b) { ++line; const bool ok = std::fabs(a - b) < 1e-9; if (!ok) std::printf("FAIL scheduler check %d: %.9f vs %.9f\n", line, a, b); return ok; };
    int rc = 0;
    { SGD o({p}, SGDOptions(1.0)); StepLR s(o, 2, 0.5); for (int i = 0; i < 5; ++i) s.step(); rc |= !near(o.get_lr(), 0.25); }
    { SGD o({p}, SGDOptions(1.0)); MultiStepLR s(o, {1, 3}, 0.1); for (int i = 0; i < 4; ++i) s.step(); rc |= !near(o.get_lr(), 0.01); }
    { SGD o({p}, SGDOptions(1.0)); ExponentialLR s(o, 0.5); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 0.25); }
    { SGD o({p}, SGDOptions(1.0)); CosineAnnealingLR s(o, 10, 0.0); for (int i = 0; i < 6; ++i) s.step(); rc |= !near(o.get_lr(), 0.5); }
    { SGD o({p}, SGDOptions(1.0)); LinearLR s(o, 0.5, 1.0, 4); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 0.75); }
    { SGD o({p}, SGDOptions(1.0)); ConstantLR s(o, 0.25, 2); s.step(); rc |= !near(o.get_lr(), 0.25); s.step(); s.step(); rc |= !near(o.get_lr(), 1.0); }
    { SGD o({p}, SGDOptions(1.0)); ReduceLROnPlateau s(o, ReduceLROnPlateau::Mode::Min, 0.5, 1); s.step(1.0); s.step(1.0); s.step(1.0); rc |= !near(o.get_lr(), 0.5); }
    { SGD o({p}, SGDOptions(1.0)); WarmupCosineAnnealingLR s(o, 4, 12); s.step(); rc |= !near(o.get_lr(), 0.25); for (int i = 0; i < 8; ++i) s.step(); rc |= !near(o.get_lr(), 0.5); }
    { SGD o({p}, SGDOptions(1.0)); OneCycleLR s(o, 1.0, 10); rc |= !near(o.get_lr(), 0.04); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 1.0); }
    { SGD o({p}, SGDOptions(1.0)); CosineAnnealingWarmRestarts s(o, 4); for (int i = 0; i < 4; ++i) s.step(); rc |= !near(o.get_lr(), 1.0); s.step(); rc |= !near(o.get_lr(), (1 + std::cos(M_PI / 4)) / 2); }
    { SGD o({p}, SGDOptions(1.0)); CyclicLR s(o, 0.1, 1.1, 4); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 0.6); }
    { SGD o({p}, SGDOptions(1.0)); PolynomialLR s(o, 4, 2.0); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 0.25); }
    { SGD o({p}, SGDOptions(1.0)); LambdaLR s(o, [](int64_t e) { return 1.0 / (1 + e); }); for (int i = 0; i < 4; ++i) s.step(); rc |= !near(o.get_lr(), 0.25); }
    { SGD o({p}, SGDOptions(1.0)); MultiplicativeLR s(o, [](int64_t) { return 0.5; }); for (int i = 0; i < 3; ++i) s.step(); rc |= !near(o.get_lr(), 0.25); }
    {
        SGD o({p}, SGDOptions(1.0));
        auto a = std::make_shared<ConstantLR>(o, 0.5, 100);
        auto b = std::make_shared<ExponentialLR>(o, 0.5);
        SequentialLR s(o, {a, b}, {2});
        s.step(); s.step(); rc |= !near(o.get_lr(), 0.5);
        s.step(); rc |= !near(o.get_lr(), 1.0);          // the second scheduler starts at its epoch 0
    }
    {
        SGD o({p}, SGDOptions(1.0));
        auto a = std::make_shared<ExponentialLR>(o, 0.5);
        auto b = std::make_shared<ExponentialLR>(o, 0.5);
        ChainedScheduler s(o, {a, b});
        s.step(); s.step(); rc |= !near(o.get_lr(), 0.25);
    }
    if (rc) std::printf("FAIL schedulers\n");
    return rc;
}

static int ddp_worker(const pt::distributed::DistArgs& a) {
    namespace D = pt::distributed;
    D::DDPConfig cfg;
    cfg.rank = a.rank; cfg.world_size = a.world_size; cfg.master_addr = a.master_addr; cfg.master_port = a.master_port; cfg.timeout_sec = 30;
    D::init_process_group(cfg);
    pt::manual_seed(100 + a.rank);                      // different initial weights: the constructor must broadcast rank 0's
    Net net;
    D::DistributedDataParallel<Net> ddp(net);
    auto t = pt::full({3}, (float)(a.rank + 1));
    D::all_reduce(t);
    if (!pt::allclose(t, pt::full({3}, 3.0f))) return 2;
    pt::manual_seed(7 + a.rank);                        // different data per rank
    auto x = pt::rand({8, 784});
    auto y = pt::randint(0, 10, {8});
    {   // two micro-batches: the first accumulates locally under the guard, the second synchronises the sum
        D::DDPNoSyncGuard<decltype(ddp)> guard(ddp);
        pt::nn::functional::cross_entropy(ddp(x), y).backward();
        ddp.allreduce_grads();                          // no-op inside the guard
    }
    pt::nn::functional::cross_entropy(ddp(x), y).backward();
    ddp.allreduce_grads();
    // every rank must now hold the same averaged gradient
    auto g = net->l3->weight.grad().clone();
    auto parts = D::default_group()->all_gather(g);
    if (!pt::allclose(parts[0], parts[1], 1e-6, 1e-7)) return 3;
    // tensor-parallel linear layers reproduce the unsharded layer with the same seed
    pt::nn::parallel::TPConfig tp;
    tp.rank = a.rank; tp.world_size = a.world_size;
    pt::nn::parallel::ColumnParallelLinear col(16, 8, tp, true, false, 5);
    pt::nn::parallel::RowParallelLinear row(16, 8, tp, false, false, 5);
    pt::manual_seed(9);
    auto z = pt::randn({4, 16});
    auto full = pt::nn::functional::linear(z, pt::nn::parallel::tp_full_weight(8, 16, 5));
    if (!pt::allclose(col(z), full, 1e-5, 1e-6) || !pt::allclose(row(z), full, 1e-5, 1e-6)) return 4;
    D::barrier();
    D::destroy_process_group();
    return 0;
}

int main(int argc, char** argv) {
    // the ranks are forked first: a process that has already started libtorch's worker threads must not fork
    const int port = argc > 1 ? std::atoi(argv[1]) : 29731;
    const int drc = pt::distributed::launch(2, ddp_worker, "127.0.0.1", port);
    if (drc) std::printf("FAIL ddp worker exit code %d\n", drc);
    int rc = drc;
    rc |= train_mlp();
    rc |= optimizers();
    rc |= schedulers();
    {
        pt::data::DistributedSampler s0(10, 2, 0, true, 3), s1(10, 2, 1, true, 3);
        auto a = s0.indices(), b = s1.indices();
        std::vector<int> seen(10, 0);
        for (auto i : a) seen[i]++;
        for (auto i : b) seen[i]++;
        for (int v : seen) rc |= v != 1;
    }
    std::printf(rc ? "CPP_API_FAIL\n" : "CPP_API_OK\n");
    return rc;
}
