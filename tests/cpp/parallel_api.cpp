// Exercises the rest of the C++ API on the CPU: GradScaler and autocast guards, datasets / samplers / DataLoader with
// worker threads, the GPipe pipeline, and (over forked ranks) FullyShardedDataParallel with a ZeRO optimizer, the offload
// optimizer, the split all-gather, and a two-stage 1F1B pipeline whose gradients equal the single-process model's.
#include <promethorch/torch.h>

#include <cstdio>
#include <iostream>

namespace pt = promethorch;
namespace dist = promethorch::distributed;

#undef CHECK
#define CHECK(cond)                                                              \
    do {                                                                         \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); std::fflush(stdout); return 1; } \
    } while (0)
#define CHECK_VOID(cond)                                                         \
    do {                                                                         \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); std::fflush(stdout); std::exit(1); } \
    } while (0)

struct MLPImpl : pt::nn::Module {
    MLPImpl(int in, int hid, int out) {
        l1 = register_module("l1", pt::nn::Linear(in, hid));
        l2 = register_module("l2", pt::nn::Linear(hid, out));
    }
    pt::Tensor forward(const pt::Tensor& x) { return l2(pt::tanh(l1(x))); }
    pt::nn::Linear l1{nullptr}, l2{nullptr};
};
TORCH_MODULE(MLP);

static bool close(const pt::Tensor& a, const pt::Tensor& b, double tol = 1e-5) { return (a - b).abs().max().item<double>() <= tol; }

// ---- two ranks: sharded data parallelism
static int fsdp_rank(const dist::DistArgs& a) {
    dist::DDPConfig cfg;
    cfg.rank = a.rank; cfg.world_size = a.world_size; cfg.master_addr = a.master_addr; cfg.master_port = a.master_port; cfg.timeout_sec = 60;
    dist::init_process_group(cfg);
    pt::manual_seed(7);
    MLP net(12, 9, 5), ref(12, 9, 5);                       // 9 and 5 do not divide by 2: shards are padded
    {
        pt::NoGradGuard ng;
        auto rp = ref->parameters();
        auto np = net->parameters();
        for (size_t i = 0; i < rp.size(); ++i) rp[i].copy_(np[i]);
    }
    dist::FullyShardedDataParallel<MLP> fsdp(net);
    CHECK(fsdp.sharded_numel() * 2 >= fsdp.full_numel() && fsdp.sharded_numel() < fsdp.full_numel());
    dist::ZeROOptimizer<MLP, pt::optim::Adam> zero(fsdp, pt::optim::AdamOptions(1e-2));
    pt::optim::Adam ref_opt(ref->parameters(), pt::optim::AdamOptions(1e-2));
    pt::manual_seed(100);
    auto X = pt::randn({2, 6, 12});                          // one batch per rank, the same on both processes
    auto Y = pt::randn({2, 6, 5});
    for (int step = 0; step < 3; ++step) {
        zero.zero_grad();
        pt::mse_loss(fsdp.forward(X[a.rank]), Y[a.rank]).backward();
        zero.step();
        fsdp.reshard_params();
        CHECK(!fsdp.params_gathered() && net->parameters()[0].numel() == 0);      // the full parameters are gone
        ref_opt.zero_grad();
        ((pt::mse_loss(ref->forward(X[0]), Y[0]) + pt::mse_loss(ref->forward(X[1]), Y[1])) / 2).backward();
        ref_opt.step();
        fsdp.all_gather_params();
        auto rp = ref->parameters();
        auto np = net->parameters();
        for (size_t i = 0; i < rp.size(); ++i) CHECK(close(rp[i], np[i], 2e-5));
    }
    // SyncBatchNorm over the two ranks == BatchNorm over the concatenated batch, forward and backward
    {
        pt::manual_seed(11);
        auto full = pt::randn({8, 3, 5});
        auto go = pt::randn({8, 3, 5});
        pt::nn::BatchNorm1d bn(3);
        {
            pt::NoGradGuard ng;
            bn->weight.copy_(pt::tensor({1.5f, 0.5f, 2.0f}));
            bn->bias.copy_(pt::tensor({0.1f, -0.2f, 0.3f}));
        }
        pt::nn::Sequential holder(pt::nn::BatchNorm1d(3));
        {
            pt::NoGradGuard ng;
            auto* inner = holder->ptr(0)->as<pt::nn::BatchNorm1dImpl>();
            inner->weight.copy_(bn->weight);
            inner->bias.copy_(bn->bias);
        }
        holder = dist::convert_sync_batchnorm(holder);
        auto xf = full.clone().set_requires_grad(true);
        auto yf = bn->forward(xf);
        (yf * go).sum().backward();
        auto xl = full.narrow(0, a.rank * 4, 4).clone().set_requires_grad(true);
        auto yl = holder->forward(xl);
        (yl * go.narrow(0, a.rank * 4, 4)).sum().backward();
        CHECK(close(yl, yf.narrow(0, a.rank * 4, 4), 1e-5));
        CHECK(close(xl.grad(), xf.grad().narrow(0, a.rank * 4, 4), 1e-5));
        auto* sbn = holder->ptr(0)->as<dist::SyncBatchNormImpl>();
        CHECK(sbn != nullptr && close(sbn->running_mean, bn->running_mean, 1e-6) && close(sbn->running_var, bn->running_var, 1e-5));
        // the weight gradient is a per-rank partial sum, as any data-parallel gradient: the two ranks' sums add up
        auto gw = sbn->weight.grad().clone();
        dist::all_reduce(gw);
        CHECK(close(gw, bn->weight.grad(), 1e-4));
    }
    // split all-gather
    std::vector<float> buf(2 * 3, -1.f);
    for (int k = 0; k < 3; ++k) buf[a.rank * 3 + k] = (float)(10 * a.rank + k);
    auto h = dist::all_gather_post(buf.data(), 3);
    dist::all_gather_wait(h);
    for (int r = 0; r < 2; ++r)
        for (int k = 0; k < 3; ++k) CHECK(buf[r * 3 + k] == (float)(10 * r + k));
    dist::barrier();
    dist::destroy_process_group();
    return 0;
}

// ---- two ranks: a two-stage 1F1B pipeline
struct StageAImpl : pt::nn::Module {
    StageAImpl() { l = register_module("l", pt::nn::Linear(8, 16)); }
    pt::Tensor forward(const pt::Tensor& x) { return pt::tanh(l(x)); }
    pt::nn::Linear l{nullptr};
};
TORCH_MODULE(StageA);
struct StageBImpl : pt::nn::Module {
    StageBImpl() { l = register_module("l", pt::nn::Linear(16, 4)); }
    pt::Tensor forward(const pt::Tensor& x) { return l(x); }
    pt::nn::Linear l{nullptr};
};
TORCH_MODULE(StageB);

static int pipeline_rank(const dist::DistArgs& a) {
    pt::manual_seed(3);
    StageA sa;                                               // both processes build both stages from the same seed
    StageB sb;
    pt::manual_seed(4);
    const int M = 4;
    auto X = pt::randn({M * 3, 8}), Y = pt::randn({M * 3, 4});
    auto xs = X.chunk(M, 0), ys = Y.chunk(M, 0);
    // single-process gradients of the whole model: mean over the micro-batches of the per-micro-batch loss
    pt::Tensor total = pt::zeros({});
    for (int i = 0; i < M; ++i) total = total + pt::mse_loss(sb->forward(sa->forward(xs[i])), ys[i]) / (double)M;
    total.backward();
    std::vector<pt::Tensor> want;
    for (auto& p : (a.rank == 0 ? sa->parameters() : sb->parameters())) { want.push_back(p.grad().clone()); }
    sa->zero_grad();
    sb->zero_grad();
    dist::PipelineScheduleConfig cfg;
    cfg.num_stages = 2; cfg.num_micros = M; cfg.base_port = a.master_port + 7; cfg.timeout_ms = 30000;
    auto loss_fn = [](const pt::Tensor& o, const pt::Tensor& t) { return pt::mse_loss(o, t); };
    double loss = 0;
    int alive = 0;
    std::vector<pt::Tensor> got;
    if (a.rank == 0) {
        dist::Pipeline1F1BStage<StageA> st(sa, 0, cfg);
        loss = st.train_step({xs.begin(), xs.end()}, {}, nullptr);
        alive = st.max_alive_micro_batches();
        for (auto& p : sa->parameters()) got.push_back(p.grad());
        CHECK(alive == 2 && loss == 0.0);
    } else {
        dist::Pipeline1F1BStage<StageB> st(sb, 1, cfg);
        loss = st.train_step({}, {ys.begin(), ys.end()}, loss_fn);
        alive = st.max_alive_micro_batches();
        for (auto& p : sb->parameters()) got.push_back(p.grad());
        CHECK(alive == 1 && std::abs(loss - total.item<double>()) < 1e-5);
    }
    for (size_t i = 0; i < want.size(); ++i) CHECK(close(want[i], got[i], 1e-5));
    return 0;
}

// ---- Trainer: a regression module fitted with accumulation and clipping, checkpointed per epoch, resumed
struct RegImpl : pt::trainer::LightningModule {
    RegImpl() { l = register_module("l", pt::nn::Linear(4, 1)); }
    pt::Tensor training_step(const pt::data::Batch& b, int) override { return pt::mse_loss(l(b.data), b.target); }
    pt::Tensor validation_step(const pt::data::Batch& b, int) override { return pt::mse_loss(l(b.data), b.target); }
    std::shared_ptr<pt::optim::Optimizer> configure_optimizer() override {
        return std::make_shared<pt::optim::Adam>(parameters(), pt::optim::AdamOptions(0.2));
    }
    void on_train_epoch_end(int, double) override { ++epochs_seen; }
    pt::nn::Linear l{nullptr};
    int epochs_seen = 0;
};

static int trainer_test(const std::string& dir) {
    pt::manual_seed(5);
    auto X = pt::randn({64, 4});
    auto Y = X.matmul(pt::tensor({{1.0f}, {-2.0f}, {0.5f}, {3.0f}})) + 0.7;
    auto ds = std::make_shared<pt::data::TensorDataset>(X, Y);
    pt::data::DataLoader train(ds, pt::data::DataLoaderOptions(8)), val(ds, pt::data::DataLoaderOptions(16));
    pt::trainer::TrainerConfig cfg;
    cfg.max_epochs = 6; cfg.accumulate_grad_batches = 2; cfg.gradient_clip_val = 5.0; cfg.checkpoint_dir = dir;
    cfg.enable_progress_bar = false;
    RegImpl model;
    pt::trainer::Trainer tr(cfg);
    tr.fit(model, train, &val);
    CHECK(model.epochs_seen == 6 && tr.train_history().size() == 6 && tr.global_step() == 6 * 4);
    CHECK(tr.train_history().back() < 0.3 * tr.train_history().front());
    CHECK(std::abs(tr.last_val_metric() - tr.test(model, val)) < 1e-9);
    // resume from the epoch-3 checkpoint: three more epochs land on the same weights as the uninterrupted run
    RegImpl again;
    cfg.max_epochs = 6;
    pt::trainer::Trainer tr2(cfg);
    CHECK(tr2.load_checkpoint(again, dir + "/epoch_3.ptor") && tr2.next_epoch() == 3 && tr2.global_step() == 12);
    CHECK(!tr2.load_checkpoint(again, dir + "/nothing.ptor"));
    CHECK(tr2.load_checkpoint(again, dir + "/epoch_3.ptor"));
    cfg.checkpoint_dir = dir + "_resumed";
    pt::trainer::Trainer tr3(cfg);
    CHECK(tr3.load_checkpoint(again, dir + "/epoch_3.ptor"));
    tr3.fit(again, train, &val);
    CHECK(again.epochs_seen == 3 && tr3.global_step() == 24);
    CHECK(close(again.l->weight, model.l->weight, 1e-6) && close(again.l->bias, model.l->bias, 1e-6));
    return 0;
}

static int quant_and_checkpoint() {
    namespace q = pt::quantization;
    pt::manual_seed(9);
    // fake quantisation: values land on the 8-bit grid, gradients pass inside the range and stop outside
    {
        q::FakeQuantize fq(8);
        auto x = pt::linspace(-1, 1, 41).set_requires_grad(true);
        auto y = fq(x);
        const double scale = 1.0 / 127;
        CHECK(((y / scale) - pt::round(y / scale)).abs().max().item<double>() < 1e-4);
        CHECK((y - x).abs().max().item<double>() <= scale / 2 + 1e-6);
        y.sum().backward();
        CHECK(close(x.grad(), pt::ones({41})));
        fq->freeze();
        auto big = pt::tensor({5.0f, 0.5f}).set_requires_grad(true);
        fq(big).sum().backward();
        CHECK(big.grad()[0].item<float>() == 0.0f && big.grad()[1].item<float>() == 1.0f);      // 5.0 is clipped
    }
    // QAT linear trains; int8 inference layer and 4-bit layers stay close to the float layer
    {
        pt::nn::Linear lin(16, 8);
        q::QATLinear qat(lin, 8);
        auto x = pt::randn({32, 16});
        CHECK((qat(x) - lin(x)).abs().max().item<double>() < 0.1);
        qat(x).pow(2).mean().backward();
        CHECK(lin->weight.grad().defined());
        q::QuantizedLinear ql(lin);
        CHECK((ql(x) - lin(x)).abs().max().item<double>() < 0.05 && ql->weight_q.scalar_type() == pt::kChar);
        pt::nn::Linear wide(64, 8);
        q::Linear4bit nf(wide, 64, "nf4"), i4(wide, 64, "int4");
        auto xw = pt::randn({4, 64});
        const double ref = wide(xw).abs().mean().item<double>();
        CHECK((nf(xw) - wide(xw)).abs().mean().item<double>() < 0.2 * ref && (i4(xw) - wide(xw)).abs().mean().item<double>() < 0.25 * ref);
        CHECK(nf->packed.numel() == 64 * 8 / 2 && nf->absmax.numel() == 8);
        auto rt = q::dequantize_4bit(nf->packed, nf->absmax, {8, 64});
        CHECK((rt - wide->weight).abs().max().item<double>() < 0.15 * wide->weight.abs().max().item<double>());
        auto a = q::quantize_per_tensor(pt::randn({8, 16})), b = q::quantize_per_tensor(pt::randn({16, 4}));
        auto exact = (a.first.to(pt::kFloat) * a.second).matmul(b.first.to(pt::kFloat) * b.second);
        CHECK(close(q::int8_matmul(a.first, a.second, b.first, b.second), exact, 1e-5));
    }
    // checkpoint: the same output and gradients as the plain graph, for inputs and for parameters
    {
        pt::nn::Linear l1(6, 6), l2(6, 3);
        auto stage1 = [l1](const pt::Tensor& t) mutable { return pt::tanh(l1(t)); };
        auto stage2 = [l2](const pt::Tensor& t) mutable { return l2(t); };
        auto x1 = pt::randn({5, 6}).set_requires_grad(true);
        auto x2 = x1.detach().clone().set_requires_grad(true);
        auto plain = stage2(stage1(x1));
        plain.pow(2).sum().backward();
        auto gw = l1->weight.grad().clone(), gx = x1.grad().clone();
        l1->zero_grad();
        l2->zero_grad();
        auto ck = pt::utils::checkpoint_sequential({stage1, stage1, stage2}, 2, x2);      // (stage1, stage1) checkpointed, stage2 plain
        auto want = stage2(stage1(stage1(x1.detach())));
        CHECK(close(ck, want, 1e-6));
        auto one = pt::utils::checkpoint(std::function<pt::Tensor(const pt::Tensor&)>(stage1), x2);
        l1->zero_grad();
        l2->zero_grad();
        stage2(one).pow(2).sum().backward();
        CHECK(close(l1->weight.grad(), gw, 1e-5) && close(x2.grad(), gx, 1e-5));
    }
    return 0;
}

static int nn_extras() {
    namespace F = pt::nn::functional;
    pt::manual_seed(21);
    auto p = pt::rand({4, 10}) * 0.9 + 0.05, y = (pt::rand({4, 10}) > 0.5).to(pt::kFloat);
    {   // focal loss with gamma 0 and alpha 0.5 is half the binary cross entropy
        pt::nn::FocalLoss fl("mean", 0.5, 0.0);
        CHECK(close(fl(p, y), 0.5 * pt::binary_cross_entropy(p, y), 1e-5));
        pt::nn::DiceLoss dl;
        CHECK(std::fabs(dl(y, y).item<double>()) < 1e-6 && dl(p, y).item<double>() > 0);
        pt::nn::GaussianNLLLoss gl;
        auto x = pt::randn({6}), t = pt::randn({6}), v = pt::rand({6}) + 0.1;
        CHECK(close(gl(x, t, v), (0.5 * (v.log() + (x - t).pow(2) / v)).mean(), 1e-6));
    }
    {
        pt::nn::GlobalAvgPool2d gap;
        auto x = pt::randn({2, 3, 4, 5});
        CHECK(close(gap(x), x.mean({2, 3}), 1e-6));
        pt::nn::PositionalEncoding pe(8, 0.0, 32);
        auto z = pt::zeros({5, 2, 8});
        auto out = pe(z);
        CHECK(std::fabs(out[3][1][0].item<double>() - std::sin(3.0)) < 1e-5 && std::fabs(out[3][0][1].item<double>() - std::cos(3.0)) < 1e-5);
        pt::nn::Dropout1d d1(0.5);
        auto o = d1(pt::ones({8, 16, 6}));
        auto per_channel = o.amax(2) - o.amin(2);
        CHECK(per_channel.abs().max().item<double>() == 0.0 && (o == 0).any().item<bool>());      // whole channels at once
        d1->eval();
        CHECK(close(d1(pt::ones({16, 6})), pt::ones({16, 6})));
        pt::nn::LazyLinear lazy(7);
        CHECK(lazy->has_uninitialized_params());
        CHECK(lazy(pt::randn({3, 11})).sizes() == at::IntArrayRef({3, 7}) && lazy->weight.size(1) == 11 && lazy->parameters().size() == 2);
        pt::nn::Conv2d conv(pt::nn::Conv2dOptions(3, 6, 3).padding(1).stride(2));
        pt::nn::QuantizedConv2d qc(conv);
        auto img = pt::randn({2, 3, 9, 9});
        CHECK(qc(img).sizes() == conv(img).sizes() && (qc(img) - conv(img)).abs().max().item<double>() < 0.05);
        CHECK(pt::nn::num_parameters(*conv) == 6 * 3 * 9 + 6);
    }
    {
        auto x = pt::randn({5, 6}), w1 = pt::randn({8, 6}), b1 = pt::randn({8}), w2 = pt::randn({3, 8});
        CHECK(close(F::fused_mlp(x, {w1, w2}, {b1}), pt::relu(x.matmul(w1.t()) + b1).matmul(w2.t()), 1e-5));
        CHECK(close(F::fused_linear_relu(x, w1, b1), pt::relu(x.matmul(w1.t()) + b1), 1e-5));
        auto g = pt::rand({6});
        CHECK(close(F::rms_norm(x, g), x / (x.pow(2).mean(-1, true) + 1e-6).sqrt() * g, 1e-5));
        // rotation keeps the norm of each (i, i + half) pair and is the identity at position 0
        auto q = pt::randn({2, 4, 8}), pos = pt::arange(4);
        auto r = F::rotary_embedding(q, pos);
        CHECK(close(r.select(1, 0), q.select(1, 0), 1e-6));
        CHECK(close(r.slice(-1, 0, 4).pow(2) + r.slice(-1, 4, 8).pow(2), q.slice(-1, 0, 4).pow(2) + q.slice(-1, 4, 8).pow(2), 1e-5));
        // scan against the loop, with a gradient through it
        auto a = (pt::rand({3, 13}) * 0.9).set_requires_grad(true), b = pt::randn({3, 13});
        auto h = F::parallel_scan(a, b);
        auto ref = pt::zeros({3, 13});
        auto prev = pt::zeros({3});
        for (int t = 0; t < 13; ++t) {
            prev = a.detach().select(1, t) * prev + b.select(1, t);
            ref.select(1, t).copy_(prev);
        }
        CHECK(close(h, ref, 1e-5));
        h.sum().backward();
        CHECK(a.grad().defined() && a.grad().abs().sum().item<double>() > 0);
    }
    return 0;
}

static int module_hooks() {
    pt::manual_seed(5);
    pt::nn::Hooked<pt::nn::Linear> lin(pt::nn::Linear(4, 3));
    int pre_calls = 0, fwd_calls = 0, bwd_calls = 0;
    pt::Tensor seen_gin, seen_gout;
    int pre = lin.register_forward_pre_hook([&](pt::nn::Module&, std::vector<pt::Tensor>& in) { ++pre_calls; in[0] = in[0] * 2; });
    int fwd = lin.register_forward_hook([&](pt::nn::Module&, const std::vector<pt::Tensor>&, const pt::Tensor& out) { ++fwd_calls; CHECK_VOID(out.size(1) == 3); });
    int ret = lin.register_forward_hook_with_return([&](pt::nn::Module&, const std::vector<pt::Tensor>&, const pt::Tensor& out) { return out + 1; });
    int bwd = lin.register_backward_hook([&](pt::nn::Module&, const std::vector<pt::Tensor>& gin, const pt::Tensor& gout) { ++bwd_calls; seen_gin = gin[0]; seen_gout = gout; });
    auto x = pt::randn({5, 4}).set_requires_grad(true);
    auto y = lin(x);
    CHECK(close(y, lin.module()(x.detach() * 2) + 1, 1e-6) && pre_calls == 1 && fwd_calls == 1);
    y.sum().backward();
    CHECK(bwd_calls == 1 && close(seen_gout, pt::ones({5, 3})));
    CHECK(close(seen_gin, pt::ones({5, 3}).matmul(lin->weight.detach()), 1e-6));        // the gradient at the (doubled) input of the layer
    CHECK(close(x.grad(), 2 * seen_gin, 1e-6));
    CHECK(lin.remove_hook(pre) && lin.remove_hook(ret) && !lin.remove_hook(ret) && lin.num_hooks() == 2);
    auto y2 = lin(x.detach());                                                           // no input wants a gradient: fires on the output's
    CHECK(close(y2, lin.module()(x.detach()), 1e-6));
    y2.sum().backward();
    CHECK(bwd_calls == 2 && !seen_gin.defined());
    lin.remove_hook(fwd);
    lin.remove_hook(bwd);
    CHECK(lin.num_hooks() == 0);
    // a backward pass that runs after the wrapper is gone still finds the hooks (they live in shared state)
    int late = 0;
    pt::Tensor out_late;
    auto x3 = pt::randn({2, 4}).set_requires_grad(true);
    {
        pt::nn::Hooked<pt::nn::Linear> scoped(pt::nn::Linear(4, 2));
        scoped.register_backward_hook([&](pt::nn::Module&, const std::vector<pt::Tensor>&, const pt::Tensor&) { ++late; });
        out_late = scoped(x3);
    }
    out_late.sum().backward();
    CHECK(late == 1 && x3.grad().defined());
    return 0;
}

static int single_process() {
    // GradScaler
    {
        auto w = pt::ones({3}).set_requires_grad(true);
        pt::optim::SGD opt({w}, pt::optim::SGDOptions(0.5));
        pt::amp::GradScaler sc(pt::amp::GradScalerOptions().init_scale(8.0).growth_interval(2));
        sc.scale((w * 2).sum()).backward();                  // gradient 2 * 8
        CHECK(close(w.grad(), pt::full({3}, 16.0)));
        CHECK(sc.step(opt));                                 // unscaled to 2, w = 1 - 0.5 * 2
        CHECK(close(w.detach(), pt::zeros({3})));
        sc.update();
        CHECK(sc.get_scale() == 8.0);
        opt.zero_grad();
        (w * std::numeric_limits<float>::infinity()).sum().backward();
        CHECK(!sc.step(opt) && sc.found_inf());              // skipped
        CHECK(close(w.detach(), pt::zeros({3})));
        sc.update();
        CHECK(sc.get_scale() == 4.0);                        // backed off
        for (int i = 0; i < 2; ++i) {
            opt.zero_grad();
            sc.scale(w.sum()).backward();
            CHECK(sc.step(opt));
            sc.update();
        }
        CHECK(sc.get_scale() == 8.0);                        // grew after two clean steps
        auto sd = sc.state_dict();
        pt::amp::GradScaler other;
        other.load_state_dict(sd);
        CHECK(other.get_scale() == 8.0);
    }
    // autocast
    {
        auto a = pt::randn({4, 4}), b = pt::randn({4, 4});
        {
            pt::amp::AutocastCPUGuard g(pt::kBFloat16);
            CHECK(pt::matmul(a, b).scalar_type() == pt::kBFloat16);
            CHECK(pt::amp::is_autocast_enabled(c10::kCPU) && pt::amp::get_autocast_dtype(c10::kCPU) == pt::kBFloat16);
            // the table says what the guard does: matmul-like ops in the low dtype, losses back in fp32
            CHECK(pt::amp::get_autocast_policy("matmul") == pt::amp::CastPolicy::LowerPrecision);
            CHECK(pt::amp::get_autocast_policy("mse_loss") == pt::amp::CastPolicy::FP32);
            CHECK(pt::mse_loss(pt::matmul(a, b), pt::matmul(a, b)).scalar_type() == pt::kFloat);
            CHECK(pt::amp::get_autocast_policy("relu") == pt::amp::CastPolicy::Unchanged && pt::relu(pt::matmul(a, b)).scalar_type() == pt::kBFloat16);
            CHECK(pt::amp::get_autocast_policy("cat") == pt::amp::CastPolicy::Promote);
        }
        CHECK(!pt::amp::is_autocast_enabled(c10::kCPU));
        CHECK(pt::matmul(a, b).scalar_type() == pt::kFloat);
    }
    // datasets, samplers, loader
    {
        auto X = pt::arange(20, pt::kFloat).reshape({10, 2});
        auto Y = pt::arange(10);
        auto ds = std::make_shared<pt::data::TensorDataset>(X, Y);
        pt::data::DataLoader seq(ds, pt::data::DataLoaderOptions(4));
        CHECK(seq.size() == 3);
        std::vector<int64_t> seen;
        size_t nb = 0;
        for (auto& b : seq) {
            ++nb;
            for (int64_t i = 0; i < b.target.size(0); ++i) seen.push_back(b.target[i].item<int64_t>());
            CHECK(b.data.size(1) == 2);
        }
        CHECK(nb == 3 && seen.size() == 10 && seen[0] == 0 && seen[9] == 9);
        pt::data::DataLoader dropped(ds, pt::data::DataLoaderOptions(4).drop_last(true));
        nb = 0;
        for (auto& b : dropped) { ++nb; CHECK(b.target.size(0) == 4); }
        CHECK(nb == 2);
        // the same seed gives the same shuffle; worker threads keep the sampler's order
        auto order = [&](size_t workers) {
            pt::data::DataLoader dl(ds, pt::data::DataLoaderOptions(3).shuffle(true).seed(5).num_workers(workers));
            std::vector<int64_t> v;
            for (auto& b : dl)
                for (int64_t i = 0; i < b.target.size(0); ++i) v.push_back(b.target[i].item<int64_t>());
            return v;
        };
        auto o0 = order(0), o3 = order(3);
        CHECK(o0.size() == 10 && o0 == o3);
        std::vector<int64_t> sorted = o0;
        std::sort(sorted.begin(), sorted.end());
        for (int i = 0; i < 10; ++i) CHECK(sorted[i] == i);
        CHECK(o0 != sorted);
        auto sub = std::make_shared<pt::data::Subset>(ds, std::vector<size_t>{7, 2});
        auto cat = std::make_shared<pt::data::ConcatDataset>(std::vector<pt::data::DatasetPtr>{sub, ds});
        CHECK(cat->size() == 12 && cat->get(0).target.item<int64_t>() == 7 && cat->get(2).target.item<int64_t>() == 0);
        auto mapped = std::make_shared<pt::data::MapDataset>(ds, [](pt::data::Example e) { e.data = e.data * 2; return e; });
        CHECK(mapped->get(3).data[1].item<float>() == 14.0f);
        pt::data::WeightedRandomSampler ws({0.0, 1.0, 0.0}, 5, 1);
        for (size_t i : ws.indices()) CHECK(i == 1);
        pt::data::DistributedSampler s0(10, 2, 0, true, 3), s1(10, 2, 1, true, 3);
        s0.set_epoch(1);
        s1.set_epoch(1);
        auto i0 = s0.indices(), i1 = s1.indices();
        CHECK(i0.size() == 5 && i1.size() == 5);
    }
    // GPipe == the stages in sequence
    {
        pt::manual_seed(1);
        pt::nn::Sequential a(pt::nn::Linear(6, 8), pt::nn::Tanh()), b(pt::nn::Linear(8, 3));
        auto pipe = pt::nn::parallel::Pipeline::from_modules({a, b}, 4);
        auto x = pt::randn({8, 6});
        CHECK(close(pipe.forward(x), b->forward(a->forward(x)), 1e-6) && pipe.num_stages() == 2);
        pipe.forward(x).sum().backward();
        CHECK(a->parameters()[0].grad().defined());
    }
    // offload optimizer == the plain optimizer
    {
        pt::manual_seed(2);
        auto w1 = pt::randn({4, 3}).set_requires_grad(true);
        auto w2 = w1.detach().clone().set_requires_grad(true);
        pt::deepspeed::OffloadOptimizer<pt::optim::AdamW> off({w1}, pt::optim::AdamWOptions(1e-2));
        pt::optim::AdamW plain({w2}, pt::optim::AdamWOptions(1e-2));
        for (int i = 0; i < 3; ++i) {
            off.zero_grad();
            plain.zero_grad();
            (w1 * w1).sum().backward();
            (w2 * w2).sum().backward();
            off.step();
            plain.step();
        }
        CHECK(close(w1.detach(), w2.detach(), 1e-6) && off.master_params()[0].device().is_cpu());
    }
    return 0;
}

int main(int argc, char** argv) {
    const int port = argc > 1 ? std::atoi(argv[1]) : 29800;
    // the forked parts first: a child forked after libtorch has started its worker threads would inherit their locks
    if (dist::launch(2, fsdp_rank, "127.0.0.1", port) != 0) { std::printf("FAIL fsdp ranks\n"); return 1; }
    if (dist::launch(2, pipeline_rank, "127.0.0.1", port + 20) != 0) { std::printf("FAIL pipeline ranks\n"); return 1; }
    if (single_process() != 0) return 1;
    if (quant_and_checkpoint() != 0) return 1;
    if (nn_extras() != 0) return 1;
    if (module_hooks() != 0) return 1;
    if (trainer_test(argc > 2 ? argv[2] : "/tmp/ptb_cpp_trainer") != 0) return 1;
    std::printf("CPP_PARALLEL_API_OK\n");
    return 0;
}
