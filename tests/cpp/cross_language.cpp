// What the C++ API computes, printed so that the Python package can compute the same and compare (the two are separate
// implementations of the same rules):
//   (no arguments)          every element-wise optimizer for a few steps on a fixed, formula-made sequence of gradients
//                           ("NAME v v v ..."), and the learning-rate sequence of every scheduler ("S:NAME lr lr ...")
//   io DIR                  checkpoints written by Python read and written back (PTOR container, PyTorch zip)
//   llama DIR OUT           a Hugging Face Llama directory: logits, greedy and sampled continuation, safetensors written back
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

// One learning-rate sequence per scheduler: "S:NAME lr lr lr ..." (the rate after construction, then after every step).
template <typename Make>
static void schedule(const char* name, Make make, int steps = 24) {
    using namespace pt::optim;
    auto w = pt::zeros({2}).requires_grad_(true);
    SGD opt({w}, SGDOptions(0.5));
    auto stepper = make(opt);
    std::printf("S:%s %.12g", name, opt.get_lr(0));
    for (int i = 0; i < steps; ++i) {
        stepper(i);
        std::printf(" %.12g", opt.get_lr(0));
    }
    std::printf("\n");
}

static void schedulers() {
    using namespace pt::optim;
    auto plain = [](auto sched) { return [sched](int) { sched->step(); }; };
    schedule("StepLR", [&](SGD& o) { return plain(std::make_shared<StepLR>(o, 5, 0.5)); });
    schedule("MultiStepLR", [&](SGD& o) { return plain(std::make_shared<MultiStepLR>(o, std::vector<int64_t>{3, 7, 15}, 0.3)); });
    schedule("ExponentialLR", [&](SGD& o) { return plain(std::make_shared<ExponentialLR>(o, 0.9)); });
    schedule("CosineAnnealingLR", [&](SGD& o) { return plain(std::make_shared<CosineAnnealingLR>(o, 10, 0.01)); });
    schedule("LinearLR", [&](SGD& o) { return plain(std::make_shared<LinearLR>(o, 0.25, 1.0, 8)); });
    schedule("ConstantLR", [&](SGD& o) { return plain(std::make_shared<ConstantLR>(o, 0.2, 6)); });
    schedule("WarmupCosineAnnealingLR", [&](SGD& o) { return plain(std::make_shared<WarmupCosineAnnealingLR>(o, 4, 20, 0.05)); });
    schedule("OneCycleLR", [&](SGD& o) { return plain(std::make_shared<OneCycleLR>(o, 1.0, 24, 0.25)); });
    schedule("CosineAnnealingWarmRestarts", [&](SGD& o) { return plain(std::make_shared<CosineAnnealingWarmRestarts>(o, 4, 2, 0.02)); });
    schedule("CyclicLR", [&](SGD& o) { return plain(std::make_shared<CyclicLR>(o, 0.1, 0.9, 3, 5)); });
    schedule("CyclicLR_triangular2", [&](SGD& o) { return plain(std::make_shared<CyclicLR>(o, 0.1, 0.9, 2, -1, CyclicLR::Mode::Triangular2)); });
    schedule("PolynomialLR", [&](SGD& o) { return plain(std::make_shared<PolynomialLR>(o, 12, 2.0)); });
    schedule("LambdaLR", [&](SGD& o) { return plain(std::make_shared<LambdaLR>(o, [](int64_t e) { return 1.0 / (1.0 + 0.5 * e); })); });
    schedule("MultiplicativeLR", [&](SGD& o) { return plain(std::make_shared<MultiplicativeLR>(o, [](int64_t e) { return e % 3 == 0 ? 0.8 : 1.0; })); });
    schedule("ReduceLROnPlateau", [&](SGD& o) {
        auto s = std::make_shared<ReduceLROnPlateau>(o, ReduceLROnPlateau::Mode::Min, 0.5, 2, 1e-3, 0.01);
        return [s](int i) { s->step(i < 5 ? 1.0 - 0.1 * i : 0.7); };
    });
    schedule("SequentialLR", [&](SGD& o) {
        std::vector<std::shared_ptr<LRScheduler>> parts{std::make_shared<LinearLR>(o, 0.1, 1.0, 5), std::make_shared<ExponentialLR>(o, 0.8)};
        return plain(std::make_shared<SequentialLR>(o, parts, std::vector<int64_t>{5}));
    });
    schedule("ChainedScheduler", [&](SGD& o) {
        std::vector<std::shared_ptr<LRScheduler>> parts{std::make_shared<StepLR>(o, 4, 0.5), std::make_shared<ExponentialLR>(o, 0.95)};
        return plain(std::make_shared<ChainedScheduler>(o, parts));
    });
}

// Checkpoints across the two languages: read what Python wrote (PTOR container and a PyTorch zip), print name, dtype, shape and
// sums, then write the same tensors back for Python to read.
static int checkpoints(const std::string& dir) {
    for (const char* kind : {"ptor", "pt"}) {
        const std::string path = dir + "/py." + kind;
        auto sd = std::string(kind) == "ptor" ? pt::load_state_dict(path) : pt::load_pytorch(path);
        for (const auto& kv : sd) {
            std::printf("C:%s %s %s", kind, kv.first.c_str(), c10::toString(kv.second.scalar_type()));
            for (auto d : kv.second.sizes()) std::printf(" %lld", (long long)d);
            std::printf(" | %.9g %.9g\n", kv.second.to(pt::kDouble).sum().item<double>(),
                        kv.second.numel() ? kv.second.to(pt::kDouble).abs().max().item<double>() : 0.0);
        }
        if (std::string(kind) == "ptor") pt::save_state_dict(sd, dir + "/cpp.ptor");
        else pt::save_pytorch(sd, dir + "/cpp.pt");
    }
    return 0;
}

// A Hugging Face Llama directory: logits of a prompt, greedy continuation, and the safetensors round trip.
static int llama(const std::string& dir, const std::string& out_path) {
    auto cfg = pt::models::LlamaConfig::from_json(dir + "/config.json");
    pt::models::Llama model(cfg);
    model->load_hf(dir);
    model->eval();
    pt::NoGradGuard ng;
    const std::vector<int64_t> prompt{1, 17, 250, 3, 99, 42};
    auto logits = model->forward(pt::tensor(prompt, pt::kLong).unsqueeze(0));
    std::printf("L:shape %lld %lld %lld\n", (long long)logits.size(0), (long long)logits.size(1), (long long)logits.size(2));
    std::printf("L:last");
    auto last = logits[0][(int64_t)prompt.size() - 1].to(pt::kDouble);
    for (int64_t i = 0; i < 16; ++i) std::printf(" %.7g", last[i].item<double>());
    std::printf("\nL:argmax");
    auto am = logits[0].argmax(-1);
    for (int64_t i = 0; i < am.numel(); ++i) std::printf(" %lld", (long long)am[i].item<int64_t>());
    std::printf("\nL:greedy");
    for (auto t : model->generate(prompt, 10, 0.0, 0, false)) std::printf(" %lld", (long long)t);
    std::printf("\nL:sampled");
    pt::manual_seed(3);
    for (auto t : model->generate(prompt, 6, 0.9, 20, false)) std::printf(" %lld", (long long)t);
    std::printf("\n");
    pt::save_safetensors(model->hf_state_dict(), out_path, {{"format", "pt"}});
    return 0;
}

// vision / text / audio helpers on inputs the Python test wrote into DIR; results as "E:name v v v ..." lines and files.
static void line(const char* name, const pt::Tensor& t) {
    std::printf("E:%s", name);
    auto f = t.reshape(-1).to(pt::kDouble);
    for (int64_t i = 0; i < f.numel(); ++i) std::printf(" %.9g", f[i].item<double>());
    std::printf("\n");
}
static int ecosystem(const std::string& dir) {
    namespace V = pt::vision;
    namespace T = pt::text;
    namespace A = pt::audio;
    auto img = V::load_pnm(dir + "/py.ppm");
    line("ppm_shape", pt::tensor({img.size(0), img.size(1), img.size(2)}));
    line("ppm_sum", img.sum());
    line("pgm_ascii", V::load_pnm(dir + "/ascii.pgm"));
    V::save_pnm(dir + "/cpp.ppm", img);
    auto tf = V::transforms::Compose({V::transforms::Resize(6, 8), V::transforms::CenterCrop(4), V::transforms::Normalize({0.5, 0.4, 0.3}, {0.2, 0.3, 0.4})});
    line("transformed", tf(img));
    line("random_crop_shape", pt::tensor({V::transforms::RandomCrop(3, 2, 1)(img).size(1), V::transforms::RandomCrop(3, 2, 1)(img).size(2)}));
    line("flip", V::transforms::RandomHorizontalFlip(1.0)(img).slice(0, 0, 1).slice(1, 0, 1));
    V::ImageFolder folder(dir + "/set", V::transforms::Resize(8));
    line("folder", pt::tensor({(int64_t)folder.size(), (int64_t)folder.classes.size(), folder.get(folder.size() - 1).second, folder.get(0).first.size(1)}));
    std::printf("E:classes %s %s\n", folder.classes[0].c_str(), folder.classes[1].c_str());
    // text
    auto vocab = T::Vocab::build({"the cat sat", "the dog sat down", "a cat"}, 1);
    line("vocab_encode", pt::tensor(vocab.encode("the cat flew down")));
    std::printf("E:vocab_decode %s\n", vocab.decode({2, 4, 3}).c_str());
    std::printf("E:basic");
    for (const auto& t : T::BasicTokenizer().tokenize("Hello, World! it's")) std::printf(" %s", t.c_str());
    std::printf("\n");
    T::CharTokenizer ct("hello world");
    line("char", pt::tensor(ct.encode("held z")));
    T::WordPieceTokenizer wp({"[UNK]", "un", "##aff", "##able", "play", "##ing", "##ed"});
    line("wordpiece", pt::tensor(wp.encode("unaffable playing xyz played")));
    std::vector<std::vector<int64_t>> batch{{1, 2, 3}, {4}, {5, 6}};
    line("pad", T::pad_sequence(batch, 9, true, 2));
    line("pad_tb", T::pad_sequence(batch, 0, false));
    line("lengths", T::sequence_lengths(batch));
    line("mask", T::padding_mask(batch).to(pt::kLong));
    // audio
    auto t = pt::linspace(0, 1, 16000);
    auto x = pt::sin(2 * M_PI * 440 * t);
    auto spec = A::spectrogram(x, 400, 160);
    line("spec_shape", pt::tensor({spec.size(0), spec.size(1)}));
    line("spec_peak", spec.mean(1).argmax());
    line("spec_probe", spec.slice(0, 9, 13).slice(1, 10, 12));
    line("fbanks_sum", A::melscale_fbanks(201, 40, 16000).sum(0));
    line("mfcc_probe", A::mfcc(x).slice(0, 0, 4).slice(1, 5, 7));
    auto q = A::mu_law_encoding(x.slice(0, 0, 64));
    line("mulaw", q);
    line("mulaw_back", A::mu_law_decoding(q));
    line("db", A::amplitude_to_db(spec.slice(0, 9, 13).slice(1, 10, 12), 10.0, 1e-10, 0.0, 20.0));
    line("resample", A::resample(x.slice(0, 0, 100), 16000, 8000));
    auto wav = A::load_wav(dir + "/py.wav");
    line("wav", pt::tensor({(double)wav.second, (double)wav.first.numel(), wav.first.abs().max().item<double>()}));
    A::save_wav(dir + "/cpp.wav", x.slice(0, 0, 800), 8000);
    return 0;
}

// The exporters: a Sequential built from the weights Python saved in DIR/mlp.ptor, written as ONNX, MLIR and PTMB; the PTMB
// file Python wrote is run by the C++ executor.
static int exporters(const std::string& dir) {
    auto sd = pt::load_state_dict(dir + "/mlp.ptor");
    // (libtorch cannot nest a Sequential in a Sequential; the Python model nests one, the op order is the same)
    pt::nn::Sequential seq(pt::nn::Linear(6, 5), pt::nn::ReLU(), pt::nn::Linear(5, 4), pt::nn::Tanh(), pt::nn::Linear(pt::nn::LinearOptions(4, 3).bias(false)), pt::nn::Softmax(-1));
    pt::NoGradGuard ng;
    auto params = seq->parameters();
    if (params.size() != sd.size()) { std::printf("FAIL %zu parameters against %zu tensors\n", params.size(), sd.size()); return 1; }
    for (size_t i = 0; i < params.size(); ++i) params[i].copy_(sd[i].second);
    pt::onnx::export_model(*seq, {2, 6}, dir + "/cpp.onnx");
    pt::mlir::export_mlir(*seq, {2, 6}, dir + "/cpp.mlir");
    pt::mobile::export_model(*seq, dir + "/cpp.ptmb");
    pt::mobile::MobileExecutor exec(dir + "/py.ptmb");
    auto x = pt::arange(12, pt::kFloat).reshape({2, 6}) / 10.0;
    line("mobile", exec.run(x));
    line("direct", seq->forward(x));
    return 0;
}

int main(int argc, char** argv) {
    using namespace pt::optim;
    if (argc > 2 && std::string(argv[1]) == "export") return exporters(argv[2]);
    if (argc > 2 && std::string(argv[1]) == "ecosystem") return ecosystem(argv[2]);
    if (argc > 2 && std::string(argv[1]) == "io") return checkpoints(argv[2]);
    if (argc > 3 && std::string(argv[1]) == "llama") return llama(argv[2], argv[3]);
    schedulers();
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
