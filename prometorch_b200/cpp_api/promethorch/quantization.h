// promethorch C++ API: quantisation.
//
// MinMaxObserver, FakeQuantize (quantise-dequantise in forward, straight-through gradient inside the representable range),
// QATLinear, int8 weight-quantised QuantizedLinear, quantize_per_tensor / int8_matmul with exact int32 accumulation, and
// 4-bit block formats (INT4, NF4) with Linear4bit (torch/quantization/*.h of the reference).
#pragma once
#include <torch/torch.h>

#include <cmath>
#include <string>
#include <utility>
#include <vector>

namespace promethorch {
namespace quantization {
using Tensor = at::Tensor;

class MinMaxObserverImpl : public torch::nn::Module {
 public:
    explicit MinMaxObserverImpl(int bits = 8, bool symmetric = true, double momentum = 0.0) : bits_(bits), symmetric_(symmetric), momentum_(momentum) {
        min_val = register_buffer("min_val", torch::tensor(INFINITY));
        max_val = register_buffer("max_val", torch::tensor(-INFINITY));
    }
    Tensor forward(const Tensor& x) {
        if (!frozen) {
            torch::NoGradGuard ng;
            Tensor mn = x.detach().amin(), mx = x.detach().amax();
            if (momentum_ > 0 && std::isfinite(min_val.item<float>())) {
                min_val.mul_(momentum_).add_(mn * (1 - momentum_));
                max_val.mul_(momentum_).add_(mx * (1 - momentum_));
            } else {
                min_val.copy_(torch::minimum(min_val, mn));
                max_val.copy_(torch::maximum(max_val, mx));
            }
        }
        return x;
    }
    // (scale, zero point)
    std::pair<Tensor, Tensor> qparams() const {
        const double qmax = symmetric_ ? std::pow(2.0, bits_ - 1) - 1 : std::pow(2.0, bits_) - 1;
        if (symmetric_) {
            Tensor scale = torch::maximum(max_val.abs(), min_val.abs()).clamp_min(1e-12) / qmax;
            return {scale, torch::zeros_like(scale)};
        }
        Tensor scale = (max_val - min_val).clamp_min(1e-12) / qmax;
        return {scale, torch::round(-min_val / scale)};
    }
    Tensor min_val, max_val;
    bool frozen = false;

 private:
    int bits_;
    bool symmetric_;
    double momentum_;
};
TORCH_MODULE(MinMaxObserver);

namespace detail {
struct FakeQuantSTE : public torch::autograd::Function<FakeQuantSTE> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, Tensor x, Tensor scale, Tensor zp, double qmin, double qmax) {
        Tensor v = x / scale + zp;
        ctx->save_for_backward({(v >= qmin).logical_and(v <= qmax)});
        return (torch::clamp(torch::round(x / scale) + zp, qmin, qmax) - zp) * scale;
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list g) {
        return {g[0] * ctx->get_saved_variables()[0], Tensor(), Tensor(), Tensor(), Tensor()};
    }
};
}  // namespace detail

class FakeQuantizeImpl : public torch::nn::Module {
 public:
    explicit FakeQuantizeImpl(int bits = 8, bool symmetric = true) : bits_(bits), symmetric_(symmetric) {
        observer = register_module("observer", MinMaxObserver(bits, symmetric));
    }
    Tensor forward(const Tensor& x) {
        observer->forward(x);
        if (!enabled) return x;
        auto qp = observer->qparams();
        const double qmin = symmetric_ ? -std::pow(2.0, bits_ - 1) : 0.0;
        const double qmax = symmetric_ ? std::pow(2.0, bits_ - 1) - 1 : std::pow(2.0, bits_) - 1;
        return detail::FakeQuantSTE::apply(x, qp.first, qp.second, qmin, qmax);
    }
    void freeze() { observer->frozen = true; }
    MinMaxObserver observer{nullptr};
    bool enabled = true;

 private:
    int bits_;
    bool symmetric_;
};
TORCH_MODULE(FakeQuantize);

// A linear layer trained through fake-quantised weights and activations.
class QATLinearImpl : public torch::nn::Module {
 public:
    QATLinearImpl(int64_t in, int64_t out, bool bias = true, int bits = 8) {
        linear = register_module("linear", torch::nn::Linear(torch::nn::LinearOptions(in, out).bias(bias)));
        weight_fq = register_module("weight_fq", FakeQuantize(bits));
        act_fq = register_module("act_fq", FakeQuantize(bits));
    }
    explicit QATLinearImpl(torch::nn::Linear from, int bits = 8) {
        linear = register_module("linear", std::move(from));          // weights shared with the float layer
        weight_fq = register_module("weight_fq", FakeQuantize(bits));
        act_fq = register_module("act_fq", FakeQuantize(bits));
    }
    Tensor forward(const Tensor& x) { return torch::nn::functional::linear(act_fq(x), weight_fq(linear->weight), linear->bias); }
    torch::nn::Linear linear{nullptr};
    FakeQuantize weight_fq{nullptr}, act_fq{nullptr};
};
TORCH_MODULE(QATLinear);

// (int8 tensor, scale): symmetric per-tensor quantisation.
inline std::pair<Tensor, Tensor> quantize_per_tensor(const Tensor& x, int bits = 8) {
    const double qmax = std::pow(2.0, bits - 1) - 1;
    Tensor scale = x.abs().amax().clamp_min(1e-12) / qmax;
    return {torch::round(x / scale).clamp(-qmax, qmax).to(torch::kChar), scale};
}
// (a_q * a_scale) @ (b_q * b_scale) with exact int32 accumulation.
inline Tensor int8_matmul(const Tensor& a_q, const Tensor& a_scale, const Tensor& b_q, const Tensor& b_scale) {
    Tensor acc = a_q.is_cuda() ? a_q.to(torch::kFloat).matmul(b_q.to(torch::kFloat)) : a_q.to(torch::kInt).matmul(b_q.to(torch::kInt)).to(torch::kFloat);
    return acc.to(torch::kFloat) * (a_scale * b_scale);
}

// Inference layer with int8 weights (per output row) dequantised on the fly.
class QuantizedLinearImpl : public torch::nn::Module {
 public:
    explicit QuantizedLinearImpl(const torch::nn::Linear& lin) {
        torch::NoGradGuard ng;
        Tensor w = lin->weight.detach().to(torch::kFloat);
        Tensor s = w.abs().amax(1, true).clamp_min(1e-12) / 127.0;
        weight_q = register_buffer("weight_q", torch::round(w / s).clamp(-127, 127).to(torch::kChar));
        scale = register_buffer("scale", s);
        if (lin->bias.defined()) bias = register_buffer("bias", lin->bias.detach().clone());
    }
    Tensor forward(const Tensor& x) {
        return torch::nn::functional::linear(x, (weight_q.to(torch::kFloat) * scale).to(x.dtype()), bias.defined() ? bias.to(x.dtype()) : bias);
    }
    Tensor weight_q, scale, bias;
};
TORCH_MODULE(QuantizedLinear);

// ---- 4-bit block formats
inline Tensor nf4_table() {
    return torch::tensor({-1.0f, -0.6961928f, -0.5250730f, -0.3949175f, -0.2844414f, -0.1848449f, -0.0910500f, 0.0f, 0.0795803f, 0.1609302f,
                          0.2461123f, 0.3379152f, 0.4407098f, 0.5626170f, 0.7229568f, 1.0f});
}
// (packed uint8 [numel / 2], absmax [numel / block])
inline std::pair<Tensor, Tensor> quantize_4bit(const Tensor& w, int64_t block = 64, const std::string& kind = "nf4") {
    Tensor flat = w.detach().to(torch::kFloat).reshape({-1, block});
    Tensor absmax = flat.abs().amax(1).clamp_min(1e-12);
    Tensor x = flat / absmax.unsqueeze(1);
    Tensor idx;
    if (kind == "nf4") idx = (x.unsqueeze(-1) - nf4_table().to(x.device())).abs().argmin(-1);
    else idx = torch::round(x * 7).clamp(-8, 7).to(torch::kLong) + 8;
    idx = idx.reshape(-1).to(torch::kByte);
    const int64_t n = idx.numel();
    Tensor lo = idx.slice(0, 0, n, 2), hi = idx.slice(0, 1, n, 2);
    return {lo.bitwise_or(hi.bitwise_left_shift(4)), absmax};
}
inline Tensor dequantize_4bit(const Tensor& packed, const Tensor& absmax, at::IntArrayRef shape, int64_t block = 64, const std::string& kind = "nf4") {
    Tensor idx = torch::stack({packed.bitwise_and(0xF), packed.bitwise_right_shift(4)}, 1).reshape(-1).to(torch::kLong);
    Tensor vals = kind == "nf4" ? nf4_table().to(packed.device()).index_select(0, idx) : (idx.to(torch::kFloat) - 8) / 7;
    return (vals.reshape({-1, block}) * absmax.unsqueeze(1)).reshape(shape);
}
class Linear4bitImpl : public torch::nn::Module {
 public:
    explicit Linear4bitImpl(const torch::nn::Linear& lin, int64_t block = 64, std::string kind = "nf4")
        : shape_(lin->weight.sizes().vec()), block_(block), kind_(std::move(kind)) {
        auto q = quantize_4bit(lin->weight, block_, kind_);
        packed = register_buffer("packed", q.first);
        absmax = register_buffer("absmax", q.second);
        if (lin->bias.defined()) bias = register_parameter("bias", lin->bias.detach().clone());
    }
    Tensor forward(const Tensor& x) {
        return torch::nn::functional::linear(x, dequantize_4bit(packed, absmax, shape_, block_, kind_).to(x.dtype()), bias);
    }
    Tensor packed, absmax, bias;

 private:
    std::vector<int64_t> shape_;
    int64_t block_;
    std::string kind_;
};
TORCH_MODULE(Linear4bit);

}  // namespace quantization
}  // namespace promethorch
