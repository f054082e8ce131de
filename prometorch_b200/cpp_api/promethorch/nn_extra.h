// promethorch C++ API: the modules and fused functions the reference has and libtorch's C++ front end lacks.
//
// Losses: FocalLoss, DiceLoss, GaussianNLLLoss (torch/nn/modules/loss.h).  Layers: GlobalAvgPool2d, PositionalEncoding,
// Dropout1d, LazyLinear (its weight takes shape at the first call), QuantizedConv2d.  Functions: fused_linear,
// fused_linear_relu, fused_mlp (one call for bias + activation chains, FusedBackward.h of the reference), rms_norm,
// rotary_embedding, parallel_scan (a first-order linear recurrence), and num_parameters.
#pragma once
#include <torch/torch.h>

#include <cmath>
#include <string>
#include <vector>

namespace promethorch {
namespace nn {
using Tensor = at::Tensor;

namespace detail {
inline Tensor reduce(const Tensor& v, const std::string& reduction) {
    if (reduction == "mean") return v.mean();
    if (reduction == "sum") return v.sum();
    TORCH_CHECK(reduction == "none", "reduction must be none, mean or sum");
    return v;
}
}  // namespace detail

// Binary focal loss on probabilities: -alpha_t (1 - p_t)^gamma log p_t.
class FocalLossImpl : public torch::nn::Module {
 public:
    explicit FocalLossImpl(std::string reduction = "mean", double alpha = 0.25, double gamma = 2.0)
        : reduction_(std::move(reduction)), alpha_(alpha), gamma_(gamma) {}
    Tensor forward(const Tensor& input, const Tensor& target) {
        TORCH_CHECK(input.sizes() == target.sizes(), "Input and target must have the same shape");
        Tensor p = input.clamp(1e-7, 1 - 1e-7);
        Tensor pt = target * p + (1 - target) * (1 - p);
        Tensor at = target * alpha_ + (1 - target) * (1 - alpha_);
        return detail::reduce(-at * (1 - pt).pow(gamma_) * pt.log(), reduction_);
    }

 private:
    std::string reduction_;
    double alpha_, gamma_;
};
TORCH_MODULE(FocalLoss);

// 1 - (2 sum(xy) + s) / (sum x + sum y + s) per sample.
class DiceLossImpl : public torch::nn::Module {
 public:
    explicit DiceLossImpl(std::string reduction = "mean", double smooth = 1.0) : reduction_(std::move(reduction)), smooth_(smooth) {}
    Tensor forward(const Tensor& input, const Tensor& target) {
        TORCH_CHECK(input.sizes() == target.sizes(), "Input and target must have the same shape");
        Tensor x = input.flatten(1), y = target.flatten(1);
        Tensor dice = (2 * (x * y).sum(1) + smooth_) / (x.sum(1) + y.sum(1) + smooth_);
        return detail::reduce(1 - dice, reduction_);
    }

 private:
    std::string reduction_;
    double smooth_;
};
TORCH_MODULE(DiceLoss);

// 0.5 (log max(var, eps) + (x - target)^2 / max(var, eps)) [+ 0.5 log 2 pi].
class GaussianNLLLossImpl : public torch::nn::Module {
 public:
    explicit GaussianNLLLossImpl(bool full = false, double eps = 1e-6, std::string reduction = "mean")
        : full_(full), eps_(eps), reduction_(std::move(reduction)) {}
    Tensor forward(const Tensor& input, const Tensor& target, const Tensor& var) {
        TORCH_CHECK((var.detach() >= 0).all().item<bool>(), "var has negative entries");
        Tensor v = var.clamp_min(eps_);
        Tensor loss = 0.5 * (v.log() + (input - target).pow(2) / v);
        if (full_) loss = loss + 0.5 * std::log(2 * M_PI);
        return detail::reduce(loss, reduction_);
    }

 private:
    bool full_;
    double eps_;
    std::string reduction_;
};
TORCH_MODULE(GaussianNLLLoss);

class GlobalAvgPool2dImpl : public torch::nn::Module {
 public:
    Tensor forward(const Tensor& x) { return x.mean({-2, -1}); }
};
TORCH_MODULE(GlobalAvgPool2d);

// Sinusoidal positions added to [T, B, D] (or [B, T, D] with batch_first), then dropout.
class PositionalEncodingImpl : public torch::nn::Module {
 public:
    explicit PositionalEncodingImpl(int64_t d_model, double dropout = 0.1, int64_t max_len = 5000, bool batch_first = false) : batch_first_(batch_first) {
        drop = register_module("dropout", torch::nn::Dropout(dropout));
        Tensor pos = torch::arange(max_len, torch::kFloat).unsqueeze(1);
        Tensor div = torch::exp(torch::arange(0, d_model, 2, torch::kFloat) * (-std::log(10000.0) / (double)d_model));
        Tensor table = torch::zeros({max_len, d_model});
        table.slice(1, 0, d_model, 2).copy_(torch::sin(pos * div));
        table.slice(1, 1, d_model, 2).copy_(torch::cos(pos * div).slice(1, 0, d_model / 2));
        pe = register_buffer("pe", table);
    }
    Tensor forward(const Tensor& x) {
        if (batch_first_) return drop(x + pe.slice(0, 0, x.size(1)).unsqueeze(0));
        return drop(x + pe.slice(0, 0, x.size(0)).unsqueeze(1));
    }
    Tensor pe;
    torch::nn::Dropout drop{nullptr};

 private:
    bool batch_first_;
};
TORCH_MODULE(PositionalEncoding);

// Whole channels of [N, C, L] (or [C, L]) dropped together.
class Dropout1dImpl : public torch::nn::Module {
 public:
    explicit Dropout1dImpl(double p = 0.5) : p_(p) {}
    Tensor forward(const Tensor& x) {
        TORCH_CHECK(x.dim() == 2 || x.dim() == 3, "Dropout1d: expected [C, L] or [N, C, L]");
        if (!is_training() || p_ == 0) return x;
        const bool batched = x.dim() == 3;
        Tensor y = torch::feature_dropout(batched ? x : x.unsqueeze(0), p_, true);
        return batched ? y : y.squeeze(0);
    }

 private:
    double p_;
};
TORCH_MODULE(Dropout1d);

// A linear layer whose input width is read from the first batch it sees.
class LazyLinearImpl : public torch::nn::Module {
 public:
    explicit LazyLinearImpl(int64_t out_features, bool bias = true) : out_(out_features), with_bias_(bias) {}
    Tensor forward(const Tensor& x) {
        if (!weight.defined()) materialize(x.size(-1), x.options());
        return torch::nn::functional::linear(x, weight, bias);
    }
    bool has_uninitialized_params() const { return !weight.defined(); }
    Tensor weight, bias;

 private:
    void materialize(int64_t in, const at::TensorOptions& like) {
        const double bound = 1.0 / std::sqrt((double)in);
        weight = register_parameter("weight", torch::empty({out_, in}, like.requires_grad(false)).uniform_(-bound, bound));
        if (with_bias_) bias = register_parameter("bias", torch::empty({out_}, like.requires_grad(false)).uniform_(-bound, bound));
    }
    int64_t out_;
    bool with_bias_;
};
TORCH_MODULE(LazyLinear);

// A convolution with int8 weights (one scale per output channel) dequantised on the fly.
class QuantizedConv2dImpl : public torch::nn::Module {
 public:
    explicit QuantizedConv2dImpl(const torch::nn::Conv2d& conv) : opt_(conv->options) {
        torch::NoGradGuard ng;
        Tensor w = conv->weight.detach().to(torch::kFloat);
        Tensor s = w.abs().amax({1, 2, 3}, true).clamp_min(1e-12) / 127.0;
        qweight = register_buffer("qweight", torch::round(w / s).clamp(-127, 127).to(torch::kChar));
        scale = register_buffer("scale", s);
        if (conv->bias.defined()) bias = register_buffer("bias", conv->bias.detach().clone());
    }
    Tensor forward(const Tensor& x) {
        Tensor w = (qweight.to(torch::kFloat) * scale).to(x.dtype());
        const auto& pad = opt_.padding();
        TORCH_CHECK(std::holds_alternative<torch::ExpandingArray<2>>(pad), "QuantizedConv2d: numeric padding only");
        return torch::conv2d(x, w, bias, *opt_.stride(), *std::get<torch::ExpandingArray<2>>(pad), *opt_.dilation(), opt_.groups());
    }
    Tensor qweight, scale, bias;

 private:
    torch::nn::detail::ConvNdOptions<2> opt_;
};
TORCH_MODULE(QuantizedConv2d);

inline int64_t num_parameters(const torch::nn::Module& m, bool only_trainable = false) {
    int64_t n = 0;
    for (const auto& p : m.parameters())
        if (p.requires_grad() || !only_trainable) n += p.numel();
    return n;
}

namespace functional {
using namespace ::torch::nn::functional;

inline Tensor fused_linear(const Tensor& x, const Tensor& w, const Tensor& b = {}) { return torch::nn::functional::linear(x, w, b); }
inline Tensor fused_linear_relu(const Tensor& x, const Tensor& w, const Tensor& b = {}) { return torch::relu(torch::nn::functional::linear(x, w, b)); }
// relu(linear) for every layer but the last.
inline Tensor fused_mlp(const Tensor& x, const std::vector<Tensor>& weights, const std::vector<Tensor>& biases = {}) {
    Tensor h = x;
    for (size_t i = 0; i < weights.size(); ++i) {
        h = torch::nn::functional::linear(h, weights[i], i < biases.size() ? biases[i] : Tensor());
        if (i + 1 < weights.size()) h = torch::relu(h);
    }
    return h;
}
inline Tensor rms_norm(const Tensor& x, const Tensor& weight, double eps = 1e-6, bool add_one = false) {
    Tensor v = x.to(torch::kFloat);
    Tensor n = v * torch::rsqrt(v.pow(2).mean(-1, true) + eps);
    return (n * (add_one ? weight + 1 : weight)).to(x.dtype());
}
// NeoX-style rotation of x[..., T, D] by position: the two halves of the head rotate against each other.
inline Tensor rotary_embedding(const Tensor& x, const Tensor& positions, double theta = 10000.0) {
    const int64_t d = x.size(-1), half = d / 2;
    Tensor inv = torch::pow(theta, -torch::arange(0, half, x.options().dtype(torch::kFloat)) / (double)half);
    Tensor ang = positions.to(torch::kFloat).unsqueeze(-1) * inv;
    Tensor c = ang.cos(), s = ang.sin();
    Tensor a = x.slice(-1, 0, half).to(torch::kFloat), b = x.slice(-1, half, d).to(torch::kFloat);
    return torch::cat({a * c - b * s, b * c + a * s}, -1).to(x.dtype());
}
// h_t = a_t h_{t-1} + b_t along `dim`, h_{-1} = 0, by log-depth doubling (every step is one fused elementwise pass).
inline Tensor parallel_scan(const Tensor& a, const Tensor& b, int64_t dim = -1) {
    Tensor A = a.movedim(dim, -1).contiguous(), B = b.movedim(dim, -1).contiguous();
    const int64_t T = A.size(-1);
    for (int64_t step = 1; step < T; step *= 2) {
        Tensor Ap = torch::constant_pad_nd(A.slice(-1, 0, T - step), {step, 0}, 1.0);
        Tensor Bp = torch::constant_pad_nd(B.slice(-1, 0, T - step), {step, 0}, 0.0);
        B = A * Bp + B;
        A = A * Ap;
    }
    return B.movedim(-1, dim);
}
}  // namespace functional

}  // namespace nn
}  // namespace promethorch
