// promethorch C++ API: batch normalisation whose statistics span all ranks.
//
// SyncBatchNorm normalises with the mean and variance of the GLOBAL batch: every rank contributes its per-channel sum,
// sum of squares and element count in one all-reduce ([2C + 1] floats; the reference issues three,
// torch/distributed/distributed.h:847-849), and the backward pass all-reduces the two per-channel gradient sums the
// input gradient needs.  convert_sync_batchnorm swaps the BatchNorm1d/2d children of a module tree for SyncBatchNorm
// carrying the same parameters and running statistics.
#pragma once
#include <torch/torch.h>

#include <memory>
#include <vector>

#include "distributed.h"

namespace promethorch {
namespace distributed {

namespace detail {
// x: [N, C, ...]; statistics over every dimension but 1.
struct SyncBNFunction : public torch::autograd::Function<SyncBNFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, Tensor x, Tensor weight, Tensor bias, Tensor running_mean, Tensor running_var,
                          double eps, double momentum, bool training, ProcessGroupPtr pg) {
        const int64_t C = x.size(1);
        std::vector<int64_t> red;
        for (int64_t d = 0; d < x.dim(); ++d)
            if (d != 1) red.push_back(d);
        std::vector<int64_t> shape(x.dim(), 1);
        shape[1] = C;
        Tensor mean, var;
        double count = (double)(x.numel() / C);
        if (training) {
            Tensor xf = x.to(torch::kFloat);
            Tensor stats = torch::cat({xf.sum(red), (xf * xf).sum(red), torch::full({1}, count)});
            if (pg && pg->world_size() > 1) pg->all_reduce(stats, ReduceOp::SUM);
            count = stats[2 * C].item<double>();
            mean = stats.narrow(0, 0, C) / count;
            var = stats.narrow(0, C, C) / count - mean * mean;
            if (running_mean.defined()) {
                torch::NoGradGuard ng;
                running_mean.mul_(1 - momentum).add_(mean, momentum);
                running_var.mul_(1 - momentum).add_(var * (count / std::max(count - 1.0, 1.0)), momentum);
            }
        } else {
            mean = running_mean.to(torch::kFloat);
            var = running_var.to(torch::kFloat);
        }
        Tensor invstd = torch::rsqrt(var + eps);
        Tensor xhat = (x.to(torch::kFloat) - mean.view(shape)) * invstd.view(shape);
        Tensor y = xhat;
        if (weight.defined()) y = y * weight.to(torch::kFloat).view(shape);
        if (bias.defined()) y = y + bias.to(torch::kFloat).view(shape);
        ctx->save_for_backward({xhat, invstd, weight.defined() ? weight : Tensor()});
        ctx->saved_data["count"] = count;
        ctx->saved_data["training"] = training;
        ctx->saved_data["has_bias"] = bias.defined();
        pg_slot() = pg;
        return y.to(x.dtype());
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grads) {
        auto saved = ctx->get_saved_variables();
        Tensor xhat = saved[0], invstd = saved[1], weight = saved[2];
        const double count = ctx->saved_data["count"].toDouble();
        const bool training = ctx->saved_data["training"].toBool();
        Tensor dy = grads[0].to(torch::kFloat);
        const int64_t C = xhat.size(1);
        std::vector<int64_t> red;
        for (int64_t d = 0; d < xhat.dim(); ++d)
            if (d != 1) red.push_back(d);
        std::vector<int64_t> shape(xhat.dim(), 1);
        shape[1] = C;
        Tensor dweight = weight.defined() ? (dy * xhat).sum(red) : Tensor();
        Tensor dbias = ctx->saved_data["has_bias"].toBool() ? dy.sum(red) : Tensor();
        Tensor g = weight.defined() ? dy * weight.to(torch::kFloat).view(shape) : dy;
        Tensor dx;
        if (training) {
            Tensor sums = torch::cat({g.sum(red), (g * xhat).sum(red)});      // over the global batch
            ProcessGroupPtr pg = pg_slot();
            if (pg && pg->world_size() > 1) pg->all_reduce(sums, ReduceOp::SUM);
            Tensor s1 = sums.narrow(0, 0, C).view(shape) / count, s2 = sums.narrow(0, C, C).view(shape) / count;
            dx = (g - s1 - xhat * s2) * invstd.view(shape);
        } else {
            dx = g * invstd.view(shape);
        }
        return {dx.to(grads[0].dtype()), dweight, dbias, Tensor(), Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
    }
    // the group of the most recent forward (module instances of one model share it)
    static ProcessGroupPtr& pg_slot() {
        static thread_local ProcessGroupPtr g;
        return g;
    }
};
}  // namespace detail

class SyncBatchNormImpl : public torch::nn::Module {
 public:
    explicit SyncBatchNormImpl(int64_t num_features, double eps = 1e-5, double momentum = 0.1, bool affine = true,
                               bool track_running_stats = true, ProcessGroupPtr pg = nullptr)
        : eps_(eps), momentum_(momentum), pg_(std::move(pg)) {
        if (affine) {
            weight = register_parameter("weight", torch::ones({num_features}));
            bias = register_parameter("bias", torch::zeros({num_features}));
        }
        if (track_running_stats) {
            running_mean = register_buffer("running_mean", torch::zeros({num_features}));
            running_var = register_buffer("running_var", torch::ones({num_features}));
        }
    }
    Tensor forward(const Tensor& x) {
        ProcessGroupPtr pg = pg_ ? pg_ : default_group();
        const bool batch_stats = is_training() || !running_mean.defined();
        return detail::SyncBNFunction::apply(x, weight, bias, running_mean, running_var, eps_, momentum_, batch_stats, pg);
    }
    Tensor weight, bias, running_mean, running_var;

 private:
    double eps_, momentum_;
    ProcessGroupPtr pg_;
};
TORCH_MODULE(SyncBatchNorm);

namespace detail {
template <typename BN>
inline SyncBatchNorm sync_from(BN* bn, ProcessGroupPtr pg) {
    const auto& o = bn->options;
    SyncBatchNorm s(o.num_features(), o.eps(), o.momentum().has_value() ? *o.momentum() : 0.1, o.affine(), o.track_running_stats(), pg);
    torch::NoGradGuard ng;
    if (o.affine()) { s->weight.copy_(bn->weight); s->bias.copy_(bn->bias); }
    if (o.track_running_stats()) { s->running_mean.copy_(bn->running_mean); s->running_var.copy_(bn->running_var); }
    s->train(bn->is_training());
    return s;
}
inline bool as_sync(torch::nn::Module* m, ProcessGroupPtr pg, SyncBatchNorm& out) {
    if (auto* b1 = dynamic_cast<torch::nn::BatchNorm1dImpl*>(m)) { out = sync_from(b1, pg); return true; }
    if (auto* b2 = dynamic_cast<torch::nn::BatchNorm2dImpl*>(m)) { out = sync_from(b2, pg); return true; }
    if (auto* b3 = dynamic_cast<torch::nn::BatchNorm3dImpl*>(m)) { out = sync_from(b3, pg); return true; }
    return false;
}
}  // namespace detail

// A Sequential with every BatchNorm1d / 2d / 3d layer replaced by a SyncBatchNorm carrying the same parameters and running
// statistics; the other layers are shared with the original.
inline torch::nn::Sequential convert_sync_batchnorm(const torch::nn::Sequential& seq, ProcessGroupPtr pg = nullptr) {
    torch::nn::Sequential out;
    for (auto& any : *seq) {
        std::shared_ptr<torch::nn::Module> m = any.ptr();
        SyncBatchNorm s{nullptr};
        if (detail::as_sync(m.get(), pg, s)) out->push_back(s);
        else out->push_back(any);
    }
    return out;
}
// For a module with registered children: swaps the registered BatchNorm children (recursively) and returns how many.
// libtorch keeps member holders and Sequential's own list apart from the registry, so a module that calls its layers
// through members must re-assign them from named_children() afterwards (use the Sequential overload for Sequentials).
inline int convert_sync_batchnorm(torch::nn::Module& module, ProcessGroupPtr pg = nullptr) {
    int n = 0;
    for (auto& child : module.named_children()) {
        torch::nn::Module* m = child.value().get();
        SyncBatchNorm s{nullptr};
        if (detail::as_sync(m, pg, s)) {
            module.replace_module(child.key(), s.ptr());
            ++n;
        } else n += convert_sync_batchnorm(*m, pg);
    }
    return n;
}

}  // namespace distributed
}  // namespace promethorch
