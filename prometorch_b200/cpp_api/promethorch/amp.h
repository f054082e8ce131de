// promethorch C++ API: mixed precision.
//
//  * GradScaler (torch/amp/grad_scaler.h:48-231 of the reference): scale(loss), unscale(optimizer) once per step with an
//    inf/nan check over every gradient, step(optimizer) that skips the update when one was found, update() that backs the
//    scale off or grows it after `growth_interval` clean steps, state_dict / load_state_dict.
//  * AutocastGuard / AutocastCPUGuard (torch/amp/autocast.h): RAII switch of libtorch's autocast for a device type and a
//    lower-precision dtype; the per-op policy (matmul-like ops in low precision, reductions / losses / norms in fp32) is
//    libtorch's own table, which matches the reference's categories.
#pragma once
#include <torch/torch.h>
#include <ATen/autocast_mode.h>

#include <map>
#include <string>

#include "optim.h"

namespace promethorch {
namespace amp {
using Tensor = at::Tensor;

struct GradScalerOptions {
    double init_scale_v = 65536.0, growth_factor_v = 2.0, backoff_factor_v = 0.5;
    int64_t growth_interval_v = 2000;
    bool enabled_v = true;
    GradScalerOptions& init_scale(double v) { init_scale_v = v; return *this; }
    GradScalerOptions& growth_factor(double v) { growth_factor_v = v; return *this; }
    GradScalerOptions& backoff_factor(double v) { backoff_factor_v = v; return *this; }
    GradScalerOptions& growth_interval(int64_t v) { growth_interval_v = v; return *this; }
    GradScalerOptions& enabled(bool v) { enabled_v = v; return *this; }
};

class GradScaler {
 public:
    explicit GradScaler(GradScalerOptions o = {}) : o_(o), scale_(o.init_scale_v) {}
    Tensor scale(const Tensor& loss) const { return o_.enabled_v ? loss * scale_ : loss; }
    // Divide every gradient by the scale and look for inf / nan.  Once per optimizer step.
    void unscale(optim::Optimizer& opt) {
        if (!o_.enabled_v || unscaled_) return;
        torch::NoGradGuard ng;
        found_inf_ = false;
        const double inv = 1.0 / scale_;
        for (auto& g : opt.param_groups())
            for (auto& p : g.params) {
                if (!p.grad().defined()) continue;
                Tensor gr = p.mutable_grad();
                gr.mul_(inv);
                if (!torch::isfinite(gr).all().item<bool>()) found_inf_ = true;
            }
        unscaled_ = true;
    }
    // Steps unless a gradient was inf / nan; returns whether the step was taken.
    bool step(optim::Optimizer& opt) {
        if (!o_.enabled_v) { opt.step(); return true; }
        unscale(opt);
        if (found_inf_) return false;
        opt.step();
        return true;
    }
    void update() {
        if (!o_.enabled_v) return;
        if (found_inf_) {
            scale_ *= o_.backoff_factor_v;
            growth_tracker_ = 0;
        } else if (++growth_tracker_ >= o_.growth_interval_v) {
            scale_ *= o_.growth_factor_v;
            growth_tracker_ = 0;
        }
        unscaled_ = false;
        found_inf_ = false;
    }
    double get_scale() const { return scale_; }
    bool found_inf() const { return found_inf_; }
    bool is_enabled() const { return o_.enabled_v; }
    std::map<std::string, double> state_dict() const {
        return {{"scale", scale_}, {"growth_factor", o_.growth_factor_v}, {"backoff_factor", o_.backoff_factor_v},
                {"growth_interval", (double)o_.growth_interval_v}, {"growth_tracker", (double)growth_tracker_}};
    }
    void load_state_dict(const std::map<std::string, double>& s) {
        auto get = [&](const char* k, double d) { auto it = s.find(k); return it == s.end() ? d : it->second; };
        scale_ = get("scale", scale_);
        o_.growth_factor_v = get("growth_factor", o_.growth_factor_v);
        o_.backoff_factor_v = get("backoff_factor", o_.backoff_factor_v);
        o_.growth_interval_v = (int64_t)get("growth_interval", (double)o_.growth_interval_v);
        growth_tracker_ = (int64_t)get("growth_tracker", 0);
    }

 private:
    GradScalerOptions o_;
    double scale_;
    int64_t growth_tracker_ = 0;
    bool found_inf_ = false, unscaled_ = false;
};

// Autocast for the lifetime of the guard; restores the previous setting.
// The four autocast categories and the op-name table behind them (torch/amp/autocast_policy.h:30-170 of the reference).
enum class CastPolicy { LowerPrecision, FP32, Promote, Unchanged };
inline const std::map<std::string, CastPolicy>& autocast_policy_table() {
    static const std::map<std::string, CastPolicy> table = [] {
        std::map<std::string, CastPolicy> t;
        for (const char* n : {"linear", "matmul", "mm", "bmm", "addmm", "addbmm", "baddbmm", "addmv", "mv", "conv1d", "conv2d", "conv3d",
                              "conv_transpose1d", "conv_transpose2d", "conv_transpose3d", "scaled_dot_product_attention", "flash_attention",
                              "prelu", "gru", "lstm", "rnn", "gru_cell", "lstm_cell", "rnn_tanh_cell", "rnn_relu_cell"})
            t[n] = CastPolicy::LowerPrecision;
        for (const char* n : {"softmax", "log_softmax", "layer_norm", "batch_norm", "group_norm", "instance_norm", "cross_entropy", "nll_loss",
                              "mse_loss", "l1_loss", "smooth_l1_loss", "huber_loss", "binary_cross_entropy", "binary_cross_entropy_with_logits",
                              "kl_div", "poisson_nll_loss", "exp", "exp2", "expm1", "log", "log2", "log10", "log1p", "pow", "reciprocal",
                              "rsqrt", "gelu", "tanh", "sum", "mean", "prod", "cumsum", "cumprod", "norm"})
            t[n] = CastPolicy::FP32;
        for (const char* n : {"add", "sub", "mul", "div", "cat", "stack", "addcmul", "addcdiv", "where", "bilinear", "dot"}) t[n] = CastPolicy::Promote;
        return t;
    }();
    return table;
}
// Ops that are not in the table keep their inputs' dtype.
inline CastPolicy get_autocast_policy(const std::string& op) {
    auto it = autocast_policy_table().find(op);
    return it == autocast_policy_table().end() ? CastPolicy::Unchanged : it->second;
}
inline bool is_autocast_enabled(c10::DeviceType device = c10::kCUDA) { return at::autocast::is_autocast_enabled(device); }
inline c10::ScalarType get_autocast_dtype(c10::DeviceType device = c10::kCUDA) { return at::autocast::get_autocast_dtype(device); }

class AutocastGuard {
 public:
    AutocastGuard(c10::DeviceType device, c10::ScalarType dtype, bool enabled = true) : device_(device) {
        prev_enabled_ = at::autocast::is_autocast_enabled(device);
        prev_dtype_ = at::autocast::get_autocast_dtype(device);
        at::autocast::set_autocast_enabled(device, enabled);
        at::autocast::set_autocast_dtype(device, dtype);
        at::autocast::increment_nesting();
    }
    ~AutocastGuard() {
        if (at::autocast::decrement_nesting() == 0) at::autocast::clear_cache();
        at::autocast::set_autocast_enabled(device_, prev_enabled_);
        at::autocast::set_autocast_dtype(device_, prev_dtype_);
    }
    AutocastGuard(const AutocastGuard&) = delete;
    AutocastGuard& operator=(const AutocastGuard&) = delete;

 private:
    c10::DeviceType device_;
    bool prev_enabled_;
    c10::ScalarType prev_dtype_;
};
struct AutocastCPUGuard : AutocastGuard {
    explicit AutocastCPUGuard(c10::ScalarType dtype = c10::kBFloat16, bool enabled = true) : AutocastGuard(c10::kCPU, dtype, enabled) {}
};

}  // namespace amp
}  // namespace promethorch
