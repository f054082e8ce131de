// promethorch C++ API: optimizers.
//
// The sixteen optimizers of the reference (torch/optim/*.h) behind the same surface: an options struct per optimizer
// with chained setters, ParamGroup with per-group overrides where NaN / -1 means "inherit from the options"
// (torch/optim/optimizer.h:45-90), state keyed by the linear parameter index and exported as "state.<i>.<key>"
// (optimizer.h:116-148).  Tensors are libtorch tensors; the update rules are tensor programs that run on whatever
// device the parameters live on (the Python package additionally routes fp32 CUDA parameters to the fused
// multi-tensor kernels of libptb200).
#pragma once
#include <torch/torch.h>

#include <cmath>
#include <functional>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace promethorch {
using Tensor = at::Tensor;

namespace optim {

constexpr double kInherit = std::numeric_limits<double>::quiet_NaN();
inline bool inherits(double v) { return std::isnan(v); }

// A set of parameters with optional overrides of the optimizer-wide options.
struct ParamGroup {
    std::vector<Tensor> params;
    double lr = kInherit, weight_decay = kInherit, beta1 = kInherit, beta2 = kInherit, eps = kInherit, momentum = kInherit;
    int amsgrad = -1;                                   // -1 inherit, 0 / 1
    ParamGroup() = default;
    explicit ParamGroup(std::vector<Tensor> p) : params(std::move(p)) {}
    ParamGroup& learning_rate(double v) { lr = v; return *this; }
    ParamGroup& weight_decay_(double v) { weight_decay = v; return *this; }
    ParamGroup& betas(double b1, double b2) { beta1 = b1; beta2 = b2; return *this; }
    ParamGroup& eps_(double v) { eps = v; return *this; }
    ParamGroup& momentum_(double v) { momentum = v; return *this; }
    ParamGroup& amsgrad_(bool v) { amsgrad = v ? 1 : 0; return *this; }
};

using StateDict = std::map<std::string, Tensor>;

class Optimizer {
 public:
    virtual ~Optimizer() = default;
    // One update from the gradients currently stored in the parameters.
    void step() {
        torch::NoGradGuard ng;
        size_t index = 0;
        for (size_t gi = 0; gi < groups_.size(); ++gi) {
            ParamGroup& g = groups_[gi];
            bool any = false;
            for (auto& p : g.params) any = any || p.grad().defined();
            if (any) ++group_steps_[gi];
            begin_group(g, group_steps_[gi]);
            for (auto& p : g.params) {
                if (p.grad().defined()) {
                    auto& st = state_[index];
                    st.step += 1;
                    update(p, p.grad(), st, g, group_steps_[gi]);
                }
                ++index;
            }
        }
    }
    // Closure form (LBFGS re-evaluates; the others evaluate once before stepping).
    virtual Tensor step(const std::function<Tensor()>& closure) {
        Tensor loss;
        {
            torch::AutoGradMode on(true);
            loss = closure();
        }
        step();
        return loss;
    }
    void zero_grad(bool set_to_none = false) {
        for (auto& g : groups_)
            for (auto& p : g.params)
                if (p.grad().defined()) {
                    if (set_to_none) p.mutable_grad().reset();
                    else p.mutable_grad().detach_().zero_();
                }
    }
    std::vector<ParamGroup>& param_groups() { return groups_; }
    void add_param_group(ParamGroup g) {
        for (size_t i = 0; i < g.params.size(); ++i) state_.emplace_back();
        groups_.push_back(std::move(g));
        group_steps_.push_back(0);
    }
    // Effective learning rate of a group (its override, else the optimizer-wide value) and a setter for schedulers.
    double get_lr(size_t group = 0) const { return inherits(groups_[group].lr) ? default_lr() : groups_[group].lr; }
    void set_lr(double lr, size_t group) { groups_[group].lr = lr; }
    void set_lr(double lr) { for (auto& g : groups_) g.lr = lr; }

    // "state.<linear parameter index>.<key>" -> tensor ("step" as a 0-dim float tensor, as the reference stores it).
    StateDict state_dict() const {
        StateDict out;
        for (size_t i = 0; i < state_.size(); ++i) {
            if (state_[i].step == 0 && state_[i].t.empty()) continue;
            out["state." + std::to_string(i) + ".step"] = torch::tensor((float)state_[i].step);
            for (auto& kv : state_[i].t) out["state." + std::to_string(i) + "." + kv.first] = kv.second;
        }
        return out;
    }
    void load_state_dict(const StateDict& sd) {
        for (auto& kv : sd) {
            const auto a = kv.first.find('.'), b = kv.first.find('.', a + 1);
            TORCH_CHECK(a != std::string::npos && b != std::string::npos, "bad optimizer state key: ", kv.first);
            const size_t i = std::stoul(kv.first.substr(a + 1, b - a - 1));
            TORCH_CHECK(i < state_.size(), "optimizer state for parameter ", i, " but only ", state_.size(), " parameters");
            const std::string key = kv.first.substr(b + 1);
            if (key == "step") state_[i].step = (int64_t)kv.second.item<float>();
            else state_[i].t[key] = kv.second.clone();
        }
        size_t index = 0;              // the bias corrections read the group counters: resume them
        for (size_t gi = 0; gi < groups_.size(); ++gi)
            for (size_t k = 0; k < groups_[gi].params.size(); ++k, ++index) group_steps_[gi] = std::max(group_steps_[gi], state_[index].step);
    }

 protected:
    struct State {
        std::map<std::string, Tensor> t;
        int64_t step = 0;
        Tensor& get(const std::string& k, const Tensor& like) {
            auto it = t.find(k);
            if (it == t.end()) it = t.emplace(k, torch::zeros_like(like)).first;
            return it->second;
        }
        bool has(const std::string& k) const { return t.count(k) != 0; }
    };
    void init_groups(std::vector<ParamGroup> groups) {
        for (auto& g : groups) add_param_group(std::move(g));
    }
    static double pick(double group_value, double dflt) { return inherits(group_value) ? dflt : group_value; }
    virtual double default_lr() const = 0;
    virtual void begin_group(ParamGroup&, int64_t /*step*/) {}
    virtual void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) = 0;

    std::vector<ParamGroup> groups_;
    std::vector<State> state_;
    std::vector<int64_t> group_steps_;
};

#define PT_OPT_FIELD(Type, name, setter, dflt) \
    Type name = dflt;                          \
    auto& setter(Type v) { name = v; return *this; }

// ------------------------------------------------------------------------------------------ SGD
struct SGDOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 0.01)
    PT_OPT_FIELD(double, momentum, momentum_, 0.0)
    PT_OPT_FIELD(double, dampening, dampening_, 0.0)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(bool, nesterov, nesterov_, false)
    SGDOptions() = default;
    SGDOptions(double l) : lr(l) {}
};
class SGD : public Optimizer {
 public:
    SGD(std::vector<Tensor> params, SGDOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }
    SGD(std::vector<ParamGroup> groups, SGDOptions o = {}) : o_(o) { init_groups(std::move(groups)); }
    SGDOptions& options() { return o_; }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay), mom = pick(g.momentum, o_.momentum);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        if (mom != 0) {
            const bool first = !st.has("momentum_buffer");
            Tensor& buf = st.get("momentum_buffer", p);
            if (first) buf.copy_(d);
            else buf.mul_(mom).add_(d, 1 - o_.dampening);
            d = o_.nesterov ? d.add(buf, mom) : buf;
        }
        p.add_(d, -lr);
    }
    SGDOptions o_;
};

// ------------------------------------------------------------------------------------------ Adam / AdamW
struct AdamOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-3)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(bool, amsgrad, amsgrad_, false)
    AdamOptions() = default;
    AdamOptions(double l) : lr(l) {}
    AdamOptions& betas(double b1, double b2) { beta1 = b1; beta2 = b2; return *this; }
};
struct AdamWOptions : AdamOptions {
    AdamWOptions() { weight_decay = 0.01; }
    AdamWOptions(double l) : AdamOptions(l) { weight_decay = 0.01; }
};
class Adam : public Optimizer {
 public:
    Adam(std::vector<Tensor> params, AdamOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }
    Adam(std::vector<ParamGroup> groups, AdamOptions o = {}) : o_(o) { init_groups(std::move(groups)); }
    AdamOptions& options() { return o_; }

 protected:
    virtual bool decoupled() const { return false; }
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay), b1 = pick(g.beta1, o_.beta1),
                     b2 = pick(g.beta2, o_.beta2), eps = pick(g.eps, o_.eps);
        const bool ams = g.amsgrad < 0 ? o_.amsgrad : g.amsgrad != 0;
        Tensor d = grad;
        if (decoupled()) p.mul_(1 - lr * wd);
        else if (wd != 0) d = grad.add(p, wd);
        Tensor& m = st.get("exp_avg", p);
        Tensor& v = st.get("exp_avg_sq", p);
        m.mul_(b1).add_(d, 1 - b1);
        v.mul_(b2).addcmul_(d, d, 1 - b2);
        const double bc1 = 1 - std::pow(b1, (double)step), bc2 = 1 - std::pow(b2, (double)step);
        Tensor vv = v;
        if (ams) {
            Tensor& mx = st.get("max_exp_avg_sq", p);
            mx.copy_(torch::maximum(mx, v));
            vv = mx;
        }
        Tensor denom = vv.sqrt().div_(std::sqrt(bc2)).add_(eps);
        p.addcdiv_(m, denom, -lr / bc1);
    }
    AdamOptions o_;
};
class AdamW : public Adam {
 public:
    AdamW(std::vector<Tensor> params, AdamWOptions o = {}) : Adam(std::move(params), o) {}
    AdamW(std::vector<ParamGroup> groups, AdamWOptions o = {}) : Adam(std::move(groups), o) {}

 protected:
    bool decoupled() const override { return true; }
};

// ------------------------------------------------------------------------------------------ RMSprop
struct RMSpropOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 0.01)
    PT_OPT_FIELD(double, alpha, alpha_, 0.99)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(double, momentum, momentum_, 0.0)
    PT_OPT_FIELD(bool, centered, centered_, false)
};
class RMSprop : public Optimizer {
 public:
    RMSprop(std::vector<Tensor> params, RMSpropOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay), mom = pick(g.momentum, o_.momentum);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        Tensor& sq = st.get("square_avg", p);
        sq.mul_(o_.alpha).addcmul_(d, d, 1 - o_.alpha);
        Tensor avg;
        if (o_.centered) {
            Tensor& ga = st.get("grad_avg", p);
            ga.mul_(o_.alpha).add_(d, 1 - o_.alpha);
            avg = (sq - ga * ga).clamp_min_(0).sqrt_().add_(o_.eps);
        } else {
            avg = sq.sqrt().add_(o_.eps);
        }
        if (mom > 0) {
            Tensor& buf = st.get("momentum_buffer", p);
            buf.mul_(mom).addcdiv_(d, avg);
            p.add_(buf, -lr);
        } else {
            p.addcdiv_(d, avg, -lr);
        }
    }
    RMSpropOptions o_;
};

// ------------------------------------------------------------------------------------------ Lion
struct LionOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-4)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.99)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    LionOptions& betas(double b1, double b2) { beta1 = b1; beta2 = b2; return *this; }
};
class Lion : public Optimizer {
 public:
    Lion(std::vector<Tensor> params, LionOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        if (wd != 0) p.mul_(1 - lr * wd);
        Tensor& m = st.get("exp_avg", p);
        p.add_(m.mul(o_.beta1).add_(grad, 1 - o_.beta1).sign_(), -lr);
        m.mul_(o_.beta2).add_(grad, 1 - o_.beta2);
    }
    LionOptions o_;
};

// ------------------------------------------------------------------------------------------ SophiaG
struct SophiaGOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-4)
    PT_OPT_FIELD(double, beta1, beta1_, 0.965)
    PT_OPT_FIELD(double, beta2, beta2_, 0.99)
    PT_OPT_FIELD(double, eps, eps_, 1e-12)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(double, rho, rho_, 0.04)
    PT_OPT_FIELD(int, hessian_update_interval, hessian_update_interval_, 10)
};
class SophiaG : public Optimizer {
 public:
    SophiaG(std::vector<Tensor> params, SophiaGOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        if (wd != 0) p.mul_(1 - lr * wd);
        Tensor& m = st.get("exp_avg", p);
        Tensor& h = st.get("hessian", p);
        m.mul_(o_.beta1).add_(grad, 1 - o_.beta1);
        h.mul_(o_.beta2).addcmul_(grad, grad, 1 - o_.beta2);
        p.add_((m / h.clamp_min(o_.eps)).clamp_(-o_.rho, o_.rho), -lr);
    }
    SophiaGOptions o_;
};
using Sophia = SophiaG;

// ------------------------------------------------------------------------------------------ LAMB
struct LAMBOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-3)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-6)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.01)
    PT_OPT_FIELD(bool, bias_correction, bias_correction_, true)
};
class LAMB : public Optimizer {
 public:
    LAMB(std::vector<Tensor> params, LAMBOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        Tensor& m = st.get("exp_avg", p);
        Tensor& v = st.get("exp_avg_sq", p);
        m.mul_(o_.beta1).add_(grad, 1 - o_.beta1);
        v.mul_(o_.beta2).addcmul_(grad, grad, 1 - o_.beta2);
        const double bc1 = o_.bias_correction ? 1 - std::pow(o_.beta1, (double)step) : 1.0;
        const double bc2 = o_.bias_correction ? 1 - std::pow(o_.beta2, (double)step) : 1.0;
        Tensor upd = (m / bc1) / ((v / bc2).sqrt_().add_(o_.eps));
        if (wd != 0) upd.add_(p, wd);
        const double wn = p.norm().item<double>(), un = upd.norm().item<double>();
        const double trust = (wn > 0 && un > 0) ? wn / un : 1.0;       // per-tensor trust ratio
        p.add_(upd, -lr * trust);
    }
    LAMBOptions o_;
};

// ------------------------------------------------------------------------------------------ Adafactor
struct AdafactorOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 0.0)              // 0: relative step size
    PT_OPT_FIELD(double, eps1, eps1_, 1e-30)
    PT_OPT_FIELD(double, eps2, eps2_, 1e-3)
    PT_OPT_FIELD(double, clip_threshold, clip_threshold_, 1.0)
    PT_OPT_FIELD(double, decay_rate, decay_rate_, -0.8)
    PT_OPT_FIELD(double, beta1, beta1_, 0.0)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(bool, scale_parameter, scale_parameter_, true)
    PT_OPT_FIELD(bool, relative_step, relative_step_, true)
    PT_OPT_FIELD(bool, warmup_init, warmup_init_, false)
};
class Adafactor : public Optimizer {
 public:
    Adafactor(std::vector<Tensor> params, AdafactorOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double t = (double)step, n = (double)std::max<int64_t>(p.numel(), 1);
        double lr_t = pick(g.lr, o_.lr);
        if (o_.relative_step || lr_t <= 0) lr_t = std::min(o_.warmup_init ? 1e-6 * t : 1e-2, 1.0 / std::sqrt(t));
        if (o_.scale_parameter) lr_t *= std::max(o_.eps2, p.norm().item<double>() / std::sqrt(n));
        const double beta2_t = 1 - std::pow(t, o_.decay_rate);
        Tensor g2 = grad * grad + o_.eps1, upd;
        if (p.dim() >= 2) {
            // factored second moment: a row and a column accumulator instead of a full tensor
            if (!st.has("exp_avg_sq_row")) {
                st.t["exp_avg_sq_row"] = torch::zeros_like(g2.mean(-1));
                st.t["exp_avg_sq_col"] = torch::zeros_like(g2.mean(-2));
            }
            Tensor& row = st.t["exp_avg_sq_row"];
            Tensor& col = st.t["exp_avg_sq_col"];
            row.mul_(beta2_t).add_(g2.mean(-1), 1 - beta2_t);
            col.mul_(beta2_t).add_(g2.mean(-2), 1 - beta2_t);
            Tensor rf = (row / row.mean(-1, true).clamp_min(o_.eps1)).unsqueeze(-1);
            upd = grad / (rf * col.unsqueeze(-2)).sqrt().clamp_min(o_.eps1);
        } else {
            Tensor& v = st.get("exp_avg_sq", p);
            v.mul_(beta2_t).add_(g2, 1 - beta2_t);
            upd = grad / v.sqrt().clamp_min(o_.eps1);
        }
        const double scale = std::max(1.0, upd.norm().item<double>() / std::sqrt(n) / o_.clip_threshold);
        if (scale > 1) upd = upd / scale;
        if (o_.beta1 > 0) {
            Tensor& m = st.get("exp_avg", p);
            m.mul_(o_.beta1).add_(upd, 1 - o_.beta1);
            upd = m;
        }
        const double wd = pick(g.weight_decay, o_.weight_decay);
        if (wd != 0) p.mul_(1 - lr_t * wd);
        p.add_(upd, -lr_t);
    }
    AdafactorOptions o_;
};

// ------------------------------------------------------------------------------------------ NAdam
struct NAdamOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 2e-3)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(double, momentum_decay, momentum_decay_, 0.004)
};
class NAdam : public Optimizer {
 public:
    NAdam(std::vector<Tensor> params, NAdamOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void begin_group(ParamGroup&, int64_t step) override {
        if (step == last_step_) return;
        last_step_ = step;
        mu_t_ = o_.beta1 * (1 - 0.5 * std::pow(0.96, step * o_.momentum_decay));
        mu_n_ = o_.beta1 * (1 - 0.5 * std::pow(0.96, (step + 1) * o_.momentum_decay));
        mu_product_ *= mu_t_;
    }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        Tensor& m = st.get("exp_avg", p);
        Tensor& v = st.get("exp_avg_sq", p);
        m.mul_(o_.beta1).add_(d, 1 - o_.beta1);
        v.mul_(o_.beta2).addcmul_(d, d, 1 - o_.beta2);
        Tensor denom = (v / (1 - std::pow(o_.beta2, (double)step))).sqrt_().add_(o_.eps);
        p.addcdiv_(d, denom, -lr * (1 - mu_t_) / (1 - mu_product_));
        p.addcdiv_(m, denom, -lr * mu_n_ / (1 - mu_product_ * mu_n_));
    }
    NAdamOptions o_;
    double mu_t_ = 0, mu_n_ = 0, mu_product_ = 1.0;
    int64_t last_step_ = 0;
};

// ------------------------------------------------------------------------------------------ RAdam
struct RAdamOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-3)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
};
class RAdam : public Optimizer {
 public:
    RAdam(std::vector<Tensor> params, RAdamOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay), b1 = o_.beta1, b2 = o_.beta2;
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        Tensor& m = st.get("exp_avg", p);
        Tensor& v = st.get("exp_avg_sq", p);
        m.mul_(b1).add_(d, 1 - b1);
        v.mul_(b2).addcmul_(d, d, 1 - b2);
        const double rho_inf = 2 / (1 - b2) - 1, b2t = std::pow(b2, (double)step);
        const double rho_t = rho_inf - 2 * step * b2t / (1 - b2t);
        Tensor mhat = m / (1 - std::pow(b1, (double)step));
        if (rho_t > 5) {
            const double rect = std::sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t));
            p.addcdiv_(mhat, (v / (1 - b2t)).sqrt_().add_(o_.eps), -lr * rect);
        } else {
            p.add_(mhat, -lr);
        }
    }
    RAdamOptions o_;
};

// ------------------------------------------------------------------------------------------ Adagrad / Adadelta / Adamax
struct AdagradOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 0.01)
    PT_OPT_FIELD(double, lr_decay, lr_decay_, 0.0)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
    PT_OPT_FIELD(double, eps, eps_, 1e-10)
    PT_OPT_FIELD(double, initial_accumulator_value, initial_accumulator_value_, 0.0)
};
class Adagrad : public Optimizer {
 public:
    Adagrad(std::vector<Tensor> params, AdagradOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        if (!st.has("sum")) st.t["sum"] = torch::full_like(p, o_.initial_accumulator_value);
        Tensor& s = st.t["sum"];
        s.addcmul_(d, d);
        p.addcdiv_(d, s.sqrt().add_(o_.eps), -lr / (1 + (step - 1) * o_.lr_decay));
    }
    AdagradOptions o_;
};
struct AdadeltaOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1.0)
    PT_OPT_FIELD(double, rho, rho_, 0.9)
    PT_OPT_FIELD(double, eps, eps_, 1e-6)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
};
class Adadelta : public Optimizer {
 public:
    Adadelta(std::vector<Tensor> params, AdadeltaOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        Tensor& sq = st.get("square_avg", p);
        Tensor& acc = st.get("acc_delta", p);
        sq.mul_(o_.rho).addcmul_(d, d, 1 - o_.rho);
        Tensor delta = (acc + o_.eps).sqrt_().div_((sq + o_.eps).sqrt_()).mul_(d);
        acc.mul_(o_.rho).addcmul_(delta, delta, 1 - o_.rho);
        p.add_(delta, -lr);
    }
    AdadeltaOptions o_;
};
struct AdamaxOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 2e-3)
    PT_OPT_FIELD(double, beta1, beta1_, 0.9)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
};
class Adamax : public Optimizer {
 public:
    Adamax(std::vector<Tensor> params, AdamaxOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        Tensor& m = st.get("exp_avg", p);
        Tensor& u = st.get("exp_inf", p);
        m.mul_(o_.beta1).add_(d, 1 - o_.beta1);
        u.copy_(torch::maximum(u * o_.beta2, d.abs() + o_.eps));
        p.addcdiv_(m, u, -lr / (1 - std::pow(o_.beta1, (double)step)));
    }
    AdamaxOptions o_;
};

// ------------------------------------------------------------------------------------------ AdamKiller
// Curvature-adaptive first-moment decay, per-layer trust ratio, gradient look-ahead and update clipping
// (torch/optim/adamkiller.h).
struct AdamKillerOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1e-3)
    PT_OPT_FIELD(double, beta1_min, beta1_min_, 0.7)
    PT_OPT_FIELD(double, beta1_max, beta1_max_, 0.95)
    PT_OPT_FIELD(double, beta2, beta2_, 0.999)
    PT_OPT_FIELD(double, eps, eps_, 1e-8)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.01)
    PT_OPT_FIELD(bool, use_adaptive_momentum, use_adaptive_momentum_, true)
    PT_OPT_FIELD(bool, use_per_layer_lr, use_per_layer_lr_, true)
    PT_OPT_FIELD(bool, use_gradient_prediction, use_gradient_prediction_, true)
    PT_OPT_FIELD(bool, use_warm_restarts, use_warm_restarts_, false)
    PT_OPT_FIELD(int, restart_period, restart_period_, 1000)
    PT_OPT_FIELD(double, max_grad_norm, max_grad_norm_, 1.0)
    PT_OPT_FIELD(double, lr_scale_min, lr_scale_min_, 0.5)
    PT_OPT_FIELD(double, lr_scale_max, lr_scale_max_, 2.0)
};
class AdamKiller : public Optimizer {
 public:
    AdamKiller(std::vector<Tensor> params, AdamKillerOptions o = {}) : o_(o) { init_groups({ParamGroup(std::move(params))}); }

 protected:
    double default_lr() const override { return o_.lr; }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t step) override {
        const double lr = pick(g.lr, o_.lr), wd = pick(g.weight_decay, o_.weight_decay);
        const double gn = grad.norm().item<double>();
        Tensor sg = grad * ((gn > o_.max_grad_norm && gn > 1e-12) ? o_.max_grad_norm / gn : 1.0);
        double beta1 = o_.beta1_max;
        const bool have_prev = st.has("prev_grad");
        if (o_.use_adaptive_momentum && have_prev) {
            const double curv = (sg - st.t["prev_grad"]).norm().item<double>() / (lr + 1e-12);
            beta1 = o_.beta1_max - std::min(curv / 100.0, 1.0) * (o_.beta1_max - o_.beta1_min);
            beta1 = std::max(o_.beta1_min, std::min(o_.beta1_max, beta1));
        }
        Tensor eff = sg.clone();
        if (o_.use_gradient_prediction) {
            Tensor& ema = st.get("grad_diff_ema", p);
            if (have_prev) {
                ema.mul_(0.5).add_(eff - st.t["prev_grad"], 0.5);
                eff.add_(ema, 0.5);
            }
        }
        st.t["prev_grad"] = sg.clone();
        Tensor& m = st.get("m", p);
        Tensor& v = st.get("v", p);
        m.mul_(beta1).add_(eff, 1 - beta1);
        v.mul_(o_.beta2).addcmul_(eff, eff, 1 - o_.beta2);
        double layer_lr = lr;
        if (o_.use_per_layer_lr) {
            const double wn = p.norm().item<double>(), en = eff.norm().item<double>();
            if (en > 1e-8 && wn > 1e-8) layer_lr = lr * std::max(o_.lr_scale_min, std::min(o_.lr_scale_max, wn / (en + wd * wn)));
        }
        const double bc1 = 1 - std::pow(beta1, (double)step), bc2 = 1 - std::pow(o_.beta2, (double)step);
        if (wd > 0) p.mul_(1 - layer_lr * wd);
        Tensor upd = (m / bc1) / ((v / bc2) + o_.eps).sqrt_() * layer_lr;
        const double un = upd.norm().item<double>();
        if (un > 2 * layer_lr && un > 1e-12) upd.mul_(2 * layer_lr / un);
        p.sub_(upd);
        if (o_.use_warm_restarts && step % o_.restart_period == 0) m.mul_(0.1);
    }
    AdamKillerOptions o_;
};

// ------------------------------------------------------------------------------------------ ASGD
struct ASGDOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 0.01)
    PT_OPT_FIELD(double, lambd, lambd_, 1e-4)
    PT_OPT_FIELD(double, alpha, alpha_, 0.75)
    PT_OPT_FIELD(double, t0, t0_, 1e6)
    PT_OPT_FIELD(double, weight_decay, weight_decay_, 0.0)
};
class ASGD : public Optimizer {
 public:
    ASGD(std::vector<Tensor> params, ASGDOptions o = {}) : o_(o), eta_(o.lr) { init_groups({ParamGroup(std::move(params))}); }
    // Copy the averaged parameters over the live ones.
    void swap_in_averaged_params() {
        torch::NoGradGuard ng;
        size_t i = 0;
        for (auto& g : groups_)
            for (auto& p : g.params) {
                if (state_[i].has("ax")) p.copy_(state_[i].t["ax"]);
                ++i;
            }
    }

 protected:
    double default_lr() const override { return o_.lr; }
    void begin_group(ParamGroup& g, int64_t step) override {
        if (step == last_step_) return;
        last_step_ = step;
        cur_eta_ = eta_;
        cur_mu_ = mu_;
        const double lr = pick(g.lr, o_.lr);
        eta_ = lr / std::pow(1 + o_.lambd * lr * step, o_.alpha);      // the schedule for the NEXT step
        mu_ = 1.0 / std::max(1.0, step - o_.t0);
    }
    void update(Tensor& p, const Tensor& grad, State& st, const ParamGroup& g, int64_t) override {
        const double wd = pick(g.weight_decay, o_.weight_decay);
        Tensor d = wd != 0 ? grad.add(p, wd) : grad;
        if (!st.has("ax")) st.t["ax"] = p.detach().clone();
        p.mul_(1 - o_.lambd * cur_eta_).add_(d, -cur_eta_);
        Tensor& ax = st.t["ax"];
        if (cur_mu_ != 1) ax.add_(p - ax, cur_mu_);
        else ax.copy_(p);
    }
    ASGDOptions o_;
    double eta_, mu_ = 1.0, cur_eta_ = 0, cur_mu_ = 1.0;
    int64_t last_step_ = 0;
};

// ------------------------------------------------------------------------------------------ LBFGS (closure-driven)
struct LBFGSOptions {
    PT_OPT_FIELD(double, lr, learning_rate, 1.0)
    PT_OPT_FIELD(int, max_iter, max_iter_, 20)
    PT_OPT_FIELD(int, max_eval, max_eval_, 25)
    PT_OPT_FIELD(double, tolerance_grad, tolerance_grad_, 1e-7)
    PT_OPT_FIELD(double, tolerance_change, tolerance_change_, 1e-9)
    PT_OPT_FIELD(int, history_size, history_size_, 100)
};
// Host-driven two-loop recursion; delegates to libtorch's implementation with the reference's defaults.
class LBFGS {
 public:
    LBFGS(std::vector<Tensor> params, LBFGSOptions o = {})
        : impl_(std::move(params), torch::optim::LBFGSOptions(o.lr).max_iter(o.max_iter).max_eval(o.max_eval).tolerance_grad(o.tolerance_grad)
                                       .tolerance_change(o.tolerance_change).history_size(o.history_size)) {}
    Tensor step(const std::function<Tensor()>& closure) { return impl_.step(closure); }
    void zero_grad() { impl_.zero_grad(); }

 private:
    torch::optim::LBFGS impl_;
};

// ------------------------------------------------------------------------------------------ EMA of parameters
// shadow = decay * shadow + (1 - decay) * w   (torch/optim/ema.h:37-122)
class EMA {
 public:
    EMA(std::vector<Tensor> params, double decay = 0.999) : params_(std::move(params)), decay_(decay) {
        TORCH_CHECK(decay >= 0.0 && decay < 1.0, "EMA decay must be in [0, 1)");
        for (auto& p : params_) shadow_.push_back(p.detach().clone());
    }
    void update() {
        torch::NoGradGuard ng;
        for (size_t i = 0; i < params_.size(); ++i) shadow_[i].mul_(decay_).add_(params_[i].detach(), 1 - decay_);
    }
    void apply_shadow() {
        torch::NoGradGuard ng;
        backup_.clear();
        for (size_t i = 0; i < params_.size(); ++i) {
            backup_.push_back(params_[i].detach().clone());
            params_[i].copy_(shadow_[i]);
        }
    }
    void restore() {
        torch::NoGradGuard ng;
        for (size_t i = 0; i < backup_.size(); ++i) params_[i].copy_(backup_[i]);
        backup_.clear();
    }
    void set_decay(double d) { decay_ = d; }
    const std::vector<Tensor>& shadow() const { return shadow_; }

 private:
    std::vector<Tensor> params_, shadow_, backup_;
    double decay_;
};

#undef PT_OPT_FIELD

}  // namespace optim

// clip_grad_norm_ / clip_grad_value_ (torch/nn/utils/clip_grad.h:29-188): returns the total norm before clipping.
inline double clip_grad_norm_(const std::vector<Tensor>& params, double max_norm, double norm_type = 2.0) {
    torch::NoGradGuard ng;
    std::vector<Tensor> norms;
    for (auto& p : params)
        if (p.grad().defined()) norms.push_back(std::isinf(norm_type) ? p.grad().abs().max() : p.grad().norm(norm_type));
    if (norms.empty()) return 0.0;
    const Tensor all = torch::stack(norms);
    const double total = std::isinf(norm_type) ? all.max().item<double>() : all.norm(norm_type).item<double>();
    const double coef = std::min(1.0, max_norm / (total + 1e-6));
    if (coef < 1.0)
        for (auto& p : params)
            if (p.grad().defined()) p.mutable_grad().mul_(coef);
    return total;
}
inline void clip_grad_value_(const std::vector<Tensor>& params, double clip_value) {
    torch::NoGradGuard ng;
    for (auto& p : params)
        if (p.grad().defined()) p.mutable_grad().clamp_(-clip_value, clip_value);
}

}  // namespace promethorch
