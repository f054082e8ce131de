// promethorch C++ API: the sixteen learning-rate schedulers (constructors and closed forms of
// torch/optim/lr_scheduler.h of the reference).  Host-side scalar programs: step() advances last_epoch (which starts
// at -1) and writes the learning rate of every parameter group of the optimizer.
#pragma once
#include "optim.h"

#include <algorithm>
#include <cmath>
#include <functional>
#include <memory>
#include <stdexcept>
#include <vector>

namespace promethorch {
namespace optim {

class LRScheduler {
 public:
    explicit LRScheduler(Optimizer& opt) : opt_(opt) {
        for (size_t i = 0; i < opt.param_groups().size(); ++i) base_lrs_.push_back(opt.get_lr(i));
    }
    virtual ~LRScheduler() = default;
    virtual std::vector<double> get_lr() const { return base_lrs_; }
    virtual void step(int64_t epoch = -1) {
        last_epoch_ = epoch == -1 ? last_epoch_ + 1 : epoch;
        apply(get_lr());
    }
    // Step and update one parameter group only.
    void step_group(size_t idx, int64_t epoch = -1) {
        last_epoch_ = epoch == -1 ? last_epoch_ + 1 : epoch;
        const auto lrs = get_lr();
        if (idx < lrs.size()) opt_.set_lr(lrs[idx], idx);
    }
    int64_t last_epoch() const { return last_epoch_; }
    double get_last_lr() const { return opt_.param_groups().empty() ? 0.0 : opt_.get_lr(0); }
    const std::vector<double>& base_lrs() const { return base_lrs_; }

 protected:
    void apply(const std::vector<double>& lrs) {
        for (size_t i = 0; i < lrs.size() && i < opt_.param_groups().size(); ++i) opt_.set_lr(lrs[i], i);
    }
    std::vector<double> scaled(double f) const {
        std::vector<double> out;
        for (double b : base_lrs_) out.push_back(b * f);
        return out;
    }
    Optimizer& opt_;
    std::vector<double> base_lrs_;
    int64_t last_epoch_ = -1;
};

class StepLR : public LRScheduler {
 public:
    StepLR(Optimizer& o, int64_t step_size, double gamma = 0.1) : LRScheduler(o), step_size_(step_size), gamma_(gamma) {}
    std::vector<double> get_lr() const override { return scaled(std::pow(gamma_, (double)(last_epoch_ / step_size_))); }

 private:
    int64_t step_size_;
    double gamma_;
};

class MultiStepLR : public LRScheduler {
 public:
    MultiStepLR(Optimizer& o, std::vector<int64_t> milestones, double gamma = 0.1) : LRScheduler(o), ms_(std::move(milestones)), gamma_(gamma) {
        std::sort(ms_.begin(), ms_.end());
    }
    std::vector<double> get_lr() const override {
        const auto n = std::count_if(ms_.begin(), ms_.end(), [&](int64_t m) { return last_epoch_ >= m; });
        return scaled(std::pow(gamma_, (double)n));
    }

 private:
    std::vector<int64_t> ms_;
    double gamma_;
};

class ExponentialLR : public LRScheduler {
 public:
    ExponentialLR(Optimizer& o, double gamma) : LRScheduler(o), gamma_(gamma) {}
    std::vector<double> get_lr() const override { return scaled(std::pow(gamma_, (double)last_epoch_)); }

 private:
    double gamma_;
};

class CosineAnnealingLR : public LRScheduler {
 public:
    CosineAnnealingLR(Optimizer& o, int64_t T_max, double eta_min = 0.0) : LRScheduler(o), T_(T_max), eta_(eta_min) {}
    std::vector<double> get_lr() const override {
        const double c = (1 + std::cos(M_PI * last_epoch_ / T_)) / 2;
        std::vector<double> out;
        for (double b : base_lrs_) out.push_back(eta_ + (b - eta_) * c);
        return out;
    }

 private:
    int64_t T_;
    double eta_;
};

class LinearLR : public LRScheduler {
 public:
    LinearLR(Optimizer& o, double start_factor = 1.0 / 3, double end_factor = 1.0, int64_t total_iters = 5)
        : LRScheduler(o), s_(start_factor), e_(end_factor), n_(total_iters) {}
    std::vector<double> get_lr() const override {
        return scaled(last_epoch_ >= n_ ? e_ : s_ + (double)last_epoch_ / n_ * (e_ - s_));
    }

 private:
    double s_, e_;
    int64_t n_;
};

class ConstantLR : public LRScheduler {
 public:
    ConstantLR(Optimizer& o, double factor = 1.0 / 3, int64_t total_iters = 5) : LRScheduler(o), f_(factor), n_(total_iters) {}
    std::vector<double> get_lr() const override { return scaled(last_epoch_ < n_ ? f_ : 1.0); }

 private:
    double f_;
    int64_t n_;
};

class ReduceLROnPlateau {
 public:
    enum class Mode { Min, Max };
    ReduceLROnPlateau(Optimizer& o, Mode mode = Mode::Min, double factor = 0.1, int patience = 10, double threshold = 1e-4, double min_lr = 0.0)
        : opt_(o), mode_(mode), factor_(factor), patience_(patience), threshold_(threshold), min_lr_(min_lr),
          best_(mode == Mode::Min ? INFINITY : -INFINITY) {}
    void step(double metric) {
        const bool better = mode_ == Mode::Min ? metric < best_ - threshold_ : metric > best_ + threshold_;
        if (better) { best_ = metric; bad_ = 0; return; }
        if (++bad_ > patience_) {
            for (size_t i = 0; i < opt_.param_groups().size(); ++i) opt_.set_lr(std::max(opt_.get_lr(i) * factor_, min_lr_), i);
            bad_ = 0;
        }
    }
    double get_last_lr() const { return opt_.get_lr(0); }

 private:
    Optimizer& opt_;
    Mode mode_;
    double factor_;
    int patience_;
    double threshold_, min_lr_, best_;
    int bad_ = 0;
};

// lr = base * (e + 1) / warmup during warm-up, then cosine from base to eta_min (lr_scheduler.h:359-398).
class WarmupCosineAnnealingLR : public LRScheduler {
 public:
    WarmupCosineAnnealingLR(Optimizer& o, int64_t warmup_epochs, int64_t total_epochs, double eta_min = 0.0)
        : LRScheduler(o), w_(warmup_epochs), T_(total_epochs), eta_(eta_min) {}
    std::vector<double> get_lr() const override {
        std::vector<double> out;
        if (last_epoch_ < w_) {
            for (double b : base_lrs_) out.push_back(b * (last_epoch_ + 1) / (double)w_);
            return out;
        }
        const double prog = std::min(1.0, (double)(last_epoch_ - w_) / (double)std::max<int64_t>(T_ - w_, 1));
        const double c = (1 + std::cos(M_PI * prog)) / 2;
        for (double b : base_lrs_) out.push_back(eta_ + (b - eta_) * c);
        return out;
    }

 private:
    int64_t w_, T_;
    double eta_;
};

class OneCycleLR {
 public:
    OneCycleLR(Optimizer& o, double max_lr, int64_t total_steps, double pct_start = 0.3, double div_factor = 25.0, double final_div_factor = 1e4)
        : opt_(o), max_(max_lr), total_(total_steps), pct_(pct_start), init_(max_lr / div_factor), min_(max_lr / div_factor / final_div_factor) {
        opt_.set_lr(init_);
    }
    void step() {
        ++n_;
        const int64_t warm = (int64_t)(total_ * pct_);
        double lr;
        if (n_ <= warm) lr = init_ + (double)n_ / std::max<int64_t>(warm, 1) * (max_ - init_);
        else lr = min_ + (max_ - min_) * (1 + std::cos(M_PI * (n_ - warm) / (double)std::max<int64_t>(total_ - warm, 1))) / 2;
        opt_.set_lr(lr);
    }
    double get_last_lr() const { return opt_.get_lr(0); }

 private:
    Optimizer& opt_;
    double max_;
    int64_t total_;
    double pct_, init_, min_;
    int64_t n_ = 0;
};

class CosineAnnealingWarmRestarts : public LRScheduler {
 public:
    CosineAnnealingWarmRestarts(Optimizer& o, int64_t T_0, int64_t T_mult = 1, double eta_min = 0.0)
        : LRScheduler(o), T0_(T_0), mult_(T_mult), eta_(eta_min), Ti_(T_0) {
        if (T_0 <= 0 || T_mult < 1) throw std::invalid_argument("CosineAnnealingWarmRestarts: T_0 > 0 and T_mult >= 1 required");
    }
    void step(int64_t epoch = -1) override {
        if (epoch == -1) {
            ++last_epoch_;
            if (++Tcur_ >= Ti_) { Tcur_ = 0; Ti_ *= mult_; }
        } else {
            last_epoch_ = epoch;
            int64_t rem = epoch, Ti = T0_;
            while (rem >= Ti) { rem -= Ti; Ti *= mult_; }
            Tcur_ = rem;
            Ti_ = Ti;
        }
        apply(get_lr());
    }
    std::vector<double> get_lr() const override {
        const double c = (1 + std::cos(M_PI * Tcur_ / (double)Ti_)) / 2;
        std::vector<double> out;
        for (double b : base_lrs_) out.push_back(eta_ + (b - eta_) * c);
        return out;
    }

 private:
    int64_t T0_, mult_;
    double eta_;
    int64_t Ti_, Tcur_ = 0;
};

class CyclicLR : public LRScheduler {
 public:
    enum class Mode { Triangular, Triangular2, ExpRange };
    CyclicLR(Optimizer& o, double base_lr, double max_lr, int64_t step_size_up = 2000, int64_t step_size_down = -1,
             Mode mode = Mode::Triangular, double gamma = 1.0)
        : LRScheduler(o), base_(base_lr), max_(max_lr), up_(step_size_up), down_(step_size_down < 0 ? step_size_up : step_size_down),
          mode_(mode), gamma_(gamma) {
        opt_.set_lr(base_lr);
        for (auto& b : base_lrs_) b = base_lr;
    }
    std::vector<double> get_lr() const override {
        const int64_t total = up_ + down_, cycle = last_epoch_ / total, pos = last_epoch_ - cycle * total;
        const double x = pos < up_ ? (double)pos / up_ : 1 - (double)(pos - up_) / down_;
        double scale = 1.0;
        if (mode_ == Mode::Triangular2) scale = 1.0 / std::pow(2.0, (double)cycle);
        else if (mode_ == Mode::ExpRange) scale = std::pow(gamma_, (double)last_epoch_);
        return std::vector<double>(base_lrs_.size(), base_ + (max_ - base_) * x * scale);
    }

 private:
    double base_, max_;
    int64_t up_, down_;
    Mode mode_;
    double gamma_;
};

class PolynomialLR : public LRScheduler {
 public:
    PolynomialLR(Optimizer& o, int64_t total_iters, double power = 1.0) : LRScheduler(o), n_(total_iters), p_(power) {}
    std::vector<double> get_lr() const override {
        return scaled(last_epoch_ >= n_ ? 0.0 : std::pow(1 - (double)last_epoch_ / n_, p_));
    }

 private:
    int64_t n_;
    double p_;
};

using LRLambda = std::function<double(int64_t)>;

class LambdaLR : public LRScheduler {
 public:
    LambdaLR(Optimizer& o, LRLambda fn) : LRScheduler(o), fns_(base_lrs_.size(), fn) {}
    LambdaLR(Optimizer& o, std::vector<LRLambda> fns) : LRScheduler(o), fns_(std::move(fns)) {
        if (fns_.size() != base_lrs_.size()) throw std::invalid_argument("LambdaLR: one function per parameter group");
    }
    std::vector<double> get_lr() const override {
        std::vector<double> out;
        for (size_t i = 0; i < base_lrs_.size(); ++i) out.push_back(base_lrs_[i] * fns_[i](last_epoch_));
        return out;
    }

 private:
    std::vector<LRLambda> fns_;
};

class MultiplicativeLR : public LRScheduler {
 public:
    MultiplicativeLR(Optimizer& o, LRLambda fn) : LRScheduler(o), fns_(base_lrs_.size(), fn) {}
    MultiplicativeLR(Optimizer& o, std::vector<LRLambda> fns) : LRScheduler(o), fns_(std::move(fns)) {
        if (fns_.size() != base_lrs_.size()) throw std::invalid_argument("MultiplicativeLR: one function per parameter group");
    }
    void step(int64_t epoch = -1) override {
        last_epoch_ = epoch == -1 ? last_epoch_ + 1 : epoch;
        if (last_epoch_ == 0) return;
        for (size_t i = 0; i < fns_.size(); ++i) opt_.set_lr(opt_.get_lr(i) * fns_[i](last_epoch_), i);
    }
    std::vector<double> get_lr() const override {
        std::vector<double> out;
        for (size_t i = 0; i < base_lrs_.size(); ++i) out.push_back(opt_.get_lr(i));
        return out;
    }

 private:
    std::vector<LRLambda> fns_;
};

// Runs scheduler i while the step count is below milestones[i] (the last one afterwards).
class SequentialLR {
 public:
    SequentialLR(Optimizer& o, std::vector<std::shared_ptr<LRScheduler>> schedulers, std::vector<int64_t> milestones)
        : opt_(o), s_(std::move(schedulers)), ms_(std::move(milestones)) {
        if (s_.empty() || ms_.size() + 1 != s_.size() || !std::is_sorted(ms_.begin(), ms_.end()))
            throw std::invalid_argument("SequentialLR: n schedulers need n - 1 increasing milestones");
    }
    void step() {
        ++n_;
        size_t active = s_.size() - 1;
        for (size_t i = 0; i < ms_.size(); ++i)
            if (n_ < ms_[i]) { active = i; break; }
        s_[active]->step();
    }
    double get_last_lr() const { return opt_.get_lr(0); }

 private:
    Optimizer& opt_;
    std::vector<std::shared_ptr<LRScheduler>> s_;
    std::vector<int64_t> ms_;
    int64_t n_ = -1;
};

// Every scheduler steps; a group's rate is its base rate times the product of each scheduler's (rate / base rate).
class ChainedScheduler {
 public:
    ChainedScheduler(Optimizer& o, std::vector<std::shared_ptr<LRScheduler>> schedulers) : opt_(o), s_(std::move(schedulers)) {
        if (s_.empty()) throw std::invalid_argument("ChainedScheduler: schedulers must not be empty");
        for (size_t i = 0; i < o.param_groups().size(); ++i) base_.push_back(o.get_lr(i));
    }
    void step() {
        std::vector<double> comb(base_.size(), 1.0);
        for (auto& s : s_) {
            s->step();
            const auto lrs = s->get_lr();
            for (size_t i = 0; i < comb.size() && i < lrs.size(); ++i) comb[i] *= lrs[i] / (s->base_lrs()[i] != 0 ? s->base_lrs()[i] : 1.0);
        }
        for (size_t i = 0; i < base_.size(); ++i) opt_.set_lr(base_[i] * comb[i], i);
    }
    double get_last_lr() const { return opt_.get_lr(0); }

 private:
    Optimizer& opt_;
    std::vector<std::shared_ptr<LRScheduler>> s_;
    std::vector<double> base_;
};

}  // namespace optim
}  // namespace promethorch
