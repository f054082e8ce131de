// promethorch C++ API: a small training loop.
//
// LightningModule {training_step, validation_step, configure_optimizer, on_train_epoch_start / on_train_epoch_end /
// on_validation_end}, TrainerConfig {max_epochs, log_every_n_steps, val_check_interval, checkpoint_dir,
// save_every_n_epochs, enable_progress_bar, gradient_clip_val, accumulate_grad_batches} and
// Trainer::{fit, test, save_checkpoint, load_checkpoint}: gradient accumulation, L2 gradient clipping, validation per
// epoch or every N steps, a PTOR checkpoint `epoch_N.ptor` per epoch with the optimizer state and the position beside it
// so that fit() can resume (torch/trainer/trainer.h:48-340 of the reference).
#pragma once
#include <torch/torch.h>
#include <sys/stat.h>

#include <cstdio>
#include <memory>
#include <string>
#include <vector>

#include "data.h"
#include "optim.h"
#include "serialization.h"

namespace promethorch {
namespace trainer {
using Tensor = at::Tensor;

class LightningModule : public torch::nn::Module {
 public:
    // The loss of one training batch (the trainer calls backward on it).  Override either form.
    virtual Tensor training_step(const Tensor& batch, int batch_idx) {
        (void)batch; (void)batch_idx;
        TORCH_CHECK(false, "LightningModule: override training_step");
    }
    virtual Tensor training_step(const data::Batch& batch, int batch_idx) { return training_step(batch.data, batch_idx); }
    // A per-batch validation metric; an undefined tensor means "nothing to report".
    virtual Tensor validation_step(const Tensor& batch, int batch_idx) { (void)batch; (void)batch_idx; return Tensor(); }
    virtual Tensor validation_step(const data::Batch& batch, int batch_idx) { return validation_step(batch.data, batch_idx); }
    virtual std::shared_ptr<optim::Optimizer> configure_optimizer() = 0;
    virtual void on_train_epoch_start(int /*epoch*/) {}
    virtual void on_train_epoch_end(int /*epoch*/, double /*avg_loss*/) {}
    virtual void on_validation_end(int /*epoch*/, double /*avg_val_loss*/) {}
};

struct TrainerConfig {
    int max_epochs = 10;
    int log_every_n_steps = 50;
    int val_check_interval = 0;          // 0: once per epoch
    std::string checkpoint_dir = "./checkpoints";
    int save_every_n_epochs = 1;         // 0: never
    bool enable_progress_bar = true;
    double gradient_clip_val = 0.0;      // 0: no clipping (L2 norm otherwise)
    int accumulate_grad_batches = 1;
};

class Trainer {
 public:
    explicit Trainer(TrainerConfig cfg = {}) : cfg_(std::move(cfg)) {}

    template <typename TrainLoader, typename ValLoader = TrainLoader>
    void fit(LightningModule& module, TrainLoader& train_loader, ValLoader* val_loader = nullptr) {
        if (!opt_) opt_ = module.configure_optimizer();
        const int accum = std::max(1, cfg_.accumulate_grad_batches);
        for (int epoch = start_epoch_; epoch < cfg_.max_epochs; ++epoch) {
            module.train();
            module.on_train_epoch_start(epoch);
            double sum = 0;
            int n = 0, batch_idx = 0;
            opt_->zero_grad();
            for (auto& batch : train_loader) {
                Tensor loss = module.training_step(batch, batch_idx);
                (loss / (double)accum).backward();
                sum += loss.template item<double>();
                ++n;
                ++batch_idx;
                if (batch_idx % accum == 0) optimizer_step(module);
                if (cfg_.enable_progress_bar && cfg_.log_every_n_steps > 0 && batch_idx % cfg_.log_every_n_steps == 0)
                    std::printf("epoch %d step %d loss %.4f\n", epoch + 1, batch_idx, sum / n);
                if (val_loader && cfg_.val_check_interval > 0 && batch_idx % cfg_.val_check_interval == 0) run_validation(module, *val_loader, epoch);
            }
            if (batch_idx % accum != 0) optimizer_step(module);            // the last, shorter accumulation window
            last_train_loss_ = n ? sum / n : 0.0;
            train_history_.push_back(last_train_loss_);
            module.on_train_epoch_end(epoch, last_train_loss_);
            if (val_loader && cfg_.val_check_interval == 0) run_validation(module, *val_loader, epoch);
            if (cfg_.save_every_n_epochs > 0 && (epoch + 1) % cfg_.save_every_n_epochs == 0) {
                ::mkdir(cfg_.checkpoint_dir.c_str(), 0777);
                start_epoch_ = epoch + 1;
                save_checkpoint(module, cfg_.checkpoint_dir + "/epoch_" + std::to_string(epoch + 1) + ".ptor");
            }
        }
        start_epoch_ = cfg_.max_epochs;
    }
    template <typename TestLoader>
    double test(LightningModule& module, TestLoader& loader) {
        torch::NoGradGuard ng;
        module.eval();
        double sum = 0;
        int n = 0, idx = 0;
        for (auto& batch : loader) {
            Tensor m = module.validation_step(batch, idx++);
            if (m.defined()) { sum += m.template item<double>(); ++n; }
        }
        return n ? sum / n : 0.0;
    }
    // Model weights as a PTOR container at `path`; optimizer state, the optimizer step count and the next epoch in
    // `path + ".state"` (also PTOR).
    void save_checkpoint(LightningModule& module, const std::string& path) {
        save(module, path);
        OrderedStateDict extra;
        if (opt_)
            for (auto& kv : opt_->state_dict()) extra.emplace_back("optimizer." + kv.first, kv.second);
        extra.emplace_back("trainer.next_epoch", torch::tensor((int64_t)start_epoch_));
        extra.emplace_back("trainer.global_step", torch::tensor((int64_t)global_step_));
        save_state_dict(extra, path + ".state");
    }
    bool load_checkpoint(LightningModule& module, const std::string& path) {
        try {
            load(module, path);
            if (!opt_) opt_ = module.configure_optimizer();
            optim::StateDict st;
            for (auto& kv : load_state_dict(path + ".state")) {
                if (kv.first.rfind("optimizer.", 0) == 0) st[kv.first.substr(10)] = kv.second;
                else if (kv.first == "trainer.next_epoch") start_epoch_ = (int)kv.second.item<int64_t>();
                else if (kv.first == "trainer.global_step") global_step_ = kv.second.item<int64_t>();
            }
            opt_->load_state_dict(st);
            return true;
        } catch (const std::exception& e) {
            std::fprintf(stderr, "load_checkpoint(%s) failed: %s\n", path.c_str(), e.what());
            return false;
        }
    }
    double last_train_loss() const { return last_train_loss_; }
    double last_val_metric() const { return last_val_; }
    const std::vector<double>& train_history() const { return train_history_; }
    int64_t global_step() const { return global_step_; }
    int next_epoch() const { return start_epoch_; }
    std::shared_ptr<optim::Optimizer> optimizer() const { return opt_; }

 private:
    void optimizer_step(LightningModule& module) {
        if (cfg_.gradient_clip_val > 0) torch::nn::utils::clip_grad_norm_(module.parameters(), cfg_.gradient_clip_val);
        opt_->step();
        opt_->zero_grad();
        ++global_step_;
    }
    template <typename ValLoader>
    void run_validation(LightningModule& module, ValLoader& loader, int epoch) {
        last_val_ = test(module, loader);
        module.train();
        module.on_validation_end(epoch, last_val_);
    }
    TrainerConfig cfg_;
    std::shared_ptr<optim::Optimizer> opt_;
    int start_epoch_ = 0;
    int64_t global_step_ = 0;
    double last_train_loss_ = 0, last_val_ = 0;
    std::vector<double> train_history_;
};

}  // namespace trainer
}  // namespace promethorch
