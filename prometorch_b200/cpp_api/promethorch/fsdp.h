// promethorch C++ API: sharded data parallelism.
//
// FullyShardedDataParallel keeps 1/world of every parameter (a flat, zero-padded shard per parameter) as the trainable
// state; the full parameters exist only between all_gather_params() and reshard_params().  reduce_scatter_grads()
// averages the gradients over the ranks and leaves each rank the slice that belongs to its shards.  An optimizer built
// over shards() therefore holds 1/world of the optimizer state (ZeRO); ZeROOptimizer wires the three calls around any
// optimizer, OffloadOptimizer keeps master weights and optimizer state in host memory for parameters that live on a
// device.  Surface of the reference's torch/distributed/fsdp.h:40-434 (FSDPConfig, all_gather_params, reshard_params /
// drop_full_param, reduce_scatter_grads) and ZeROOptimizer / ZeROStage3 / deepspeed::OffloadOptimizer; the reference
// moves the shards through files, this goes through the process group.
#pragma once
#include <torch/torch.h>

#include <memory>
#include <vector>

#include "distributed.h"
#include "optim.h"

namespace promethorch {
namespace distributed {

struct FSDPConfig {
    ProcessGroupPtr group;               // null: the default group (or a single-rank group)
    bool drop_full_param = true;         // reshard_params() releases the gathered storage
    bool broadcast_parameters = true;    // rank 0's initial values everywhere
    FSDPConfig& process_group(ProcessGroupPtr g) { group = std::move(g); return *this; }
    FSDPConfig& drop_full_param_(bool v) { drop_full_param = v; return *this; }
};
using ZeROStage3Config = FSDPConfig;

template <typename ModuleHolder>
class FullyShardedDataParallel {
 public:
    explicit FullyShardedDataParallel(ModuleHolder module, FSDPConfig cfg = {})
        : module_(std::move(module)), cfg_(cfg),
          pg_(cfg.group ? cfg.group : (default_group() ? default_group() : ProcessGroupPtr(new SingleProcessGroup()))) {
        torch::NoGradGuard ng;
        const int W = pg_->world_size(), r = pg_->rank();
        for (auto& p : module_->parameters()) {
            if (cfg_.broadcast_parameters && W > 1) pg_->broadcast(p, 0);
            Item it;
            it.param = p;
            it.shape = p.sizes().vec();
            it.numel = p.numel();
            it.per = (it.numel + W - 1) / W;
            Tensor flat = torch::zeros({it.per * W}, p.options());
            flat.narrow(0, 0, it.numel).copy_(p.detach().reshape(-1));
            it.shard = flat.narrow(0, (int64_t)r * it.per, it.per).clone().set_requires_grad(true);
            items_.push_back(std::move(it));
        }
        gathered_ = true;          // the module still holds its full parameters
    }
    // Full parameters from everybody's shards (before forward / backward).
    void all_gather_params() {
        torch::NoGradGuard ng;
        for (auto& it : items_) {
            std::vector<Tensor> parts = pg_->all_gather(it.shard.detach());
            Tensor full = torch::cat(parts).narrow(0, 0, it.numel).reshape(it.shape).to(it.shard.device());
            if (it.param.numel() != it.numel) it.param.set_data(full);
            else it.param.copy_(full);
        }
        gathered_ = true;
    }
    // Back to shards: the full parameters are released (drop_full_param) until the next gather.
    void reshard_params() {
        if (!cfg_.drop_full_param) return;
        torch::NoGradGuard ng;
        for (auto& it : items_) it.param.set_data(torch::empty({0}, it.param.options()));
        gathered_ = false;
    }
    template <typename... Args>
    auto forward(Args&&... args) {
        if (!gathered_) all_gather_params();
        return module_->forward(std::forward<Args>(args)...);
    }
    template <typename... Args>
    auto operator()(Args&&... args) { return forward(std::forward<Args>(args)...); }
    // Average of the gradients over the ranks, each rank keeping the slice of its shards (in shard.grad()); the full
    // gradients are released.
    void reduce_scatter_grads() {
        torch::NoGradGuard ng;
        const int W = pg_->world_size(), r = pg_->rank();
        for (auto& it : items_) {
            if (!it.param.grad().defined()) continue;
            Tensor flat = torch::zeros({it.per * W}, it.shard.options());
            flat.narrow(0, 0, it.numel).copy_(it.param.grad().reshape(-1));
            if (W > 1) pg_->all_reduce(flat, ReduceOp::AVG);
            Tensor mine = flat.narrow(0, (int64_t)r * it.per, it.per).clone();
            if (it.shard.grad().defined()) it.shard.mutable_grad().add_(mine);
            else it.shard.mutable_grad() = mine;
            it.param.mutable_grad().reset();
        }
    }
    // The trainable state: one flat shard per parameter (hand these to the optimizer).
    std::vector<Tensor> shards() const {
        std::vector<Tensor> v;
        for (auto& it : items_) v.push_back(it.shard);
        return v;
    }
    int64_t sharded_numel() const {
        int64_t n = 0;
        for (auto& it : items_) n += it.per;
        return n;
    }
    int64_t full_numel() const {
        int64_t n = 0;
        for (auto& it : items_) n += it.numel;
        return n;
    }
    bool params_gathered() const { return gathered_; }
    ModuleHolder& module() { return module_; }
    ProcessGroupPtr process_group() const { return pg_; }
    int rank() const { return pg_->rank(); }
    int world_size() const { return pg_->world_size(); }

 private:
    struct Item {
        Tensor param, shard;
        std::vector<int64_t> shape;
        int64_t numel = 0, per = 0;
    };
    ModuleHolder module_;
    FSDPConfig cfg_;
    ProcessGroupPtr pg_;
    std::vector<Item> items_;
    bool gathered_ = false;
};
template <typename ModuleHolder>
using ZeROStage3 = FullyShardedDataParallel<ModuleHolder>;

// An optimizer over the shards of a FullyShardedDataParallel model: step() = reduce-scatter the gradients, update the
// local shards (so moments exist for 1/world of the model only), gather the new parameters.
template <typename ModuleHolder, typename Opt>
class ZeROOptimizer {
 public:
    template <typename Options>
    ZeROOptimizer(FullyShardedDataParallel<ModuleHolder>& model, Options options) : model_(model), opt_(model.shards(), options) {}
    void step() {
        model_.reduce_scatter_grads();
        opt_.step();
        model_.all_gather_params();
    }
    void zero_grad() {
        opt_.zero_grad(true);
        for (auto& p : model_.module()->parameters())
            if (p.grad().defined()) p.mutable_grad().reset();
    }
    Opt& optimizer() { return opt_; }

 private:
    FullyShardedDataParallel<ModuleHolder>& model_;
    Opt opt_;
};

}  // namespace distributed

namespace deepspeed {
using Tensor = at::Tensor;
// Master weights (fp32) and the optimizer state live in host memory; step() brings the gradients over, updates on the
// host and copies the new values back to the parameters' device and dtype.
template <typename Opt>
class OffloadOptimizer {
 public:
    template <typename Options>
    OffloadOptimizer(std::vector<Tensor> params, Options options) : params_(std::move(params)), opt_(make_masters(params_), options) {}
    void step() {
        torch::NoGradGuard ng;
        for (size_t i = 0; i < params_.size(); ++i) {
            if (!params_[i].grad().defined()) continue;
            masters_[i].mutable_grad() = params_[i].grad().detach().to(torch::kCPU, torch::kFloat);
        }
        opt_.step();
        for (size_t i = 0; i < params_.size(); ++i) params_[i].copy_(masters_[i].to(params_[i].device(), params_[i].scalar_type()));
    }
    void zero_grad() {
        opt_.zero_grad(true);
        for (auto& p : params_)
            if (p.grad().defined()) p.mutable_grad().reset();
    }
    const std::vector<Tensor>& master_params() const { return masters_; }
    Opt& optimizer() { return opt_; }

 private:
    std::vector<Tensor>& make_masters(const std::vector<Tensor>& ps) {
        for (auto& p : ps) masters_.push_back(p.detach().to(torch::kCPU, torch::kFloat).clone().set_requires_grad(true));
        return masters_;
    }
    std::vector<Tensor> params_;
    std::vector<Tensor> masters_;      // declared before opt_: built first
    Opt opt_;
};
}  // namespace deepspeed
}  // namespace promethorch
