// promethorch C++ API, umbrella header.
//
// A torch-style C++ surface over libtorch (tensors, autograd, nn modules are libtorch's) plus what the reference adds
// on top: its sixteen optimizers and sixteen learning-rate schedulers with their option structs and parameter groups,
// the distributed API (process group, DistributedDataParallel with no_sync, tensor-parallel linear layers, launcher,
// DistributedSampler, sharded data parallelism with ZeRO / offload optimizers, GPipe and 1F1B pipelines), GradScaler and
// autocast guards, datasets and a prefetching DataLoader, the PTOR checkpoint container and PyTorch-compatible
// checkpoints, and (gguf.h, separate because
// it needs the CUDA runtime and libptb200 instead of libtorch) GGUF models on the native decode engine.
//
// Code written against the reference's headers keeps its spelling with the namespace swapped:
//     namespace pt = promethorch;
//     pt::optim::Adam opt(model->parameters(), pt::optim::AdamOptions(1e-3).betas(0.9, 0.95));
//     pt::optim::WarmupCosineAnnealingLR sched(opt, 100, 10000);
//     pt::distributed::init_process_group(cfg);  pt::distributed::DistributedDataParallel<Net> ddp(net);
// Everything of libtorch is reachable through the same prefix (pt::randn, pt::nn::Linear, ...).
#pragma once
#include <torch/torch.h>

#include "amp.h"
#include "checkpoint.h"
#include "data.h"
#include "distributed.h"
#include "ecosystem.h"
#include "export.h"
#include "fsdp.h"
#include "hooks.h"
#include "lr_scheduler.h"
#include "models.h"
#include "nn_extra.h"
#include "optim.h"
#include "pipeline.h"
#include "quantization.h"
#include "serialization.h"
#include "sync_batchnorm.h"
#include "trainer.h"

namespace promethorch {

using namespace ::torch;        // tensors, factories, autograd, data: libtorch's, under the same prefix

namespace nn {
using namespace ::torch::nn;    // the module system and the standard modules

// y = x / sqrt(mean(x^2) + eps) * weight over the last dimension (optionally (1 + weight), as the Gemma family does).
class RMSNormImpl : public torch::nn::Module {
 public:
    explicit RMSNormImpl(int64_t dim, double eps = 1e-6, bool add_one = false) : eps_(eps), add_one_(add_one) {
        weight = register_parameter("weight", add_one ? torch::zeros({dim}) : torch::ones({dim}));
    }
    Tensor forward(const Tensor& x) {
        const Tensor v = x.to(torch::kFloat);
        const Tensor n = v * torch::rsqrt(v.pow(2).mean(-1, true) + eps_);
        return (n * (add_one_ ? weight + 1 : weight)).to(x.dtype());
    }
    Tensor weight;

 private:
    double eps_;
    bool add_one_;
};
TORCH_MODULE(RMSNorm);

// y = (x U^T) V^T + b with U[rank, in], V[out, rank]: a linear layer of rank `rank` (torch/nn/modules/linear.h).
class LowRankLinearImpl : public torch::nn::Module {
 public:
    LowRankLinearImpl(int64_t in, int64_t out, int64_t rank, bool bias = true) {
        U = register_module("U", torch::nn::Linear(torch::nn::LinearOptions(in, rank).bias(false)));
        V = register_module("V", torch::nn::Linear(torch::nn::LinearOptions(rank, out).bias(bias)));
    }
    Tensor forward(const Tensor& x) { return V(U(x)); }
    torch::nn::Linear U{nullptr}, V{nullptr};
};
TORCH_MODULE(LowRankLinear);

}  // namespace nn
}  // namespace promethorch
