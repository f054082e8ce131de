// promethorch C++ API: activation checkpointing.
//
// checkpoint(fn, inputs) runs fn without recording the graph and keeps only the inputs; backward runs fn again with
// recording on and back-propagates through that second run, so the activations inside fn live only during its own
// backward.  checkpoint_sequential cuts a list of stages into segments and checkpoints all but the last
// (torch/utils/checkpoint.h:24-200 of the reference).  Parameters used inside fn receive their gradients during the
// re-run (they are leaves of the re-recorded graph).
#pragma once
#include <torch/torch.h>

#include <functional>
#include <memory>
#include <vector>

namespace promethorch {
namespace utils {
using Tensor = at::Tensor;
using CheckpointFn = std::function<Tensor(const std::vector<Tensor>&)>;

namespace detail {
struct FnHolder : public torch::CustomClassHolder {
    explicit FnHolder(std::shared_ptr<CheckpointFn> f) : fn(std::move(f)) {}
    std::shared_ptr<CheckpointFn> fn;
};
struct CheckpointFunction : public torch::autograd::Function<CheckpointFunction> {
    static Tensor forward(torch::autograd::AutogradContext* ctx, std::shared_ptr<CheckpointFn> fn, at::TensorList inputs) {
        ctx->saved_data["fn"] = c10::IValue::make_capsule(c10::make_intrusive<FnHolder>(fn));      // freed with the graph node
        ctx->save_for_backward(inputs.vec());
        std::vector<Tensor> detached;
        for (auto& t : inputs) detached.push_back(t.detach());
        torch::NoGradGuard ng;
        return (*fn)(detached);
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grads) {
        std::shared_ptr<CheckpointFn> fn = static_cast<FnHolder*>(ctx->saved_data["fn"].toCapsule().get())->fn;
        auto saved = ctx->get_saved_variables();
        std::vector<Tensor> again;
        for (auto& t : saved) again.push_back(t.detach().set_requires_grad(t.requires_grad()));
        Tensor out;
        {
            torch::AutoGradMode on(true);
            out = (*fn)(again);
        }
        // a full backward pass through the re-run: the inputs' gradients come back here, the parameters' accumulate in place
        torch::autograd::backward({out}, {grads[0]});
        torch::autograd::variable_list res;
        res.push_back(Tensor());                     // the function object
        for (auto& t : again) res.push_back(t.requires_grad() ? t.grad() : Tensor());
        return res;
    }
};
}  // namespace detail

inline Tensor checkpoint(CheckpointFn fn, const std::vector<Tensor>& inputs) {
    return detail::CheckpointFunction::apply(std::make_shared<CheckpointFn>(std::move(fn)), at::TensorList(inputs));
}
// Single-input form.
inline Tensor checkpoint(std::function<Tensor(const Tensor&)> fn, const Tensor& x) {
    return checkpoint([fn](const std::vector<Tensor>& in) { return fn(in[0]); }, std::vector<Tensor>{x});
}
// `stages` cut into `segments` runs; every run but the last is checkpointed.
inline Tensor checkpoint_sequential(const std::vector<std::function<Tensor(const Tensor&)>>& stages, int segments, const Tensor& x) {
    const int n = (int)stages.size();
    TORCH_CHECK(segments >= 1 && n >= 1, "checkpoint_sequential: needs stages and at least one segment");
    const int per = (n + segments - 1) / segments;
    Tensor h = x;
    for (int s = 0; s < n; s += per) {
        const int e = std::min(n, s + per);
        auto run = [&stages, s, e](const Tensor& in) {
            Tensor t = in;
            for (int k = s; k < e; ++k) t = stages[k](t);
            return t;
        };
        if (e < n) h = checkpoint(std::function<Tensor(const Tensor&)>(run), h);
        else h = run(h);
    }
    return h;
}

}  // namespace utils
}  // namespace promethorch
