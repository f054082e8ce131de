// promethorch C++ API: module hooks.
//
// libtorch's C++ modules have no hook registry; the reference's nn::Module has one (torch/nn/module.h:546-590:
// register_forward_pre_hook / register_forward_hook / register_forward_hook_with_return / register_backward_hook /
// remove_hook).  `Hooked<Holder>` wraps any module holder (pt::nn::Linear, a TORCH_MODULE of your own) and runs the
// hooks around its forward:
//     pt::nn::Hooked<pt::nn::Linear> lin(pt::nn::Linear(4, 3));
//     int id = lin.register_forward_hook([](auto& m, auto& in, const pt::Tensor& out) { ... });
//     auto y = lin(x);  lin.remove_hook(id);
// A backward hook fires once per call when the gradients of all inputs that require one have arrived (or, when none
// does, when the output's gradient arrives), with (module, grad_inputs, grad_output).
#pragma once
#include <torch/torch.h>

#include <functional>
#include <map>
#include <memory>
#include <vector>

namespace promethorch {
namespace nn {

template <class Holder>
class Hooked {
 public:
    using Tensor = at::Tensor;
    using Module = torch::nn::Module;
    using PreHook = std::function<void(Module&, std::vector<Tensor>&)>;                      // may replace the inputs
    using ForwardHook = std::function<void(Module&, const std::vector<Tensor>&, const Tensor&)>;
    using ForwardHookWithReturn = std::function<Tensor(Module&, const std::vector<Tensor>&, const Tensor&)>;
    using BackwardHook = std::function<void(Module&, const std::vector<Tensor>&, const Tensor&)>;

    explicit Hooked(Holder m) : s_(std::make_shared<State>(std::move(m))) {}
    Holder& module() { return s_->m; }
    auto operator->() { return s_->m.operator->(); }

    int register_forward_pre_hook(PreHook h) { s_->pre[s_->next] = std::move(h); return s_->next++; }
    int register_forward_hook(ForwardHook h) {
        s_->fwd[s_->next] = [h](Module& m, const std::vector<Tensor>& in, const Tensor& out) { h(m, in, out); return Tensor(); };
        return s_->next++;
    }
    // The hook's result, when defined, replaces the output.
    int register_forward_hook_with_return(ForwardHookWithReturn h) { s_->fwd[s_->next] = std::move(h); return s_->next++; }
    int register_backward_hook(BackwardHook h) { s_->bwd[s_->next] = std::move(h); return s_->next++; }
    bool remove_hook(int id) { return s_->pre.erase(id) + s_->fwd.erase(id) + s_->bwd.erase(id) > 0; }
    size_t num_hooks() const { return s_->pre.size() + s_->fwd.size() + s_->bwd.size(); }

    template <class... Args>
    Tensor operator()(Args&&... args) {
        std::vector<Tensor> inputs{Tensor(std::forward<Args>(args))...};
        for (auto& kv : s_->pre) kv.second(*s_->m.ptr(), inputs);
        std::shared_ptr<CallState> st;
        if (!s_->bwd.empty() && torch::GradMode::is_enabled()) st = watch_inputs(inputs);
        Tensor out = call(inputs, std::make_index_sequence<sizeof...(Args)>());
        for (auto& kv : s_->fwd) {
            Tensor r = kv.second(*s_->m.ptr(), inputs, out);
            if (r.defined()) out = r;
        }
        if (st && out.requires_grad()) out = watch_output(out, st);
        return out;
    }

 private:
    template <size_t... I>
    Tensor call(std::vector<Tensor>& in, std::index_sequence<I...>) { return s_->m->forward(in[I]...); }

    // The module and its hooks live in shared state: the gradient hooks of a call keep it alive, so a backward pass that runs
    // after the wrapper went out of scope still finds its hooks.
    struct State {
        explicit State(Holder h) : m(std::move(h)) {}
        Holder m;
        std::map<int, PreHook> pre;
        std::map<int, ForwardHookWithReturn> fwd;
        std::map<int, BackwardHook> bwd;
        int next = 0;
    };
    struct CallState {
        std::vector<Tensor> grad_inputs;
        Tensor grad_output;
        int waiting = 0;
    };
    static void fire(const std::shared_ptr<State>& s, const std::shared_ptr<CallState>& st) {
        for (auto& kv : s->bwd) kv.second(*s->m.ptr(), st->grad_inputs, st->grad_output);
    }
    // Gradients are watched on views made for this call, so no hook stays on the caller's own tensors.
    std::shared_ptr<CallState> watch_inputs(std::vector<Tensor>& inputs) {
        auto st = std::make_shared<CallState>();
        st->grad_inputs.resize(inputs.size());
        auto s = s_;
        for (size_t i = 0; i < inputs.size(); ++i) {
            if (!inputs[i].defined() || !inputs[i].requires_grad()) continue;
            inputs[i] = inputs[i].view_as(inputs[i]);
            ++st->waiting;
            inputs[i].register_hook([s, st, i](const Tensor& g) {
                st->grad_inputs[i] = g;
                if (--st->waiting == 0) fire(s, st);
            });
        }
        return st;
    }
    Tensor watch_output(const Tensor& out, const std::shared_ptr<CallState>& st) {
        Tensor o = out.view_as(out);
        const bool none = st->waiting == 0;
        auto s = s_;
        o.register_hook([s, st, none](const Tensor& g) {
            st->grad_output = g;
            if (none) fire(s, st);
        });
        return o;
    }

    std::shared_ptr<State> s_;
};

}  // namespace nn
}  // namespace promethorch
