"""The sixteen optimizers, with the option names, defaults and update rules of
the reference (torch/optim/*.h) and state keys that round-trip through
``state_dict`` (``step, exp_avg, exp_avg_sq, max_exp_avg_sq`` for Adam,
torch/optim/adam.h:39-67).

On CUDA tensors the twelve element-wise rules run as ONE multi-tensor kernel
launch per parameter group (csrc/optim_kernels.cu); the reference instead
bounces every CUDA tensor through the host (torch/optim/adam.h:192-220).  The
same rules written with tensor ops serve CPU tensors and are the oracle the
kernel is tested against.  LAMB, Adafactor and AdamKiller need per-tensor
norms and run as tensor programs; LBFGS is host-driven by nature.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Iterable, List, Optional

import torch

from .. import _native as N

__all__ = ["Optimizer", "SGD", "Adam", "AdamW", "RMSprop", "Lion", "SophiaG", "Sophia", "LAMB", "Adafactor", "NAdam",
           "RAdam", "Adagrad", "Adadelta", "Adamax", "AdamKiller", "ASGD", "LBFGS", "EMA", "ParamGroup"]

(OPT_SGD, OPT_ADAM, OPT_ADAMW, OPT_RMSPROP, OPT_LION, OPT_SOPHIA, OPT_NADAM, OPT_RADAM, OPT_ADAGRAD, OPT_ADADELTA,
 OPT_ADAMAX, OPT_ASGD, OPT_LAMB) = range(13)
OPT_ADAMKILLER = 13      # multi-launch, see AdamKiller._fused_step
OPT_ADAFACTOR = 14       # per-parameter launches, see Adafactor._fused_step


@N.register_decls
def _decls(L):
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    L.ptb_opt_chunk.restype = ci
    L.ptb_opt_tensor_bytes.restype = ci
    L.ptb_multi_tensor_opt.argtypes = [vp, vp, ci, ci, ci, C.POINTER(cf), vp, vp, vp]
    L.ptb_multi_tensor_opt.restype = ci
    L.ptb_multi_tensor_grad_norm.argtypes = [vp, vp, ci, ci, vp, cf, cf, vp, vp, vp]
    L.ptb_multi_tensor_grad_norm.restype = ci
    L.ptb_multi_tensor_scale.argtypes = [vp, vp, ci, ci, vp, vp]
    L.ptb_multi_tensor_scale.restype = ci
    L.ptb_multi_tensor_lamb.argtypes = [vp, vp, ci, vp, ci, ci, C.POINTER(cf), vp, vp, vp, vp, vp]
    L.ptb_multi_tensor_lamb.restype = ci
    L.ptb_multi_tensor_adamkiller.argtypes = [vp, vp, vp, ci, vp, ci, ci, C.POINTER(cf), vp, vp, vp, vp, vp]
    L.ptb_multi_tensor_adamkiller.restype = ci
    L.ptb_adafactor_step.argtypes = [vp, vp, ci, vp, vp, vp, vp, vp, ci, ci, C.POINTER(cf), vp, vp, vp, vp, vp]
    L.ptb_adafactor_step.restype = ci


def ParamGroup(params, **overrides) -> dict:
    """A parameter group with per-group overrides (``lr``, ``weight_decay``, ...); options left out
    inherit the optimizer's defaults (torch/optim/optimizer.h:45-90)."""
    d = {"params": list(params)}
    d.update(overrides)
    return d


class TensorTable:
    """Device-side table of {param, grad, state slots, bf16 shadow} rows plus the chunk list, rebuilt
    only when an address changes."""

    def __init__(self):
        self.key = None
        self.rows = self.chunks = None
        self.n_chunks = 0

    def build(self, ps, gs, slots, lowp, device):
        key = tuple((p.data_ptr(), g.data_ptr(), tuple(0 if s is None else s.data_ptr() for s in sl),
                     0 if lp is None else lp.data_ptr()) for p, g, sl, lp in zip(ps, gs, slots, lowp))
        if key == self.key:
            return
        lib = N.lib()
        chunk = lib.ptb_opt_chunk()
        assert lib.ptb_opt_tensor_bytes() == 56
        rows = torch.empty(len(ps), 7, dtype=torch.int64)
        ck = []
        for i, (p, g, sl, lp) in enumerate(zip(ps, gs, slots, lowp)):
            rows[i, 0], rows[i, 1] = p.data_ptr(), g.data_ptr()
            for k in range(3):
                rows[i, 2 + k] = 0 if sl[k] is None else sl[k].data_ptr()
            rows[i, 5] = 0 if lp is None else lp.data_ptr()
            rows[i, 6] = p.numel()
            ck += [(i, c) for c in range((p.numel() + chunk - 1) // chunk)]
        self.rows = rows.to(device)
        self.chunks = torch.tensor(ck, dtype=torch.int32).reshape(-1, 2).to(device)
        self.n_chunks = len(ck)
        # first chunk of every tensor (+ the total): what a per-tensor reduction over chunk partials needs
        starts = [0]
        for p in ps:
            starts.append(starts[-1] + (p.numel() + chunk - 1) // chunk)
        self.chunk_start = torch.tensor(starts, dtype=torch.int32).to(device)
        self.key = key


class Optimizer(torch.optim.Optimizer):
    """Base class: ``torch.optim.Optimizer`` bookkeeping (param groups, ``state_dict``,
    ``zero_grad``) plus the fused multi-tensor dispatch."""

    kind: Optional[int] = None          # element-wise rule id of the fused kernel, None = tensor program only
    slots: tuple = ()                   # names of the (up to three) per-parameter state tensors

    def __init__(self, params, defaults, fused: Optional[bool] = None):
        super().__init__(params, defaults)
        self.fused = fused
        self._tables: Dict[int, TensorTable] = {}
        self.grad_scale: Optional[torch.Tensor] = None     # device scalar folded into every gradient
        self.skip_flag: Optional[torch.Tensor] = None      # device flag: non-zero => skip the step
        self.lowp_params: Dict[int, torch.Tensor] = {}     # id(param) -> bf16 shadow written by the step
        self.ext_grads: Dict[int, torch.Tensor] = {}       # id(param) -> gradient held outside ``param.grad``

    # -- reference-style flat export: "state.<linear param index>.<key>" (optimizer.h:116-148)
    def flat_state_dict(self) -> Dict[str, torch.Tensor]:
        out, i = {}, 0
        for g in self.param_groups:
            for p in g["params"]:
                for k, v in self.state.get(p, {}).items():
                    out[f"state.{i}.{k}"] = v if torch.is_tensor(v) else torch.tensor(float(v))
                i += 1
        return out

    def load_flat_state_dict(self, flat: Dict[str, torch.Tensor]):
        params = [p for g in self.param_groups for p in g["params"]]
        for key, v in flat.items():
            _, idx, name = key.split(".", 2)
            st = self.state[params[int(idx)]]
            st[name] = v.clone() if name != "step" else torch.as_tensor(float(v))
        # the bias corrections and first-step rules read the group's counter: resume it from the restored steps
        for g in self.param_groups:
            steps = [float(self.state[p]["step"]) for p in g["params"] if "step" in self.state.get(p, {})]
            if steps:
                g["_step"] = int(max(steps))

    def set_grad_source(self, param: torch.Tensor, grad: Optional[torch.Tensor]):
        """Read this parameter's gradient from ``grad`` instead of ``param.grad``.  PyTorch only lets
        ``.grad`` hold the parameter's own dtype; fp32 master weights whose gradients arrive in bf16 (a
        reduce-scattered bucket, a bf16 model replica) register the bf16 tensor here."""
        if grad is None:
            self.ext_grads.pop(id(param), None)
        else:
            self.ext_grads[id(param)] = grad

    def _grad(self, p):
        g = self.ext_grads.get(id(p))
        return g if g is not None else p.grad

    def attach_lowp(self, param: torch.Tensor, shadow: torch.Tensor):
        """Have the fused step also write ``shadow`` (bf16, same shape) = the updated fp32 ``param``."""
        self.lowp_params[id(param)] = shadow

    # -- subclass interface
    def _init_state(self, p: torch.Tensor, group: dict) -> dict:
        return {name: torch.zeros_like(p, memory_format=torch.preserve_format) for name in self.slots}

    def _scalars(self, group: dict, step: int) -> List[float]:
        raise NotImplementedError

    def _update(self, p, g, st, h, group):
        """Tensor-op form of the rule for one parameter (CPU path and oracle)."""
        raise NotImplementedError

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            ps = [p for p in group["params"] if self._grad(p) is not None]
            if not ps:
                continue
            if "_step" not in group:        # state restored by another route: continue from its step count
                group["_step"] = int(max((float(self.state[p]["step"]) for p in ps if "step" in self.state[p]), default=0))
            for p in ps:
                st = self.state[p]
                if "step" not in st:
                    st.update(self._init_state(p, group))
                    st["step"] = torch.tensor(0.0)
            group["_step"] = group["_step"] + 1
            step = group["_step"]
            for p in ps:
                self.state[p]["step"] += 1
            h = self._scalars(group, step)
            use_fused = self.kind is not None and all(
                p.is_cuda and p.dtype == torch.float32 and p.is_contiguous() and self._grad(p).is_contiguous()
                and self._grad(p).dtype in (torch.float32, torch.bfloat16) for p in ps)
            if self.fused is False:
                use_fused = False
            if self.fused is True and not use_fused and ps[0].is_cuda:
                raise RuntimeError(f"{type(self).__name__}: fused step needs contiguous fp32 CUDA parameters with fp32/bf16 grads")
            if use_fused:
                for dt in (torch.float32, torch.bfloat16):
                    sub = [p for p in ps if self._grad(p).dtype == dt]
                    if sub:
                        self._fused_step(gi * 2 + (dt == torch.bfloat16), sub, h, dt == torch.bfloat16)
            else:
                for p in ps:
                    g = self._grad(p)
                    g = g.float() if g.dtype != p.dtype else g
                    if self.grad_scale is not None:
                        g = g * self.grad_scale.to(g.device)
                    if self.skip_flag is not None and int(self.skip_flag) != 0:
                        continue
                    self._update(p, g, self.state[p], h, group)
                    lp = self.lowp_params.get(id(p))
                    if lp is not None:
                        lp.copy_(p)
        return loss

    def _fused_step(self, key, ps, h, bf16):
        lib = N.lib()
        dev = ps[0].device
        tab = self._tables.setdefault(key, TensorTable())
        slots = [tuple(self.state[p].get(n) for n in self.slots) + (None,) * (3 - len(self.slots)) for p in ps]
        tab.build(ps, [self._grad(p) for p in ps], slots, [self.lowp_params.get(id(p)) for p in ps], dev)
        harr = (C.c_float * 16)(*(list(h) + [0.0] * (16 - len(h))))
        st = torch.cuda.current_stream(dev).cuda_stream
        N.check(lib.ptb_multi_tensor_opt(tab.rows.data_ptr(), tab.chunks.data_ptr(), tab.n_chunks, self.kind, int(bf16), harr,
                                         N.ptr(self.grad_scale), N.ptr(self.skip_flag), st), "multi_tensor_opt")


def _wd_l2(p, g, wd):
    return g.add(p, alpha=wd) if wd != 0 else g


class SGD(Optimizer):
    kind, slots = OPT_SGD, ("momentum_buffer",)

    def __init__(self, params, lr=0.01, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, fused=None):
        super().__init__(params, dict(lr=lr, momentum=momentum, dampening=dampening, weight_decay=weight_decay,
                                      nesterov=nesterov), fused)

    def _init_state(self, p, group):
        return {"momentum_buffer": torch.zeros_like(p)} if group["momentum"] != 0 else {}

    def _scalars(self, g, step):
        return [g["lr"], g["momentum"], g["dampening"], g["weight_decay"], float(g["nesterov"]), float(step == 1)]

    def _update(self, p, g, st, h, group):
        lr, mom, damp, wd, nest, first = h
        g = _wd_l2(p, g, wd)
        if mom != 0:
            buf = st["momentum_buffer"]
            if first:
                buf.copy_(g)
            else:
                buf.mul_(mom).add_(g, alpha=1 - damp)
            g = g.add(buf, alpha=mom) if nest else buf
        p.add_(g, alpha=-lr)


class Adam(Optimizer):
    kind, slots = OPT_ADAM, ("exp_avg", "exp_avg_sq", "max_exp_avg_sq")

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, amsgrad=False, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad), fused)

    def _init_state(self, p, group):
        st = {"exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
        if group["amsgrad"]:
            st["max_exp_avg_sq"] = torch.zeros_like(p)
        return st

    def _scalars(self, g, step):
        b1, b2 = g["betas"]
        return [g["lr"], b1, b2, g["eps"], g["weight_decay"], 1 - b1 ** step, 1 - b2 ** step, float(g["amsgrad"])]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, bc1, bc2, ams = h
        if self.kind == OPT_ADAMW:
            p.mul_(1 - lr * wd)
        else:
            g = _wd_l2(p, g, wd)
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        v = st["exp_avg_sq"]
        if ams:
            torch.maximum(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
            v = st["max_exp_avg_sq"]
        denom = v.sqrt().div_(math.sqrt(bc2)).add_(eps)
        p.addcdiv_(st["exp_avg"], denom, value=-lr / bc1)


class AdamW(Adam):
    kind = OPT_ADAMW

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False, fused=None):
        super().__init__(params, lr, betas, eps, weight_decay, amsgrad, fused)


class RMSprop(Optimizer):
    kind, slots = OPT_RMSPROP, ("square_avg", "momentum_buffer", "grad_avg")

    def __init__(self, params, lr=0.01, alpha=0.99, eps=1e-8, weight_decay=0.0, momentum=0.0, centered=False, fused=None):
        super().__init__(params, dict(lr=lr, alpha=alpha, eps=eps, weight_decay=weight_decay, momentum=momentum,
                                      centered=centered), fused)

    def _init_state(self, p, group):
        st = {"square_avg": torch.zeros_like(p)}
        if group["momentum"] > 0:
            st["momentum_buffer"] = torch.zeros_like(p)
        if group["centered"]:
            st["grad_avg"] = torch.zeros_like(p)
        return st

    def _scalars(self, g, step):
        return [g["lr"], g["alpha"], g["eps"], g["weight_decay"], g["momentum"], float(g["centered"])]

    def _update(self, p, g, st, h, group):
        lr, alpha, eps, wd, mom, centered = h
        g = _wd_l2(p, g, wd)
        st["square_avg"].mul_(alpha).addcmul_(g, g, value=1 - alpha)
        if centered:
            st["grad_avg"].mul_(alpha).add_(g, alpha=1 - alpha)
            avg = (st["square_avg"] - st["grad_avg"] ** 2).clamp_min_(0).sqrt_().add_(eps)
        else:
            avg = st["square_avg"].sqrt().add_(eps)
        if mom > 0:
            st["momentum_buffer"].mul_(mom).addcdiv_(g, avg)
            p.add_(st["momentum_buffer"], alpha=-lr)
        else:
            p.addcdiv_(g, avg, value=-lr)


class Lion(Optimizer):
    kind, slots = OPT_LION, ("exp_avg",)

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay), fused)

    def _scalars(self, g, step):
        return [g["lr"], g["betas"][0], g["betas"][1], g["weight_decay"]]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, wd = h
        if wd != 0:
            p.mul_(1 - lr * wd)
        u = st["exp_avg"].mul(b1).add_(g, alpha=1 - b1).sign_()
        p.add_(u, alpha=-lr)
        st["exp_avg"].mul_(b2).add_(g, alpha=1 - b2)


class SophiaG(Optimizer):
    kind, slots = OPT_SOPHIA, ("exp_avg", "hessian")

    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), eps=1e-12, weight_decay=0.0, rho=0.04,
                 hessian_update_interval=10, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, rho=rho,
                                      hessian_update_interval=hessian_update_interval), fused)

    def _scalars(self, g, step):
        return [g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"], g["rho"]]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, rho = h
        if wd != 0:
            p.mul_(1 - lr * wd)
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["hessian"].mul_(b2).addcmul_(g, g, value=1 - b2)
        p.add_((st["exp_avg"] / st["hessian"].clamp_min(eps)).clamp_(-rho, rho), alpha=-lr)


Sophia = SophiaG


class NAdam(Optimizer):
    kind, slots = OPT_NADAM, ("exp_avg", "exp_avg_sq")

    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, momentum_decay=0.004, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                      momentum_decay=momentum_decay), fused)

    def _scalars(self, g, step):
        b1, b2 = g["betas"]
        md = g["momentum_decay"]
        mu_t = b1 * (1 - 0.5 * 0.96 ** (step * md))
        mu_n = b1 * (1 - 0.5 * 0.96 ** ((step + 1) * md))
        g["_mu_product"] = g.get("_mu_product", 1.0) * mu_t
        return [g["lr"], b1, b2, g["eps"], g["weight_decay"], mu_t, mu_n, g["_mu_product"], g["_mu_product"] * mu_n,
                1 - b2 ** step]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, mu_t, mu_n, mp, mpn, bc2 = h
        g = _wd_l2(p, g, wd)
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        denom = (st["exp_avg_sq"] / bc2).sqrt_().add_(eps)
        p.addcdiv_(g, denom, value=-lr * (1 - mu_t) / (1 - mp))
        p.addcdiv_(st["exp_avg"], denom, value=-lr * mu_n / (1 - mpn))


class RAdam(Optimizer):
    kind, slots = OPT_RADAM, ("exp_avg", "exp_avg_sq")

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay), fused)

    def _scalars(self, g, step):
        b1, b2 = g["betas"]
        rho_inf = 2 / (1 - b2) - 1
        b2t = b2 ** step
        rho_t = rho_inf - 2 * step * b2t / (1 - b2t)
        rect = 0.0
        if rho_t > 5:
            rect = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t))
        return [g["lr"], b1, b2, g["eps"], g["weight_decay"], 1 - b1 ** step, rect, 1 - b2t]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, bc1, rect, bc2 = h
        g = _wd_l2(p, g, wd)
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        mhat = st["exp_avg"] / bc1
        if rect > 0:
            p.addcdiv_(mhat, (st["exp_avg_sq"] / bc2).sqrt_().add_(eps), value=-lr * rect)
        else:
            p.add_(mhat, alpha=-lr)


class Adagrad(Optimizer):
    kind, slots = OPT_ADAGRAD, ("sum",)

    def __init__(self, params, lr=0.01, lr_decay=0.0, weight_decay=0.0, eps=1e-10, initial_accumulator_value=0.0, fused=None):
        super().__init__(params, dict(lr=lr, lr_decay=lr_decay, weight_decay=weight_decay, eps=eps,
                                      initial_accumulator_value=initial_accumulator_value), fused)

    def _init_state(self, p, group):
        return {"sum": torch.full_like(p, group["initial_accumulator_value"])}

    def _scalars(self, g, step):
        return [g["lr"] / (1 + (step - 1) * g["lr_decay"]), g["eps"], g["weight_decay"]]

    def _update(self, p, g, st, h, group):
        clr, eps, wd = h
        g = _wd_l2(p, g, wd)
        st["sum"].addcmul_(g, g)
        p.addcdiv_(g, st["sum"].sqrt().add_(eps), value=-clr)


class Adadelta(Optimizer):
    kind, slots = OPT_ADADELTA, ("square_avg", "acc_delta")

    def __init__(self, params, lr=1.0, rho=0.9, eps=1e-6, weight_decay=0.0, fused=None):
        super().__init__(params, dict(lr=lr, rho=rho, eps=eps, weight_decay=weight_decay), fused)

    def _scalars(self, g, step):
        return [g["lr"], g["rho"], g["eps"], g["weight_decay"]]

    def _update(self, p, g, st, h, group):
        lr, rho, eps, wd = h
        g = _wd_l2(p, g, wd)
        st["square_avg"].mul_(rho).addcmul_(g, g, value=1 - rho)
        d = (st["acc_delta"] + eps).sqrt_().div_((st["square_avg"] + eps).sqrt_()).mul_(g)
        st["acc_delta"].mul_(rho).addcmul_(d, d, value=1 - rho)
        p.add_(d, alpha=-lr)


class Adamax(Optimizer):
    kind, slots = OPT_ADAMAX, ("exp_avg", "exp_inf")

    def __init__(self, params, lr=2e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay), fused)

    def _scalars(self, g, step):
        return [g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"], 1 - g["betas"][0] ** step]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, bc1 = h
        g = _wd_l2(p, g, wd)
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        torch.maximum(st["exp_inf"] * b2, g.abs() + eps, out=st["exp_inf"])
        p.addcdiv_(st["exp_avg"], st["exp_inf"], value=-lr / bc1)


class ASGD(Optimizer):
    kind, slots = OPT_ASGD, ("ax",)

    def __init__(self, params, lr=0.01, lambd=1e-4, alpha=0.75, t0=1e6, weight_decay=0.0, fused=None):
        super().__init__(params, dict(lr=lr, lambd=lambd, alpha=alpha, t0=t0, weight_decay=weight_decay), fused)

    def _init_state(self, p, group):
        return {"ax": p.detach().clone()}

    def _scalars(self, g, step):
        eta = g.get("_eta", g["lr"])
        mu = g.get("_mu", 1.0)
        # schedule for the NEXT step, as in the reference (asgd.h: eta and mu are updated after the step)
        g["_eta"] = g["lr"] / (1 + g["lambd"] * g["lr"] * step) ** g["alpha"]
        g["_mu"] = 1.0 / max(1.0, step - g["t0"])
        return [eta, g["lambd"], g["weight_decay"], mu]

    def _update(self, p, g, st, h, group):
        eta, lambd, wd, mu = h
        g = _wd_l2(p, g, wd)
        p.mul_(1 - lambd * eta).add_(g, alpha=-eta)
        if mu != 1:
            st["ax"].add_(p - st["ax"], alpha=mu)
        else:
            st["ax"].copy_(p)

    @torch.no_grad()
    def swap_in_averaged_params(self):
        for g in self.param_groups:
            for p in g["params"]:
                if "ax" in self.state.get(p, {}):
                    p.copy_(self.state[p]["ax"])


class LAMB(Optimizer):
    """Layer-wise adaptive moments (torch/optim/lamb.h).  On CUDA the step is three launches over the whole parameter
    group (moments + update direction + partial norms, per-tensor trust ratios, apply); ``lamb_update`` is the buffer
    that carries the update direction between them."""

    kind, slots = OPT_LAMB, ("exp_avg", "exp_avg_sq", "lamb_update")

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, bias_correction=True, fused=None):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, bias_correction=bias_correction),
                         fused)

    def _init_state(self, p, group):
        st = {"exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
        if p.is_cuda and self.fused is not False:
            st["lamb_update"] = torch.zeros_like(p)
        return st

    def _fused_step(self, key, ps, h, bf16):
        lib = N.lib()
        dev = ps[0].device
        for p in ps:
            if "lamb_update" not in self.state[p]:
                self.state[p]["lamb_update"] = torch.zeros_like(p)
        tab = self._tables.setdefault(key, TensorTable())
        slots = [tuple(self.state[p][n] for n in self.slots) for p in ps]
        tab.build(ps, [self._grad(p) for p in ps], slots, [self.lowp_params.get(id(p)) for p in ps], dev)
        if getattr(tab, "lamb_partial", None) is None or tab.lamb_partial.numel() < 2 * tab.n_chunks:
            tab.lamb_partial = torch.empty(2 * max(tab.n_chunks, 1), device=dev)
            tab.lamb_trust = torch.ones(len(ps), device=dev)
        harr = (C.c_float * 16)(*(list(h) + [0.0] * (16 - len(h))))
        st = torch.cuda.current_stream(dev).cuda_stream
        N.check(lib.ptb_multi_tensor_lamb(tab.rows.data_ptr(), tab.chunks.data_ptr(), tab.n_chunks, tab.chunk_start.data_ptr(),
                                          len(ps), int(bf16), harr, N.ptr(self.grad_scale), N.ptr(self.skip_flag),
                                          tab.lamb_partial.data_ptr(), tab.lamb_trust.data_ptr(), st), "multi_tensor_lamb")

    def _scalars(self, g, step):
        b1, b2 = g["betas"]
        bc = g["bias_correction"]
        return [g["lr"], b1, b2, g["eps"], g["weight_decay"], (1 - b1 ** step) if bc else 1.0, (1 - b2 ** step) if bc else 1.0]

    def _update(self, p, g, st, h, group):
        lr, b1, b2, eps, wd, bc1, bc2 = h
        st["exp_avg"].mul_(b1).add_(g, alpha=1 - b1)
        st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
        upd = (st["exp_avg"] / bc1) / ((st["exp_avg_sq"] / bc2).sqrt_().add_(eps))
        if wd != 0:
            upd.add_(p, alpha=wd)
        wn, un = p.norm(), upd.norm()
        trust = torch.where((wn > 0) & (un > 0), wn / un, torch.ones_like(wn))
        p.add_(upd * trust, alpha=-lr)


class Adafactor(Optimizer):
    """Factored second moments (torch/optim/adafactor.h).  On CUDA a matrix or vector parameter steps in seven small
    launches (row sums and weight norm, column sums, the fold that advances both vectors and sets the step size, the norm
    of the update, its clip factor, apply) with no value coming back to the host; parameters of more than two
    dimensions take the tensor program."""

    kind = OPT_ADAFACTOR

    def __init__(self, params, lr=0.0, eps1=1e-30, eps2=1e-3, clip_threshold=1.0, decay_rate=-0.8, beta1=0.0,
                 weight_decay=0.0, scale_parameter=True, relative_step=True, warmup_init=False, fused=None):
        super().__init__(params, dict(lr=lr, eps1=eps1, eps2=eps2, clip_threshold=clip_threshold, decay_rate=decay_rate,
                                      beta1=beta1, weight_decay=weight_decay, scale_parameter=scale_parameter,
                                      relative_step=relative_step, warmup_init=warmup_init), fused)

    def _fused_step(self, key, ps, h, bf16):
        lib = N.lib()
        dev = ps[0].device
        group = next(g for g in self.param_groups if any(q is ps[0] for q in g["params"]))
        t = h[0]
        lr_t = group["lr"]
        if group["relative_step"] or lr_t <= 0:
            lr_t = min(1e-6 * t if group["warmup_init"] else 1e-2, 1 / math.sqrt(t))
        hh = [lr_t, group["eps1"], group["eps2"], group["clip_threshold"], 1 - t ** group["decay_rate"], group["beta1"],
              group["weight_decay"], float(group["scale_parameter"])]
        harr = (C.c_float * 16)(*(hh + [0.0] * (16 - len(hh))))
        st = torch.cuda.current_stream(dev).cuda_stream
        def scratch_floats(p):          # row sums + column sums per split of 256 rows + two partial-sum arrays
            rows = p.shape[0] if p.dim() == 2 else 1
            return rows + (rows + 255) // 256 * p.shape[-1] + 2 * 592
        need = max((scratch_floats(p) for p in ps if 1 <= p.dim() <= 2), default=0)
        if need and (getattr(self, "_af_scratch", None) is None or self._af_scratch.numel() < need):
            self._af_scratch = torch.empty(need, device=dev)
        for p in ps:
            s_ = self.state[p]
            g = self._grad(p)
            if p.dim() > 2 or p.dim() == 0:
                gg = g.float() if g.dtype != p.dtype else g
                if self.grad_scale is not None:
                    gg = gg * self.grad_scale
                self._update(p, gg, s_, h, group)
                continue
            if "af_scalars" not in s_:
                s_["af_scalars"] = torch.zeros(8, device=dev)
            rows, cols = (p.shape[0], p.shape[1]) if p.dim() == 2 else (1, p.numel())
            fact = p.dim() == 2
            N.check(lib.ptb_adafactor_step(p.data_ptr(), g.data_ptr(), int(bf16), N.ptr(s_["exp_avg_sq_row"]) if fact else None,
                                           N.ptr(s_["exp_avg_sq_col"]) if fact else None, None if fact else N.ptr(s_["exp_avg_sq"]),
                                           N.ptr(s_.get("exp_avg")), N.ptr(self.lowp_params.get(id(p))), rows, cols, harr,
                                           N.ptr(self.grad_scale), N.ptr(self.skip_flag), self._af_scratch.data_ptr(),
                                           s_["af_scalars"].data_ptr(), st), "adafactor_step")

    def _init_state(self, p, group):
        st = {}
        if p.dim() >= 2:
            st["exp_avg_sq_row"] = torch.zeros(p.shape[:-1], dtype=p.dtype, device=p.device)
            st["exp_avg_sq_col"] = torch.zeros(p.shape[:-2] + p.shape[-1:], dtype=p.dtype, device=p.device)
        else:
            st["exp_avg_sq"] = torch.zeros_like(p)
        if group["beta1"] > 0:
            st["exp_avg"] = torch.zeros_like(p)
        return st

    def _scalars(self, g, step):
        return [float(step)]

    def _update(self, p, g, st, h, group):
        t = h[0]
        eps1, eps2 = group["eps1"], group["eps2"]
        rms_p = float(p.norm() / math.sqrt(max(p.numel(), 1)))
        lr_t = group["lr"]
        if group["relative_step"] or lr_t <= 0:
            lr_t = min(1e-6 * t if group["warmup_init"] else 1e-2, 1 / math.sqrt(t))
        if group["scale_parameter"]:
            lr_t *= max(eps2, rms_p)
        beta2_t = 1 - t ** group["decay_rate"]
        g2 = g * g + eps1
        if p.dim() >= 2:
            st["exp_avg_sq_row"].mul_(beta2_t).add_(g2.mean(-1), alpha=1 - beta2_t)
            st["exp_avg_sq_col"].mul_(beta2_t).add_(g2.mean(-2), alpha=1 - beta2_t)
            row = st["exp_avg_sq_row"]
            rf = (row / row.mean(-1, keepdim=True).clamp_min(eps1)).unsqueeze(-1)
            v = rf * st["exp_avg_sq_col"].unsqueeze(-2)
            upd = g / v.sqrt().clamp_min(eps1)
        else:
            st["exp_avg_sq"].mul_(beta2_t).add_(g2, alpha=1 - beta2_t)
            upd = g / st["exp_avg_sq"].sqrt().clamp_min(eps1)
        rms_u = float(upd.norm() / math.sqrt(max(p.numel(), 1)))
        scale = max(1.0, rms_u / group["clip_threshold"])
        if scale > 1:
            upd = upd / scale
        if group["beta1"] > 0:
            st["exp_avg"].mul_(group["beta1"]).add_(upd, alpha=1 - group["beta1"])
            upd = st["exp_avg"]
        if group["weight_decay"] != 0:
            p.mul_(1 - lr_t * group["weight_decay"])
        p.add_(upd, alpha=-lr_t)


class AdamKiller(Optimizer):
    """Curvature-adaptive momentum, per-layer trust ratio, gradient lookahead and update clipping
    (torch/optim/adamkiller.h:29-62 for the options, :92-340 for the rule)."""

    kind = OPT_ADAMKILLER

    def __init__(self, params, lr=1e-3, beta1_min=0.7, beta1_max=0.95, beta2=0.999, eps=1e-8, weight_decay=0.01,
                 use_adaptive_momentum=True, use_per_layer_lr=True, use_gradient_prediction=True, use_warm_restarts=False,
                 restart_period=1000, max_grad_norm=1.0, lr_scale_min=0.5, lr_scale_max=2.0, fused=None):
        super().__init__(params, dict(lr=lr, beta1_min=beta1_min, beta1_max=beta1_max, beta2=beta2, eps=eps,
                                      weight_decay=weight_decay, use_adaptive_momentum=use_adaptive_momentum,
                                      use_per_layer_lr=use_per_layer_lr, use_gradient_prediction=use_gradient_prediction,
                                      use_warm_restarts=use_warm_restarts, restart_period=restart_period,
                                      max_grad_norm=max_grad_norm, lr_scale_min=lr_scale_min, lr_scale_max=lr_scale_max), fused)

    def _fused_step(self, key, ps, h, bf16):
        """Four element-wise launches over the whole group with a one-warp-per-tensor fold between them (per-tensor
        clipping, momentum coefficient, step size and update cap are formed on the device)."""
        lib = N.lib()
        dev = ps[0].device
        o = next(g for g in self.param_groups if any(q is ps[0] for q in g["params"]))
        t = int(h[0])
        has_prev = all("prev_grad" in self.state[p] for p in ps)
        for p in ps:
            s_ = self.state[p]
            if "prev_grad" not in s_:
                s_["prev_grad"] = torch.zeros_like(p)
            if "ak_scratch" not in s_:
                s_["ak_scratch"] = torch.empty_like(p)
        tab_a = self._tables.setdefault(key, TensorTable())
        tab_b = self._tables.setdefault(("b", key), TensorTable())
        grads = [self._grad(p) for p in ps]
        lowp = [self.lowp_params.get(id(p)) for p in ps]
        tab_a.build(ps, grads, [(self.state[p]["m"], self.state[p]["v"], None) for p in ps], lowp, dev)
        tab_b.build(ps, grads, [(self.state[p]["prev_grad"], self.state[p].get("grad_diff_ema"), self.state[p]["ak_scratch"]) for p in ps],
                    [None] * len(ps), dev)
        if getattr(tab_a, "ak_partial", None) is None or tab_a.ak_partial.numel() < 3 * tab_a.n_chunks:
            tab_a.ak_partial = torch.empty(3 * max(tab_a.n_chunks, 1), device=dev)
            tab_a.ak_scalars = torch.zeros(len(ps), 8, device=dev)
        restart = bool(o["use_warm_restarts"] and t % o["restart_period"] == 0)
        hh = [o["lr"], o["beta1_min"], o["beta1_max"], o["beta2"], o["eps"], o["weight_decay"], float(o["use_adaptive_momentum"]),
              float(o["use_per_layer_lr"]), float(o["use_gradient_prediction"]), float(restart), o["max_grad_norm"], o["lr_scale_min"],
              o["lr_scale_max"], float(t), float(has_prev)]
        harr = (C.c_float * 16)(*(hh + [0.0] * (16 - len(hh))))
        st = torch.cuda.current_stream(dev).cuda_stream
        N.check(lib.ptb_multi_tensor_adamkiller(tab_a.rows.data_ptr(), tab_b.rows.data_ptr(), tab_a.chunks.data_ptr(), tab_a.n_chunks,
                                                tab_a.chunk_start.data_ptr(), len(ps), int(bf16), harr, N.ptr(self.grad_scale),
                                                N.ptr(self.skip_flag), tab_a.ak_partial.data_ptr(), tab_a.ak_scalars.data_ptr(), st),
                "multi_tensor_adamkiller")

    def _init_state(self, p, group):
        st = {"m": torch.zeros_like(p), "v": torch.zeros_like(p)}
        if group["use_gradient_prediction"]:
            st["grad_diff_ema"] = torch.zeros_like(p)
        return st

    def _scalars(self, g, step):
        return [float(step)]

    def _update(self, p, g, st, h, o):
        t = int(h[0])
        lr = o["lr"]
        gn = float(g.norm())
        gscale = o["max_grad_norm"] / gn if (gn > o["max_grad_norm"] and gn > 1e-12) else 1.0
        sg = g * gscale
        beta1 = o["beta1_max"]
        prev = st.get("prev_grad")
        if o["use_adaptive_momentum"] and prev is not None:
            curv = float((sg - prev).norm()) / (lr + 1e-12)
            beta1 = o["beta1_max"] - min(curv / 100.0, 1.0) * (o["beta1_max"] - o["beta1_min"])
            beta1 = max(o["beta1_min"], min(o["beta1_max"], beta1))
        eff = sg.clone()
        if o["use_gradient_prediction"] and prev is not None:
            st["grad_diff_ema"].mul_(0.5).add_(eff - prev, alpha=0.5)
            eff.add_(st["grad_diff_ema"], alpha=0.5)
        st["prev_grad"] = sg.clone()
        b2 = o["beta2"]
        st["m"].mul_(beta1).add_(eff, alpha=1 - beta1)
        st["v"].mul_(b2).addcmul_(eff, eff, value=1 - b2)
        layer_lr = lr
        if o["use_per_layer_lr"]:
            wn, en = float(p.norm()), float(eff.norm())
            if en > 1e-8 and wn > 1e-8:
                tr = wn / (en + o["weight_decay"] * wn)
                layer_lr = lr * max(o["lr_scale_min"], min(o["lr_scale_max"], tr))
        bc1, bc2 = 1 - beta1 ** t, 1 - b2 ** t
        if o["weight_decay"] > 0:
            p.mul_(1 - layer_lr * o["weight_decay"])
        upd = (st["m"] / bc1) / ((st["v"] / bc2) + o["eps"]).sqrt_() * layer_lr
        un = float(upd.norm())
        if un > 2 * layer_lr and un > 1e-12:
            upd.mul_(2 * layer_lr / un)
        p.sub_(upd)
        if o["use_warm_restarts"] and t % o["restart_period"] == 0:
            st["m"].mul_(0.1)


class LBFGS(torch.optim.LBFGS):
    """Closure-driven L-BFGS with the reference's defaults (torch/optim/lbfgs.h)."""

    def __init__(self, params, lr=1.0, max_iter=20, max_eval=25, tolerance_grad=1e-7, tolerance_change=1e-9,
                 history_size=100, line_search_fn=None):
        super().__init__(params, lr=lr, max_iter=max_iter, max_eval=max_eval, tolerance_grad=tolerance_grad,
                         tolerance_change=tolerance_change, history_size=history_size, line_search_fn=line_search_fn)


class EMA:
    """Exponential moving average of parameters: ``shadow = decay*shadow + (1-decay)*w``
    (torch/optim/ema.h:37-122)."""

    def __init__(self, parameters: Iterable[torch.Tensor], decay: float = 0.999):
        if not 0.0 <= decay < 1.0:
            raise ValueError("EMA decay must be in [0, 1)")
        self.decay = decay
        self.params = [p for p in parameters]
        self.shadow = [p.detach().clone() for p in self.params]
        self.backup: List[torch.Tensor] = []

    @torch.no_grad()
    def update(self):
        if self.params and self.params[0].is_cuda:
            torch._foreach_lerp_(self.shadow, [p.detach() for p in self.params], 1 - self.decay)
        else:
            for s, p in zip(self.shadow, self.params):
                s.mul_(self.decay).add_(p.detach(), alpha=1 - self.decay)

    @torch.no_grad()
    def apply_shadow(self):
        self.backup = [p.detach().clone() for p in self.params]
        for p, s in zip(self.params, self.shadow):
            p.copy_(s)

    @torch.no_grad()
    def restore(self):
        for p, b in zip(self.params, self.backup):
            p.copy_(b)
        self.backup = []

    def set_decay(self, decay: float):
        self.decay = decay

    def state_dict(self):
        return {"decay": self.decay, "shadow": [s.clone() for s in self.shadow]}

    def load_state_dict(self, sd):
        self.decay = sd["decay"]
        for s, v in zip(self.shadow, sd["shadow"]):
            s.copy_(v)
