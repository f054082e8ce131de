"""Automatic mixed precision: ``autocast`` and ``GradScaler``.

``autocast`` is PyTorch's (its op policy — matmul/conv families in low precision, softmax/norm/loss
families in fp32 — is the table the reference restates in torch/amp/autocast_policy.h:63-170).
``GradScaler`` keeps the reference's defaults (init 65536, x2 / x0.5, interval 2000,
torch/amp/grad_scaler.h:48-80) and API (``scale, unscale, step, update, get_scale, found_inf``);
on CUDA the unscale + inf/nan check is one multi-tensor kernel and the skip decision stays on the
device when the optimizer is one of this package's fused optimizers."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .optim.grad_utils import GradNormClipper

autocast = torch.autocast


class AutocastGuard(torch.autocast):
    """RAII-style name of the reference (torch/amp/autocast.h): ``with AutocastGuard('cuda', torch.bfloat16):``."""

    def __init__(self, device_type: str = "cuda", dtype: Optional[torch.dtype] = None, enabled: bool = True):
        super().__init__(device_type=device_type, dtype=dtype, enabled=enabled)


class AutocastCPUGuard(AutocastGuard):
    def __init__(self, dtype: torch.dtype = torch.bfloat16, enabled: bool = True):
        super().__init__("cpu", dtype, enabled)


class CastPolicy:
    """The four autocast categories (torch/amp/autocast_policy.h:30-60)."""
    LOWER_PRECISION = "lower_precision"      # runs in the autocast dtype
    FP32 = "fp32"                            # runs in fp32 whatever the inputs are
    PROMOTE = "promote"                      # runs in the widest input dtype
    UNCHANGED = "unchanged"                  # takes the dtype of its inputs


_LOWER = ("linear matmul mm bmm addmm addbmm baddbmm addmv mv conv1d conv2d conv3d conv_transpose1d conv_transpose2d "
          "conv_transpose3d scaled_dot_product_attention flash_attention prelu gru lstm rnn gru_cell lstm_cell rnn_tanh_cell "
          "rnn_relu_cell").split()
_FP32 = ("softmax log_softmax layer_norm batch_norm group_norm instance_norm cross_entropy nll_loss mse_loss l1_loss "
         "smooth_l1_loss huber_loss binary_cross_entropy binary_cross_entropy_with_logits kl_div poisson_nll_loss exp exp2 "
         "expm1 log log2 log10 log1p pow reciprocal rsqrt gelu tanh sum mean prod cumsum cumprod norm").split()
_PROMOTE = "add sub mul div cat stack addcmul addcdiv where bilinear dot".split()
AUTOCAST_POLICY = {**{n: CastPolicy.LOWER_PRECISION for n in _LOWER}, **{n: CastPolicy.FP32 for n in _FP32},
                   **{n: CastPolicy.PROMOTE for n in _PROMOTE}}


def get_autocast_policy(op_name: str) -> str:
    """Category of an op under autocast; ops that are not in the table keep their inputs' dtype."""
    return AUTOCAST_POLICY.get(op_name, CastPolicy.UNCHANGED)


def is_autocast_enabled(device_type: str = "cuda") -> bool:
    return torch.is_autocast_enabled(device_type)


def get_autocast_dtype(device_type: str = "cuda") -> torch.dtype:
    return torch.get_autocast_dtype(device_type)


# the reference's free functions over the autocast state (torch/amp/autocast.h)
get_autocast_category = get_autocast_policy
policy_for = get_autocast_policy


def is_autocast_cpu_enabled() -> bool:
    return torch.is_autocast_enabled("cpu")


def set_autocast_enabled(enabled: bool, device_type: str = "cuda"):
    torch.set_autocast_enabled(device_type, bool(enabled))


def set_autocast_dtype(dtype: torch.dtype, device_type: str = "cuda"):
    torch.set_autocast_dtype(device_type, dtype)


def set_autocast_cpu_enabled(enabled: bool):
    set_autocast_enabled(enabled, "cpu")


def set_autocast_cpu_dtype(dtype: torch.dtype):
    set_autocast_dtype(dtype, "cpu")


def has_tensor_cores() -> bool:
    """Whether the current CUDA device has tensor cores (compute capability 7.0 or later)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 7


def autocast_matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """A matrix product under the lower-precision policy whatever the surrounding autocast state is."""
    dev = a.device.type
    dt = torch.get_autocast_dtype(dev) if torch.is_autocast_enabled(dev) else (torch.bfloat16 if dev == "cpu" else torch.float16)
    return torch.matmul(a.to(dt), b.to(dt))


def autocast_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Softmax under the fp32 policy: computed in float32 whatever the input dtype."""
    return torch.softmax(x.float(), dim)


@dataclass
class GradScalerOptions:
    init_scale: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000
    enabled: bool = True


def make_grad_scaler(options: "GradScalerOptions" = None) -> "GradScaler":
    o = options or GradScalerOptions()
    return GradScaler(o.init_scale, o.growth_factor, o.backoff_factor, o.growth_interval, o.enabled)


def make_disabled_scaler() -> "GradScaler":
    return GradScaler(enabled=False)


class GradScaler:
    def __init__(self, init_scale: float = 65536.0, growth_factor: float = 2.0, backoff_factor: float = 0.5,
                 growth_interval: int = 2000, enabled: bool = True):
        self._scale, self.growth_factor, self.backoff_factor = float(init_scale), growth_factor, backoff_factor
        self.growth_interval, self.enabled = growth_interval, enabled
        self._growth_tracker = 0
        self._found_inf = False
        self._unscaled = set()
        self._clippers = {}

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * self._scale if self.enabled else loss

    def get_scale(self) -> float:
        return self._scale

    @property
    def found_inf(self) -> bool:
        return self._found_inf

    @torch.no_grad()
    def unscale(self, optimizer):
        """Divide the optimizer's gradients by the scale (once per step) and record inf/nan."""
        if not self.enabled or id(optimizer) in self._unscaled:
            return
        self._unscaled.add(id(optimizer))
        params = [p for g in optimizer.param_groups for p in g["params"] if p.grad is not None]
        if not params:
            return
        inv = 1.0 / self._scale
        if all(p.grad.is_cuda and p.grad.is_contiguous() and p.grad.dtype == torch.float32 for p in params):
            c = self._clippers.get(id(optimizer))
            if c is None or [id(p) for p in c.params] != [id(p) for p in params]:
                c = self._clippers[id(optimizer)] = GradNormClipper(params, 0.0)
            c.compute(extra_scale=inv)      # coefficient = 1/scale, found_inf flag set on the device
            c.scale_grads()
            self._found_inf = bool(int(c.found_inf))
        else:
            bad = False
            for p in params:
                p.grad.mul_(inv)
                bad = bad or not bool(torch.isfinite(p.grad).all())
            self._found_inf = bad

    unscale_ = unscale

    def step(self, optimizer, *a, **kw) -> bool:
        """Run ``optimizer.step()`` unless an inf/nan was found; returns whether the step ran."""
        if not self.enabled:
            optimizer.step(*a, **kw)
            return True
        self.unscale(optimizer)
        if self._found_inf:
            return False
        optimizer.step(*a, **kw)
        return True

    def update(self, new_scale: Optional[float] = None):
        if not self.enabled:
            return
        if new_scale is not None:
            self._scale = float(new_scale)
        elif self._found_inf:
            self._scale *= self.backoff_factor
            self._growth_tracker = 0
        else:
            self._growth_tracker += 1
            if self._growth_tracker >= self.growth_interval:
                self._scale *= self.growth_factor
                self._growth_tracker = 0
        self._found_inf = False
        self._unscaled.clear()

    def state_dict(self):
        return {"scale": self._scale, "growth_factor": self.growth_factor, "backoff_factor": self.backoff_factor,
                "growth_interval": self.growth_interval, "_growth_tracker": self._growth_tracker}

    def load_state_dict(self, sd):
        self._scale = float(sd["scale"])
        self.growth_factor, self.backoff_factor = sd["growth_factor"], sd["backoff_factor"]
        self.growth_interval, self._growth_tracker = sd["growth_interval"], sd["_growth_tracker"]
