"""Quantisation: fake-quant QAT (straight-through), observers, ``prepare_qat`` / ``convert``, ``int8_matmul``,
and 4-bit block formats (INT4 / NF4) with ``Linear4bit`` (torch/quantization/*.h in the reference)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.extras import QuantizedConv2d, QuantizedLinear


class MinMaxObserver(nn.Module):
    def __init__(self, bits: int = 8, symmetric: bool = True, momentum: float = 0.0):
        super().__init__()
        self.bits, self.symmetric, self.momentum = bits, symmetric, momentum
        self.register_buffer("min_val", torch.tensor(float("inf")))
        self.register_buffer("max_val", torch.tensor(float("-inf")))
        self.frozen = False

    def forward(self, x):
        if not self.frozen:
            mn, mx = x.detach().amin(), x.detach().amax()
            if self.momentum > 0 and torch.isfinite(self.min_val):
                self.min_val.mul_(self.momentum).add_(mn * (1 - self.momentum))
                self.max_val.mul_(self.momentum).add_(mx * (1 - self.momentum))
            else:
                self.min_val.copy_(torch.minimum(self.min_val, mn))
                self.max_val.copy_(torch.maximum(self.max_val, mx))
        return x

    def qparams(self):
        qmax = 2 ** (self.bits - 1) - 1 if self.symmetric else 2 ** self.bits - 1
        if self.symmetric:
            scale = torch.maximum(self.max_val.abs(), self.min_val.abs()).clamp_min(1e-12) / qmax
            return scale, torch.zeros_like(scale)
        scale = (self.max_val - self.min_val).clamp_min(1e-12) / qmax
        return scale, torch.round(-self.min_val / scale)


MovingAverageObserver = lambda bits=8, symmetric=True: MinMaxObserver(bits, symmetric, momentum=0.9)  # noqa: E731


class _FakeQuantSTE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zp, qmin, qmax):
        q = torch.clamp(torch.round(x / scale) + zp, qmin, qmax)
        ctx.save_for_backward((x / scale + zp >= qmin) & (x / scale + zp <= qmax))
        return (q - zp) * scale

    @staticmethod
    def backward(ctx, g):
        (mask,) = ctx.saved_tensors
        return g * mask, None, None, None, None


class FakeQuantize(nn.Module):
    """Quantise-dequantise in forward, straight-through gradient inside the representable range."""

    def __init__(self, bits: int = 8, symmetric: bool = True):
        super().__init__()
        self.observer = MinMaxObserver(bits, symmetric)
        self.bits, self.symmetric, self.enabled = bits, symmetric, True

    def forward(self, x):
        self.observer(x)
        if not self.enabled:
            return x
        scale, zp = self.observer.qparams()
        qmin, qmax = (-(2 ** (self.bits - 1)), 2 ** (self.bits - 1) - 1) if self.symmetric else (0, 2 ** self.bits - 1)
        return _FakeQuantSTE.apply(x, scale, zp, qmin, qmax)

    def freeze(self):
        self.observer.frozen = True


class QATLinear(nn.Linear):
    def __init__(self, in_features, out_features, bias=True, bits=8):
        super().__init__(in_features, out_features, bias)
        self.weight_fq, self.act_fq = FakeQuantize(bits), FakeQuantize(bits)

    def forward(self, x):
        return F.linear(self.act_fq(x), self.weight_fq(self.weight), self.bias)


def prepare_qat(model: nn.Module, bits: int = 8) -> nn.Module:
    """Swap every ``nn.Linear`` for a fake-quantised one (weights shared)."""
    for name, ch in list(model.named_children()):
        if type(ch) is nn.Linear:
            q = QATLinear(ch.in_features, ch.out_features, ch.bias is not None, bits)
            q.weight, q.bias = ch.weight, ch.bias
            setattr(model, name, q)
        else:
            prepare_qat(ch, bits)
    return model


def freeze_observers(model: nn.Module):
    for m in model.modules():
        if isinstance(m, FakeQuantize):
            m.freeze()


def convert(model: nn.Module) -> nn.Module:
    """Replace (QAT) linear and conv layers by int8 weight-quantised inference layers."""
    for name, ch in list(model.named_children()):
        if isinstance(ch, nn.Linear):
            setattr(model, name, QuantizedLinear.from_float(ch))
        elif isinstance(ch, nn.Conv2d):
            setattr(model, name, QuantizedConv2d(ch))
        else:
            convert(ch)
    return model


def quantize_per_tensor(x: torch.Tensor, bits: int = 8):
    qmax = 2 ** (bits - 1) - 1
    scale = x.abs().amax().clamp_min(1e-12) / qmax
    return torch.round(x / scale).clamp(-qmax, qmax).to(torch.int8), scale


def int8_matmul(a_q: torch.Tensor, a_scale, b_q: torch.Tensor, b_scale) -> torch.Tensor:
    """``(a_q * a_scale) @ (b_q * b_scale)`` with exact int32 accumulation."""
    if a_q.is_cuda:
        acc = torch._int_mm(a_q.contiguous(), b_q.contiguous()) if a_q.shape[0] > 16 and a_q.shape[1] % 8 == 0 and b_q.shape[1] % 8 == 0 \
            else (a_q.float() @ b_q.float())
    else:
        acc = a_q.to(torch.int32) @ b_q.to(torch.int32)
    return acc.float() * (a_scale * b_scale)


# ----------------------------------------------------------------------------- 4-bit block formats
_NF4 = torch.tensor([-1.0, -0.6961928, -0.5250730, -0.3949175, -0.2844414, -0.1848449, -0.0910500, 0.0, 0.0795803, 0.1609302,
                     0.2461123, 0.3379152, 0.4407098, 0.5626170, 0.7229568, 1.0])


def quantize_4bit(w: torch.Tensor, block: int = 64, kind: str = "nf4"):
    """Block-wise 4-bit quantisation: returns ``(packed uint8 [numel/2], absmax [numel/block])``."""
    flat = w.detach().float().reshape(-1, block)
    absmax = flat.abs().amax(dim=1).clamp_min(1e-12)
    x = flat / absmax[:, None]
    if kind == "nf4":
        idx = (x.unsqueeze(-1) - _NF4.to(x.device)).abs().argmin(-1)
    else:
        idx = torch.round(x * 7).clamp(-8, 7).to(torch.int64) + 8
    idx = idx.reshape(-1).to(torch.uint8)
    return idx[0::2] | (idx[1::2] << 4), absmax


def dequantize_4bit(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = 64, kind: str = "nf4") -> torch.Tensor:
    idx = torch.stack([packed & 0xF, packed >> 4], dim=1).reshape(-1).to(torch.int64)
    vals = _NF4.to(packed.device)[idx] if kind == "nf4" else (idx.float() - 8) / 7
    return (vals.reshape(-1, block) * absmax[:, None]).reshape(shape)


class Linear4bit(nn.Module):
    def __init__(self, lin: nn.Linear, block: int = 64, kind: str = "nf4"):
        super().__init__()
        self.shape, self.block, self.kind = tuple(lin.weight.shape), block, kind
        p, a = quantize_4bit(lin.weight, block, kind)
        self.register_buffer("packed", p)
        self.register_buffer("absmax", a)
        self.bias = nn.Parameter(lin.bias.detach().clone()) if lin.bias is not None else None

    def forward(self, x):
        w = dequantize_4bit(self.packed, self.absmax, self.shape, self.block, self.kind).to(x.dtype)
        return F.linear(x, w, self.bias)
