"""Layers of the reference that PyTorch does not ship."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class LowRankLinear(nn.Module):
    """``y = x (A B)^T + b`` with ``A [out, rank]``, ``B [rank, in]`` (torch/nn/modules/linear.h:549-640):
    uniform init with bounds ``1/sqrt(rank)`` and ``1/sqrt(in)`` so that ``A B`` has Linear-like variance."""

    def __init__(self, in_features: int, out_features: int, rank: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features, self.rank = in_features, out_features, rank
        self.A = nn.Parameter(torch.empty(out_features, rank))
        self.B = nn.Parameter(torch.empty(rank, in_features))
        self.bias = nn.Parameter(torch.empty(out_features)) if bias else None
        self.reset_parameters()

    def reset_parameters(self):
        nn.init.uniform_(self.A, -1 / math.sqrt(self.rank), 1 / math.sqrt(self.rank))
        nn.init.uniform_(self.B, -1 / math.sqrt(self.in_features), 1 / math.sqrt(self.in_features))
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, x):
        return F.linear(F.linear(x, self.B), self.A, self.bias)

    def extra_repr(self):
        return f"in_features={self.in_features}, out_features={self.out_features}, rank={self.rank}, bias={self.bias is not None}"


def _reduce(x, reduction):
    r = str(reduction).lower()
    return x.mean() if r == "mean" else x.sum() if r == "sum" else x


class FocalLoss(nn.Module):
    """Binary focal loss on probabilities: ``-alpha_t (1-p_t)^gamma log p_t`` (torch/nn/modules/loss.h:1726-1796)."""

    def __init__(self, reduction: str = "mean", alpha: float = 0.25, gamma: float = 2.0):
        super().__init__()
        self.reduction, self.alpha, self.gamma = reduction, alpha, gamma

    def forward(self, input, target):
        if input.shape != target.shape:
            raise ValueError("Input and target must have the same shape")
        p = input.clamp(1e-7, 1 - 1e-7)
        pt = target * p + (1 - target) * (1 - p)
        at = target * self.alpha + (1 - target) * (1 - self.alpha)
        return _reduce(-at * (1 - pt) ** self.gamma * pt.log(), self.reduction)


class DiceLoss(nn.Module):
    """``1 - (2 sum(xy) + s) / (sum x + sum y + s)`` per sample (torch/nn/modules/loss.h:1798-1870)."""

    def __init__(self, reduction: str = "mean", smooth: float = 1.0):
        super().__init__()
        self.reduction, self.smooth = reduction, smooth

    def forward(self, input, target):
        if input.shape != target.shape:
            raise ValueError("Input and target must have the same shape")
        x, y = input.flatten(1), target.flatten(1)
        dice = (2 * (x * y).sum(1) + self.smooth) / (x.sum(1) + y.sum(1) + self.smooth)
        return _reduce(1 - dice, self.reduction)


class GlobalAvgPool2d(nn.Module):
    def forward(self, x):
        return x.mean(dim=(-2, -1))


class PositionalEncoding(nn.Module):
    """Sinusoidal positions added to ``[T, B, D]`` (or ``[B, T, D]`` with ``batch_first``) then dropout
    (torch/nn/modules/transformer.h, ``PositionalEncoding(d_model, dropout=0.1, max_len=5000)``)."""

    def __init__(self, d_model: int, dropout: float = 0.1, max_len: int = 5000, batch_first: bool = False):
        super().__init__()
        self.dropout, self.batch_first = nn.Dropout(dropout), batch_first
        pos = torch.arange(max_len).unsqueeze(1)
        div = torch.exp(torch.arange(0, d_model, 2) * (-math.log(10000.0) / d_model))
        pe = torch.zeros(max_len, d_model)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)[:, : d_model // 2]
        self.register_buffer("pe", pe)

    def forward(self, x):
        if self.batch_first:
            return self.dropout(x + self.pe[: x.size(1)].unsqueeze(0))
        return self.dropout(x + self.pe[: x.size(0)].unsqueeze(1))


class QuantizedLinear(nn.Module):
    """Int8 weight-quantised linear layer (per-output-channel symmetric scales); built by
    ``quantization.convert`` or ``from_float`` (torch/nn/modules/quantized.h)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("qweight", torch.zeros(out_features, in_features, dtype=torch.int8))
        self.register_buffer("scale", torch.ones(out_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None

    @classmethod
    def from_float(cls, lin: nn.Linear) -> "QuantizedLinear":
        q = cls(lin.in_features, lin.out_features, lin.bias is not None)
        w = lin.weight.detach()
        scale = w.abs().amax(dim=1).clamp_min(1e-12) / 127.0
        q.qweight.copy_(torch.round(w / scale[:, None]).clamp(-127, 127).to(torch.int8))
        q.scale.copy_(scale)
        if lin.bias is not None:
            q.bias.data.copy_(lin.bias.detach())
        return q

    def forward(self, x):
        return F.linear(x, self.qweight.to(x.dtype) * self.scale[:, None].to(x.dtype), self.bias)


class QuantizedConv2d(nn.Module):
    def __init__(self, conv: nn.Conv2d):
        super().__init__()
        w = conv.weight.detach()
        scale = w.abs().amax(dim=(1, 2, 3)).clamp_min(1e-12) / 127.0
        self.register_buffer("qweight", torch.round(w / scale[:, None, None, None]).clamp(-127, 127).to(torch.int8))
        self.register_buffer("scale", scale)
        self.bias = nn.Parameter(conv.bias.detach().clone()) if conv.bias is not None else None
        self.stride, self.padding, self.dilation, self.groups = conv.stride, conv.padding, conv.dilation, conv.groups

    def forward(self, x):
        w = self.qweight.to(x.dtype) * self.scale[:, None, None, None].to(x.dtype)
        return F.conv2d(x, w, self.bias, self.stride, self.padding, self.dilation, self.groups)


def num_parameters(module: nn.Module, only_trainable: bool = False) -> int:
    return sum(p.numel() for p in module.parameters() if p.requires_grad or not only_trainable)
