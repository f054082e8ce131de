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


# ----------------------------------------------------------------------------- post-training static quantisation (torch/quantization/quantize.h)
from dataclasses import dataclass as _dataclass  # noqa: E402

Observer = MinMaxObserver                  # the reference's base-class name


@_dataclass
class QConfig:
    """What to observe and how to quantise: bit width, symmetric or affine, one scale per tensor or per output channel."""
    bits: int = 8
    symmetric: bool = True
    per_channel: bool = False
    momentum: float = 0.0                  # 0: running min / max; > 0: moving average of the batch extremes


def default_qconfig() -> QConfig:
    return QConfig()


def default_per_channel_qconfig() -> QConfig:
    return QConfig(per_channel=True)


@_dataclass
class QuantizedTensor:
    """Integer values with the scale (and zero point) that maps them back: ``(q - zero_point) * scale``."""
    q: torch.Tensor
    scale: torch.Tensor
    zero_point: torch.Tensor
    axis: int = -1                         # -1: one scale for the tensor; otherwise the channel axis of `scale`

    def dequantize(self) -> torch.Tensor:
        if self.axis < 0:
            return (self.q.float() - self.zero_point) * self.scale
        shape = [1] * self.q.dim()
        shape[self.axis] = -1
        return (self.q.float() - self.zero_point.view(shape)) * self.scale.view(shape)


def quantize_per_channel(x: torch.Tensor, axis: int = 0, bits: int = 8) -> QuantizedTensor:
    """Symmetric quantisation with one scale per slice along ``axis``."""
    qmax = 2 ** (bits - 1) - 1
    dims = [d for d in range(x.dim()) if d != axis]
    scale = x.abs().amax(dim=dims).clamp_min(1e-12) / qmax
    shape = [1] * x.dim()
    shape[axis] = -1
    q = torch.round(x / scale.view(shape)).clamp(-qmax, qmax).to(torch.int8)
    return QuantizedTensor(q, scale, torch.zeros_like(scale), axis)


def fake_quantize_qdq(x: torch.Tensor, scale, zero_point=0.0, qmin: float = -128, qmax: float = 127) -> torch.Tensor:
    """Quantise and dequantise in one go (no gradient treatment)."""
    return (torch.clamp(torch.round(x / scale) + zero_point, qmin, qmax) - zero_point) * scale


def fake_quantize_ste(x: torch.Tensor, scale, zero_point=0.0, qmin: float = -128, qmax: float = 127) -> torch.Tensor:
    """The same values as :func:`fake_quantize_qdq`; the gradient passes unchanged inside the representable range and is zero
    outside it (straight-through estimator)."""
    return _FakeQuantSTE.apply(x, torch.as_tensor(scale, dtype=x.dtype), torch.as_tensor(zero_point, dtype=x.dtype), qmin, qmax)


class _Observed(nn.Module):
    """A layer with an observer on its input (what ``prepare`` puts in place of a Linear / Conv2d)."""

    def __init__(self, layer: nn.Module, qconfig: QConfig):
        super().__init__()
        self.layer, self.qconfig = layer, qconfig
        self.observer = MinMaxObserver(qconfig.bits, qconfig.symmetric, qconfig.momentum)

    def forward(self, x):
        return self.layer(self.observer(x))


def prepare(model: nn.Module, qconfig: QConfig = None) -> nn.Module:
    """Wrap every Linear / Conv2d so that calibration batches record the range of its input."""
    qconfig = qconfig or default_qconfig()
    for name, ch in list(model.named_children()):
        if isinstance(ch, (nn.Linear, nn.Conv2d)):
            setattr(model, name, _Observed(ch, qconfig))
        elif not isinstance(ch, _Observed):
            prepare(ch, qconfig)
    return model


@torch.no_grad()
def calibrate(model: nn.Module, batches) -> int:
    """Run the calibration batches through a prepared model; returns how many there were."""
    model.eval()
    n = 0
    for b in batches:
        model(*(b if isinstance(b, (tuple, list)) else (b,)))
        n += 1
    return n


@_dataclass
class QuantizationResult:
    model: nn.Module
    num_quantized: int
    fp32_bytes: int
    int8_bytes: int

    @property
    def compression(self) -> float:
        return self.fp32_bytes / max(self.int8_bytes, 1)


def _convert_prepared(model: nn.Module) -> int:
    n = 0
    for name, ch in list(model.named_children()):
        if isinstance(ch, _Observed):
            layer = ch.layer
            q = QuantizedLinear.from_float(layer) if isinstance(layer, nn.Linear) else QuantizedConv2d(layer)
            scale, zp = ch.observer.qparams()
            q.register_buffer("input_scale", scale.detach().clone())          # the calibrated activation range travels with the layer
            q.register_buffer("input_zero_point", zp.detach().clone())
            setattr(model, name, q)
            n += 1
        else:
            n += _convert_prepared(ch)
    return n


def quantize_model(model: nn.Module, calibration_batches=(), qconfig: QConfig = None) -> QuantizationResult:
    """prepare -> calibrate -> convert: int8 weights per output channel, calibrated input ranges stored on the layers."""
    fp32 = sum(p.numel() * p.element_size() for p in model.parameters())
    prepare(model, qconfig)
    calibrate(model, calibration_batches)
    n = _convert_prepared(model)
    small = sum(b.numel() * b.element_size() for b in model.buffers()) + sum(p.numel() * p.element_size() for p in model.parameters())
    return QuantizationResult(model, n, fp32, small)


# ----------------------------------------------------------------------------- 4-bit blocks under the reference's names (torch/quantization/quant4.h)
@_dataclass
class Int4Block:
    """64 values as 32 packed bytes and one scale: ``value = (nibble - 8) / 7 * absmax``."""
    packed: torch.Tensor
    absmax: torch.Tensor


@_dataclass
class NF4Block:
    """64 values as 32 packed bytes indexing the 16 NormalFloat levels, and one scale."""
    packed: torch.Tensor
    absmax: torch.Tensor


def pack_nibble(lo: torch.Tensor, hi: torch.Tensor) -> torch.Tensor:
    return (lo.to(torch.uint8) & 0xF) | ((hi.to(torch.uint8) & 0xF) << 4)


def dequantize_int4(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = 64) -> torch.Tensor:
    return dequantize_4bit(packed, absmax, shape, block, "int4")


def dequantize_nf4(packed: torch.Tensor, absmax: torch.Tensor, shape, block: int = 64) -> torch.Tensor:
    return dequantize_4bit(packed, absmax, shape, block, "nf4")
