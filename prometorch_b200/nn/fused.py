"""Modules built on the hand-written sm_100a kernels.  On CPU tensors each falls back to the same
math in tensor ops, so models built from them also run (and are tested) without a GPU."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import fused_ops as K
from ..ops.gemm import linear as fused_linear


class FusedLinear(nn.Linear):
    """``nn.Linear`` whose bf16 CUDA path is the tcgen05 GEMM (forward and both backward products)."""

    def forward(self, x):
        return fused_linear(x, self.weight, self.bias)


class FusedRMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.eps = eps

    def forward(self, x, residual: Optional[torch.Tensor] = None):
        if residual is None:
            return K.rms_norm(x, self.weight, self.eps)
        return K.add_rms_norm(x, residual, self.weight, self.eps)

    def extra_repr(self):
        return f"{self.weight.numel()}, eps={self.eps}"


class FusedSwiGLU(nn.Module):
    """Gated MLP: ``down(act(gate(x)) * up(x))`` with gate and up stored as one ``[2*I, H]`` weight so a
    single GEMM produces both halves and one kernel applies the activation."""

    def __init__(self, hidden_size: int, intermediate_size: int, gelu: bool = False, bias: bool = False):
        super().__init__()
        self.gate_up = FusedLinear(hidden_size, 2 * intermediate_size, bias=bias)
        self.down = FusedLinear(intermediate_size, hidden_size, bias=bias)
        self.gelu = gelu

    def forward(self, x):
        return self.down(K.swiglu(self.gate_up(x), self.gelu))


class FusedCrossEntropyLoss(nn.Module):
    def __init__(self, ignore_index: int = -100, inplace_grad: bool = False):
        super().__init__()
        self.ignore_index, self.inplace_grad = ignore_index, inplace_grad

    def forward(self, logits, target):
        return K.cross_entropy(logits, target, self.ignore_index, self.inplace_grad)


class FlashSelfAttention(nn.Module):
    """Causal self-attention with grouped-query heads and rotary embedding.  Projections are fused
    (``qkv`` in one GEMM); the attention core is :func:`prometorch_b200.ops.attention.flash_attention`."""

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None,
                 rope_theta: float = 10000.0, max_seq: int = 4096, neox: bool = True, bias: bool = False, causal: bool = True,
                 use_rope: bool = True):
        super().__init__()
        self.h, self.kv = num_heads, num_kv_heads or num_heads
        self.d = head_dim or hidden_size // num_heads
        self.neox, self.causal, self.use_rope = neox, causal, use_rope
        self.qkv = FusedLinear(hidden_size, (self.h + 2 * self.kv) * self.d, bias=bias)
        self.out = FusedLinear(self.h * self.d, hidden_size, bias=bias)
        if use_rope:
            inv = rope_theta ** (-torch.arange(0, self.d, 2, dtype=torch.float64) / self.d)
            ang = torch.arange(max_seq, dtype=torch.float64)[:, None] * inv[None]
            self.register_buffer("cos", ang.cos().float(), persistent=False)
            self.register_buffer("sin", ang.sin().float(), persistent=False)

    def forward(self, x, pos_offset: int = 0):
        from ..ops.attention import flash_attention
        B, T, _ = x.shape
        if self.use_rope:
            q, k, v = K.qkv_rope_split(self.qkv(x), self.h, self.kv, self.d, self.cos, self.sin, self.neox, pos_offset)
        else:
            qkv = self.qkv(x).view(B, T, self.h + 2 * self.kv, self.d)
            q, k, v = qkv[:, :, :self.h], qkv[:, :, self.h:self.h + self.kv], qkv[:, :, self.h + self.kv:]
        o = flash_attention(q, k, v, causal=self.causal)
        return self.out(o.reshape(B, T, self.h * self.d))
