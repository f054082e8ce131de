"""Character-level GPT of the DDP benchmark config: pre-LayerNorm blocks, GELU MLP (4x), learned
positions, weight-tied embedding/unembedding.  6 layers, d_model 384, 6 heads, context 256, vocab 65."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..nn.fused import FusedCrossEntropyLoss, FusedLinear
from ..ops.attention import flash_attention


@dataclass
class GPTConfig:
    vocab_size: int = 65
    block_size: int = 256
    n_layer: int = 6
    n_head: int = 6
    n_embd: int = 384
    dropout: float = 0.0


class GPTBlock(nn.Module):
    def __init__(self, c: GPTConfig):
        super().__init__()
        self.ln1, self.ln2 = nn.LayerNorm(c.n_embd), nn.LayerNorm(c.n_embd)
        self.qkv = FusedLinear(c.n_embd, 3 * c.n_embd)
        self.proj = FusedLinear(c.n_embd, c.n_embd)
        self.fc = FusedLinear(c.n_embd, 4 * c.n_embd)
        self.fc2 = FusedLinear(4 * c.n_embd, c.n_embd)
        self.n_head = c.n_head
        self.drop = nn.Dropout(c.dropout)

    def forward(self, x):
        B, T, Cc = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.n_head, Cc // self.n_head).unbind(2)
        a = flash_attention(q, k, v, causal=True).reshape(B, T, Cc)
        x = x + self.drop(self.proj(a))
        return x + self.drop(self.fc2(F.gelu(self.fc(self.ln2(x)), approximate="tanh")))


class CharGPT(nn.Module):
    def __init__(self, c: GPTConfig = GPTConfig()):
        super().__init__()
        self.cfg = c
        self.wte = nn.Embedding(c.vocab_size, c.n_embd)
        self.wpe = nn.Embedding(c.block_size, c.n_embd)
        self.blocks = nn.ModuleList(GPTBlock(c) for _ in range(c.n_layer))
        self.ln_f = nn.LayerNorm(c.n_embd)
        self.loss_fn = FusedCrossEntropyLoss()
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, std=0.02)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, idx, targets: Optional[torch.Tensor] = None):
        B, T = idx.shape
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)        # tied unembedding (vocab 65: too narrow for a 128-wide MMA tile)
        if targets is None:
            return logits
        return self.loss_fn(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))
