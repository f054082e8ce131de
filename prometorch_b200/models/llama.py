"""Llama-style decoder for training (the 1.1B FSDP and 7B TP x PP benchmark shapes).

Pre-RMSNorm blocks: fused residual-add + RMSNorm, one QKV GEMM, RoPE, causal GQA FlashAttention,
output GEMM, gated MLP with packed gate/up GEMM, fused softmax-cross-entropy on the logits.  Every
GEMM is the tcgen05 kernel when the module is bf16 on CUDA.  ``LlamaConfig`` presets name the
shapes used by the benchmark configs."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from ..nn.fused import FlashSelfAttention, FusedCrossEntropyLoss, FusedLinear, FusedRMSNorm, FusedSwiGLU


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    num_layers: int = 22
    num_heads: int = 32
    num_kv_heads: int = 4
    intermediate_size: int = 5632
    max_seq: int = 2048
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = False

    @classmethod
    def llama_1b(cls):          # 22 layers, 2048 hidden, 32q/4kv heads, FFN 5632 (~1.1 B parameters)
        return cls()

    @classmethod
    def llama2_7b(cls):
        return cls(hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=32, intermediate_size=11008, max_seq=4096)

    @classmethod
    def tiny(cls, **kw):
        d = dict(vocab_size=512, hidden_size=128, num_layers=2, num_heads=2, num_kv_heads=1, intermediate_size=256, max_seq=128)
        d.update(kw)
        return cls(**d)


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.attn_norm = FusedRMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.attn = FlashSelfAttention(cfg.hidden_size, cfg.num_heads, cfg.num_kv_heads, rope_theta=cfg.rope_theta,
                                       max_seq=cfg.max_seq, neox=True)
        self.mlp_norm = FusedRMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.mlp = FusedSwiGLU(cfg.hidden_size, cfg.intermediate_size)

    def forward(self, x, delta=None):
        """``x``: the residual stream; ``delta``: the previous block's MLP output, not yet added.  Every residual
        add is fused into the RMSNorm that follows it (one kernel reads both, writes the sum and the normalised
        row); returns the updated stream and this block's pending MLP output."""
        if delta is None:
            h = self.attn_norm(x)
        else:
            h, x = self.attn_norm(delta, x)
        h, x = self.mlp_norm(self.attn(h), x)
        return x, self.mlp(h)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.blocks = nn.ModuleList(LlamaBlock(cfg) for _ in range(cfg.num_layers))
        self.norm = FusedRMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.lm_head = FusedLinear(cfg.hidden_size, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.embed.weight
        self.loss_fn = FusedCrossEntropyLoss()
        self.apply(self._init)

    def _init(self, m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=self.cfg.init_std)
            if getattr(m, "bias", None) is not None:
                nn.init.zeros_(m.bias)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        x, delta = self.embed(tokens), None
        for blk in self.blocks:
            x, delta = blk(x, delta)
        h = self.norm(x) if delta is None else self.norm(delta, x)[0]
        logits = self.lm_head(h)
        if targets is None:
            return logits
        return self.loss_fn(logits.view(-1, logits.shape[-1]), targets.reshape(-1))

    def num_parameters(self):
        return sum(p.numel() for p in self.parameters())
