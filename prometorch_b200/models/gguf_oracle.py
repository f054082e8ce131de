"""Plain PyTorch fp32 forward of a GGUF decoder — the end-to-end logits oracle.

Every CUDA decode kernel is checked against this: weights are dequantised once
to fp32 and the forward is ordinary eager PyTorch (RMSNorm, optional per-head
QK RMSNorm, RoPE in NeoX or interleaved pairing, GQA attention over a growing
KV cache, SiLU- or GELU-gated MLP).  It mirrors what the reference's CPU path
computes (torch/io/gguf_model.h:7300-7340 for the layer, :7495-7505 for the
two RoPE conventions), which is also that project's own oracle.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..io.config import TransformerConfig, layer_matrix_sources
from ..io.gguf import GGUFReader
from ..io.gguf_quant import quantize_activation_q8


def rms_norm(x, w, eps, add_one=False):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return v * ((1.0 + w) if add_one else w)


def rope_tables(cfg: TransformerConfig, max_pos: int, device="cpu", freq_base: Optional[float] = None):
    """cos/sin tables ``[max_pos, head_dim/2]`` in fp32 computed in float64."""
    d = cfg.head_dim
    base = float(freq_base if freq_base is not None else cfg.rope_freq_base)
    i = torch.arange(0, d // 2, dtype=torch.float64)
    inv_freq = base ** (-2.0 * i / d)
    mscale = 1.0
    if cfg.rope_yarn and cfg.yarn_factor > 1.0 and cfg.yarn_orig_ctx > 0:
        # YaRN: blend interpolated and extrapolated frequencies between two correction dims
        def corr_dim(n_rot):
            return d * math.log(cfg.yarn_orig_ctx / (n_rot * 2 * math.pi)) / (2 * math.log(base))
        lo = max(math.floor(corr_dim(cfg.yarn_beta_fast)), 0)
        hi = min(math.ceil(corr_dim(cfg.yarn_beta_slow)), d // 2 - 1)
        ramp = ((i - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        mix = 1.0 - ramp
        inv_freq = inv_freq / cfg.yarn_factor * (1 - mix) + inv_freq * mix
        mscale = 0.1 * math.log(cfg.yarn_factor) + 1.0
    elif cfg.rope_scale != 1.0:
        inv_freq = inv_freq / cfg.rope_scale
    factors = cfg.rope_factors_for(max_pos)          # phi-3 LongRoPE: short or long factors by sequence length
    if factors is not None:
        inv_freq = inv_freq / torch.tensor(factors, dtype=torch.float64)
    pos = torch.arange(max_pos, dtype=torch.float64)
    ang = pos[:, None] * inv_freq[None, :]
    m = mscale * cfg.rope_attn_factor
    return (ang.cos() * m).float().to(device), (ang.sin() * m).float().to(device)


def apply_rope(x, cos, sin, neox: bool):
    """x ``[T, heads, d]``; cos/sin ``[T, d/2]``."""
    c, s = cos[:, None, :], sin[:, None, :]
    if neox:
        h = x.shape[-1] // 2
        x1, x2 = x[..., :h], x[..., h:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    x1, x2 = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x1 * c - x2 * s
    out[..., 1::2] = x2 * c + x1 * s
    return out


class OracleModel:
    """fp32 decoder with an explicit KV cache; ``forward(tokens)`` appends to it."""

    def __init__(self, path_or_reader, device="cpu", max_seq: int = 4096, emulate_q8: bool = False):
        r = path_or_reader if isinstance(path_or_reader, GGUFReader) else GGUFReader(path_or_reader)
        self.reader = r
        self.cfg = TransformerConfig.from_gguf(r)
        self.device = device
        self.emulate_q8 = emulate_q8
        cfg = self.cfg
        ld = lambda n: r.load(n, device=device)
        self.tok = ld("token_embd.weight")
        self.out_norm = ld("output_norm.weight")
        self.out = ld("output.weight") if r.has_tensor("output.weight") else self.tok
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"blk.{i}."
            L = {k: ld(p + k + ".weight") for k in ("attn_norm", "ffn_norm")}
            names = {"q": "attn_q", "k": "attn_k", "v": "attn_v", "o": "attn_output", "gate": "ffn_gate", "up": "ffn_up",
                     "down": "ffn_down"}
            for key, (tname, rows) in layer_matrix_sources(r, cfg, i).items():      # merged qkv / gate+up are row ranges
                w = ld(tname)
                L[names[key]] = w if rows is None else w[rows[0]:rows[1]]
            for opt in ("attn_q_norm", "attn_k_norm", "post_attention_norm", "post_ffw_norm"):
                if r.has_tensor(p + opt + ".weight"):
                    L[opt] = ld(p + opt + ".weight")
            for b in ("attn_q", "attn_k", "attn_v"):
                if r.has_tensor(p + b + ".bias"):
                    L[b + "_b"] = ld(p + b + ".bias")
            self.layers.append(L)
        self.cos, self.sin = rope_tables(cfg, max_seq, device)
        self.k_cache: List[Optional[torch.Tensor]] = [None] * cfg.num_layers
        self.v_cache: List[Optional[torch.Tensor]] = [None] * cfg.num_layers
        self.pos = 0

    def reset(self):
        self.k_cache = [None] * self.cfg.num_layers
        self.v_cache = [None] * self.cfg.num_layers
        self.pos = 0

    def _lin(self, x, w):
        if self.emulate_q8:
            x = quantize_activation_q8(x)
        return x @ w.t()

    @torch.no_grad()
    def forward(self, tokens) -> torch.Tensor:
        """Run ``tokens`` (list/1-D tensor) through the model; returns logits ``[T, vocab]``."""
        cfg = self.cfg
        tokens = torch.as_tensor(tokens, dtype=torch.long, device=self.device)
        T = tokens.numel()
        x = self.tok[tokens]
        if cfg.scale_embeddings:
            x = x * math.sqrt(cfg.hidden_size)
        cos_g, sin_g = self.cos[self.pos:self.pos + T], self.sin[self.pos:self.pos + T]
        cos_l = sin_l = None
        if cfg.swa_window and cfg.rope_swa_freq_base != cfg.rope_freq_base:
            if not hasattr(self, "_swa_tables"):
                self._swa_tables = rope_tables(cfg, self.cos.shape[0], self.device, freq_base=cfg.rope_swa_freq_base)
            cos_l, sin_l = self._swa_tables[0][self.pos:self.pos + T], self._swa_tables[1][self.pos:self.pos + T]
        group = cfg.num_heads // cfg.num_kv_heads
        for li, L in enumerate(self.layers):
            # sliding-window layers (all but every swa_pattern-th): local RoPE base and a window over the keys
            swa = bool(cfg.swa_window and cfg.swa_pattern and (li + 1) % cfg.swa_pattern != 0)
            cos, sin = (cos_l, sin_l) if (swa and cos_l is not None) else (cos_g, sin_g)
            h = rms_norm(x, L["attn_norm"], cfg.rms_norm_eps, cfg.gemma_norm_add_one)
            q, k, v = self._lin(h, L["attn_q"]), self._lin(h, L["attn_k"]), self._lin(h, L["attn_v"])
            if "attn_q_b" in L:
                q, k, v = q + L["attn_q_b"], k + L["attn_k_b"], v + L["attn_v_b"]
            q = q.view(T, cfg.num_heads, cfg.head_dim)
            k = k.view(T, cfg.num_kv_heads, cfg.head_dim)
            v = v.view(T, cfg.num_kv_heads, cfg.head_dim)
            if "attn_q_norm" in L:
                q = rms_norm(q, L["attn_q_norm"], cfg.rms_norm_eps)
                k = rms_norm(k, L["attn_k_norm"], cfg.rms_norm_eps)
            q = apply_rope(q, cos, sin, cfg.rope_neox)
            k = apply_rope(k, cos, sin, cfg.rope_neox)
            # the decode engine keeps K/V in fp16
            k, v = k.half().float(), v.half().float()
            self.k_cache[li] = k if self.k_cache[li] is None else torch.cat([self.k_cache[li], k], 0)
            self.v_cache[li] = v if self.v_cache[li] is None else torch.cat([self.v_cache[li], v], 0)
            K, Vc = self.k_cache[li], self.v_cache[li]
            S = K.shape[0]
            Kh = K.repeat_interleave(group, dim=1).permute(1, 0, 2)       # [H, S, d]
            Vh = Vc.repeat_interleave(group, dim=1).permute(1, 0, 2)
            sc = torch.einsum("thd,hsd->hts", q, Kh) / math.sqrt(cfg.head_dim)
            qpos = torch.arange(self.pos, self.pos + T, device=self.device)[:, None]
            kpos = torch.arange(S, device=self.device)[None, :]
            hidden = kpos > qpos
            if swa:
                hidden = hidden | (kpos <= qpos - cfg.swa_window)         # a query sees the last `window` positions
            sc = sc.masked_fill(hidden[None], float("-inf"))
            a = torch.einsum("hts,hsd->thd", sc.softmax(-1), Vh).reshape(T, cfg.q_dim)
            o = self._lin(a, L["attn_output"])
            if "post_attention_norm" in L:
                o = rms_norm(o, L["post_attention_norm"], cfg.rms_norm_eps)
            x = x + o
            h = rms_norm(x, L["ffn_norm"], cfg.rms_norm_eps, cfg.gemma_norm_add_one)
            g, u = self._lin(h, L["ffn_gate"]), self._lin(h, L["ffn_up"])
            act = F.gelu(g, approximate="tanh") if cfg.ffn_gelu else F.silu(g)
            dn = self._lin(act * u, L["ffn_down"])
            if "post_ffw_norm" in L:
                dn = rms_norm(dn, L["post_ffw_norm"], cfg.rms_norm_eps)
            x = x + dn
        self.pos += T
        x = rms_norm(x, self.out_norm, cfg.rms_norm_eps, cfg.gemma_norm_add_one)
        return self._lin(x, self.out)

    @torch.no_grad()
    def generate_greedy(self, prompt, n_new: int):
        self.reset()
        logits = self.forward(prompt)
        out = []
        for _ in range(n_new):
            t = int(logits[-1].argmax())
            out.append(t)
            logits = self.forward([t])
        return out


class TPOracleModel(OracleModel):
    """The oracle cut for tensor parallelism with the partition rule of the decode engine (io/gguf_model.py): rank r holds the
    query heads ``[r H/W, (r+1) H/W)`` with their KV heads, the FFN columns of its share of 256-wide blocks (``split_blocks``: the
    first ``blocks % W`` ranks take one more), the matching input columns of the attention-output and FFN-down projections, and
    rows ``[V r / W, V (r+1) / W)`` of the output head.  The two partial sums per layer are all-reduced over the process group
    and the logits are all-gathered, which is what the reference's CPU tensor-parallel decode does
    (torch/io/gguf_model.h:6197-6225, 6442, 6512).  Runs on CPU ranks (gloo); checked against the single-process oracle."""

    def __init__(self, path_or_reader, tp_rank: int, tp_world: int, group=None, max_seq: int = 4096):
        super().__init__(path_or_reader, device="cpu", max_seq=max_seq)
        from ..io.gguf_model import split_blocks
        cfg, W, rk = self.cfg, tp_world, tp_rank
        if cfg.num_heads % W or cfg.num_kv_heads % W or cfg.intermediate_size % 256:
            raise ValueError(f"tensor parallel {W}: needs heads ({cfg.num_heads}) and KV heads ({cfg.num_kv_heads}) divisible "
                             f"and an FFN size ({cfg.intermediate_size}) that is a multiple of 256")
        self.tp_rank, self.tp_world, self.group = rk, W, group
        d = cfg.head_dim
        self.hq, self.hkv = cfg.num_heads // W, cfg.num_kv_heads // W
        fb0, fb1 = split_blocks(cfg.intermediate_size // 256, W, rk)
        q0, q1 = rk * self.hq * d, (rk + 1) * self.hq * d
        k0, k1 = rk * self.hkv * d, (rk + 1) * self.hkv * d
        f0, f1 = fb0 * 256, fb1 * 256
        for L in self.layers:
            L["attn_q"], L["attn_k"], L["attn_v"] = L["attn_q"][q0:q1], L["attn_k"][k0:k1], L["attn_v"][k0:k1]
            L["attn_output"] = L["attn_output"][:, q0:q1]
            L["ffn_gate"], L["ffn_up"], L["ffn_down"] = L["ffn_gate"][f0:f1], L["ffn_up"][f0:f1], L["ffn_down"][:, f0:f1]
            for b, (lo, hi) in (("attn_q_b", (q0, q1)), ("attn_k_b", (k0, k1)), ("attn_v_b", (k0, k1))):
                if b in L:
                    L[b] = L[b][lo:hi]
        V = cfg.vocab_size
        self.v0, self.v1 = V * rk // W, V * (rk + 1) // W
        self.out = self.out[self.v0:self.v1]
        self.local_inter = f1 - f0

    def _allreduce(self, t):
        if self.tp_world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=self.group)
        return t

    @torch.no_grad()
    def forward(self, tokens) -> torch.Tensor:
        cfg = self.cfg
        tokens = torch.as_tensor(tokens, dtype=torch.long)
        T = tokens.numel()
        x = self.tok[tokens]
        if cfg.scale_embeddings:
            x = x * math.sqrt(cfg.hidden_size)
        cos, sin = self.cos[self.pos:self.pos + T], self.sin[self.pos:self.pos + T]
        group = self.hq // self.hkv
        for li, L in enumerate(self.layers):
            h = rms_norm(x, L["attn_norm"], cfg.rms_norm_eps, cfg.gemma_norm_add_one)
            q, k, v = h @ L["attn_q"].t(), h @ L["attn_k"].t(), h @ L["attn_v"].t()
            if "attn_q_b" in L:
                q, k, v = q + L["attn_q_b"], k + L["attn_k_b"], v + L["attn_v_b"]
            q, k, v = q.view(T, self.hq, cfg.head_dim), k.view(T, self.hkv, cfg.head_dim), v.view(T, self.hkv, cfg.head_dim)
            if "attn_q_norm" in L:
                q, k = rms_norm(q, L["attn_q_norm"], cfg.rms_norm_eps), rms_norm(k, L["attn_k_norm"], cfg.rms_norm_eps)
            q, k = apply_rope(q, cos, sin, cfg.rope_neox), apply_rope(k, cos, sin, cfg.rope_neox)
            k, v = k.half().float(), v.half().float()
            self.k_cache[li] = k if self.k_cache[li] is None else torch.cat([self.k_cache[li], k], 0)
            self.v_cache[li] = v if self.v_cache[li] is None else torch.cat([self.v_cache[li], v], 0)
            K, Vc = self.k_cache[li], self.v_cache[li]
            S = K.shape[0]
            Kh, Vh = K.repeat_interleave(group, dim=1).permute(1, 0, 2), Vc.repeat_interleave(group, dim=1).permute(1, 0, 2)
            sc = torch.einsum("thd,hsd->hts", q, Kh) / math.sqrt(cfg.head_dim)
            qpos, kpos = torch.arange(self.pos, self.pos + T)[:, None], torch.arange(S)[None, :]
            sc = sc.masked_fill((kpos > qpos)[None], float("-inf"))
            a = torch.einsum("hts,hsd->thd", sc.softmax(-1), Vh).reshape(T, self.hq * cfg.head_dim)
            x = x + self._allreduce(a @ L["attn_output"].t())                 # partial sums over this rank's heads
            h = rms_norm(x, L["ffn_norm"], cfg.rms_norm_eps, cfg.gemma_norm_add_one)
            g, u = h @ L["ffn_gate"].t(), h @ L["ffn_up"].t()
            act = F.gelu(g, approximate="tanh") if cfg.ffn_gelu else F.silu(g)
            x = x + self._allreduce((act * u) @ L["ffn_down"].t())             # partial sums over this rank's FFN columns
        self.pos += T
        x = rms_norm(x, self.out_norm, cfg.rms_norm_eps, cfg.gemma_norm_add_one)
        local = x @ self.out.t()                                               # this rank's rows of the vocabulary
        if self.tp_world == 1:
            return local
        import torch.distributed as dist
        V, W = cfg.vocab_size, self.tp_world
        sizes = [V * (r + 1) // W - V * r // W for r in range(W)]
        pad = max(sizes)
        buf = torch.zeros(T, pad)
        buf[:, :local.shape[1]] = local
        parts = [torch.zeros(T, pad) for _ in range(W)]
        dist.all_gather(parts, buf, group=self.group)
        return torch.cat([p[:, :n] for p, n in zip(parts, sizes)], dim=1)
