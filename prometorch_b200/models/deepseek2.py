"""deepseek2 decoders (DeepSeek-V2/V3, GigaChat3): multi-head latent attention and a mixture-of-experts FFN.

What the reference decodes on the CPU one token at a time with per-head loops and a materialised K/V cache
(torch/io/deepseek2_forward.h:117-395 ``mla_attention_forward_decode``, :397-520 ``moe_ffn_forward_decode``) runs
here as batched tensor programs on any device, for any number of tokens per call, with two changes of design:

* the cache holds the *latent*: per token the normalised ``kv_lora_rank`` vector and the rotated shared rope key
  (``kv_lora_rank + rope_dim`` values, 576 for GigaChat3) instead of ``heads x (key_length + value_length)`` values
  (14336 there).  The K up-projection is folded into the query (``q_abs[h] = W_kb[h] q_nope[h]``) and the V
  up-projection is applied to the attention-weighted latent, which gives the same numbers as materialising K and V;
* routed experts are evaluated grouped by expert over all tokens of the call, not token by token.

Semantics kept from the reference: NeoX-style rotation of the rope part, YaRN frequency blend with the rope
``mscale = 1 + log_multiplier * ln(factor)``, attention scale ``kq_mscale^2 / sqrt(key_length)`` with
``kq_mscale = (1 + 0.1 ln f)(1 + 0.1 log_multiplier ln f)``, sigmoid router scores, top-k, weights normalised to sum 1,
shared experts always on, the first ``leading_dense_block_count`` layers dense.

Tensor names (llama.cpp's deepseek2 conversion): ``attn_q`` (or ``attn_q_a`` / ``attn_q_a_norm`` / ``attn_q_b``),
``attn_kv_a_mqa``, ``attn_kv_a_norm``, ``attn_k_b`` ``[heads, kv_lora, qk_nope]``, ``attn_v_b`` ``[heads, v, kv_lora]``,
``attn_output``; ``ffn_gate_inp`` (router), ``ffn_{gate,up,down}_exps`` ``[experts, ...]``, ``ffn_{gate,up,down}_shexp``,
optional ``exp_probs_b`` (selection bias).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..io.gguf import GGUFReader


@dataclass
class DeepSeek2Config:
    vocab_size: int = 0
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    intermediate_size: int = 0
    kv_lora_rank: int = 0
    q_lora_rank: int = 0
    key_length: int = 0            # per head: qk_nope + rope (attention.key_length_mla)
    value_length: int = 0          # per head (attention.value_length_mla)
    rope_dim: int = 0
    expert_count: int = 0
    expert_used_count: int = 0
    expert_shared_count: int = 0
    expert_ff: int = 0
    leading_dense: int = 0
    expert_weights_scale: float = 1.0
    expert_weights_norm: bool = True
    expert_gating_sigmoid: bool = True
    rms_norm_eps: float = 1e-6
    rope_freq_base: float = 10000.0
    rope_yarn: bool = False
    yarn_factor: float = 1.0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_orig_ctx: int = 0
    yarn_log_multiplier: float = 0.0
    context_length: int = 4096
    eos_token_id: int = -1

    @property
    def qk_nope(self) -> int:
        return self.key_length - self.rope_dim

    @classmethod
    def from_gguf(cls, r: GGUFReader) -> "DeepSeek2Config":
        g = r.get_arch
        c = cls()
        c.hidden_size = int(g("embedding_length", 0))
        c.num_layers = int(g("block_count", 0))
        c.num_heads = int(g("attention.head_count", 0))
        c.intermediate_size = int(g("feed_forward_length", 0))
        c.kv_lora_rank = int(g("attention.kv_lora_rank", 0))
        c.q_lora_rank = int(g("attention.q_lora_rank", 0))
        c.key_length = int(g("attention.key_length_mla", 0))
        c.value_length = int(g("attention.value_length_mla", 0))
        # attention.key_length is the latent row: kv_lora_rank + rope part (the reference derives rope_dim that way too)
        klen = int(g("attention.key_length", 0))
        c.rope_dim = int(g("rope.dimension_count", klen - c.kv_lora_rank if klen > c.kv_lora_rank else 0))
        c.expert_count = int(g("expert_count", 0))
        c.expert_used_count = int(g("expert_used_count", 0))
        c.expert_shared_count = int(g("expert_shared_count", 0))
        c.expert_ff = int(g("expert_feed_forward_length", 0))
        c.leading_dense = int(g("leading_dense_block_count", 0))
        c.expert_weights_scale = float(g("expert_weights_scale", 1.0))
        c.expert_weights_norm = bool(g("expert_weights_norm", True))
        c.expert_gating_sigmoid = int(g("expert_gating_func", 2)) != 1          # 1 = softmax, 2 = sigmoid
        c.rms_norm_eps = float(g("attention.layer_norm_rms_epsilon", 1e-6))
        c.rope_freq_base = float(g("rope.freq_base", 10000.0))
        c.context_length = int(g("context_length", 4096))
        if g("rope.scaling.type", "") == "yarn":
            c.rope_yarn = True
            c.yarn_factor = float(g("rope.scaling.factor", 1.0))
            c.yarn_beta_fast = float(g("rope.scaling.yarn_beta_fast", 32.0))
            c.yarn_beta_slow = float(g("rope.scaling.yarn_beta_slow", 1.0))
            c.yarn_orig_ctx = int(g("rope.scaling.original_context_length", 0))
            c.yarn_log_multiplier = float(g("rope.scaling.yarn_log_multiplier", 0.0))
        c.vocab_size = int(r.tensors["token_embd.weight"].shape[0])
        c.eos_token_id = int(r.get("tokenizer.ggml.eos_token_id", -1))
        if not (c.kv_lora_rank and c.key_length and c.value_length and c.rope_dim):
            raise ValueError("not a deepseek2 file: kv_lora_rank / key_length_mla / value_length_mla / rope dimension missing")
        return c


def yarn_rope_tables(cfg: DeepSeek2Config, max_pos: int, device="cpu"):
    """cos/sin ``[max_pos, rope_dim/2]``: plain RoPE, or YaRN's blend of extrapolated (low index, high frequency) and
    interpolated (high index) frequencies over the ramp between the two correction dimensions, times the rope mscale."""
    d = cfg.rope_dim
    i = torch.arange(d // 2, dtype=torch.float64)
    inv = cfg.rope_freq_base ** (-2.0 * i / d)
    mscale = 1.0
    if cfg.rope_yarn and cfg.yarn_orig_ctx > 0:
        f = cfg.yarn_factor
        if cfg.yarn_log_multiplier > 0 and f > 1:
            mscale = 1.0 + cfg.yarn_log_multiplier * math.log(f)

        def find_dim(beta):
            return d * math.log(cfg.yarn_orig_ctx / (2 * math.pi * beta)) / (2 * math.log(cfg.rope_freq_base))
        lo = max(math.floor(find_dim(cfg.yarn_beta_fast)), 0.0)
        hi = min(math.ceil(find_dim(cfg.yarn_beta_slow)), d // 2 - 1)
        if hi - lo < 0.001:
            hi = lo + 0.001
        mask = ((i - lo) / (hi - lo)).clamp(0, 1)
        inv = inv / f * mask + inv * (1 - mask)
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return (ang.cos() * mscale).float().to(device), (ang.sin() * mscale).float().to(device)


def _rms(x, w, eps):
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope_neox(x, cos, sin):
    """x ``[T, ..., rope_dim]``, cos/sin ``[T, rope_dim/2]`` broadcast over the middle dims."""
    h = x.shape[-1] // 2
    while cos.dim() < x.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


class DeepSeek2Model:
    """Decoder with a latent KV cache.  ``forward(tokens)`` appends to the cache and returns logits ``[T, vocab]``."""

    def __init__(self, path_or_reader, device="cpu", max_seq: int = 4096, dtype=torch.float32):
        r = path_or_reader if isinstance(path_or_reader, GGUFReader) else GGUFReader(path_or_reader)
        if r.arch() != "deepseek2":
            raise ValueError(f"architecture {r.arch()!r} is not deepseek2")
        self.reader, self.device, self.dtype = r, torch.device(device), dtype
        self.cfg = cfg = DeepSeek2Config.from_gguf(r)
        self.max_seq = int(min(max_seq, cfg.context_length))

        def ld(n, dt=dtype):
            return r.load(n, device=device).to(dt)

        def opt(n, dt=dtype):
            return ld(n, dt) if r.has_tensor(n) else None
        self.tok = ld("token_embd.weight")
        self.out_norm = ld("output_norm.weight", torch.float32)
        self.out = ld("output.weight") if r.has_tensor("output.weight") else self.tok
        self.layers: List[dict] = []
        for i in range(cfg.num_layers):
            p = f"blk.{i}."
            L = dict(attn_norm=ld(p + "attn_norm.weight", torch.float32), ffn_norm=ld(p + "ffn_norm.weight", torch.float32),
                     kv_a=ld(p + "attn_kv_a_mqa.weight"), kv_a_norm=ld(p + "attn_kv_a_norm.weight", torch.float32),
                     k_b=ld(p + "attn_k_b.weight"), v_b=ld(p + "attn_v_b.weight"), o=ld(p + "attn_output.weight"))
            if r.has_tensor(p + "attn_q.weight"):
                L["q"] = ld(p + "attn_q.weight")
            else:
                L.update(q_a=ld(p + "attn_q_a.weight"), q_a_norm=ld(p + "attn_q_a_norm.weight", torch.float32),
                         q_b=ld(p + "attn_q_b.weight"))
            if i < cfg.leading_dense or cfg.expert_count == 0:
                L.update(gate=ld(p + "ffn_gate.weight"), up=ld(p + "ffn_up.weight"), down=ld(p + "ffn_down.weight"))
            else:
                L.update(router=ld(p + "ffn_gate_inp.weight", torch.float32), gate_exps=ld(p + "ffn_gate_exps.weight"),
                         up_exps=ld(p + "ffn_up_exps.weight"), down_exps=ld(p + "ffn_down_exps.weight"),
                         probs_b=opt(p + "exp_probs_b.bias", torch.float32), gate_sh=opt(p + "ffn_gate_shexp.weight"),
                         up_sh=opt(p + "ffn_up_shexp.weight"), down_sh=opt(p + "ffn_down_shexp.weight"))
            self.layers.append(L)
        self.cos, self.sin = yarn_rope_tables(cfg, self.max_seq, device)
        kq = 1.0
        if cfg.rope_yarn and cfg.yarn_factor > 1.0:
            lf = math.log(cfg.yarn_factor)
            kq = (1.0 + 0.1 * lf) * (1.0 + 0.1 * cfg.yarn_log_multiplier * lf)
        self.scale = kq * kq / math.sqrt(cfg.key_length)
        # latent cache per layer: [max_seq, kv_lora_rank] normalised latents and [max_seq, rope_dim] rotated rope keys
        self.lat = [torch.zeros(self.max_seq, cfg.kv_lora_rank, dtype=torch.float32, device=device) for _ in self.layers]
        self.kpe = [torch.zeros(self.max_seq, cfg.rope_dim, dtype=torch.float32, device=device) for _ in self.layers]
        self.pos = 0

    def reset(self):
        self.pos = 0

    @property
    def cache_bytes_per_token(self) -> int:
        return 4 * self.cfg.num_layers * (self.cfg.kv_lora_rank + self.cfg.rope_dim)

    # ------------------------------------------------------------------ attention
    def _attention(self, li: int, L: dict, h: torch.Tensor, pos0: int) -> torch.Tensor:
        cfg = self.cfg
        T, nh, nope, rope, kvl, vd = h.shape[0], cfg.num_heads, cfg.qk_nope, cfg.rope_dim, cfg.kv_lora_rank, cfg.value_length
        hd = h.to(self.dtype)
        if "q" in L:
            q = hd @ L["q"].t()
        else:
            q = _rms(hd @ L["q_a"].t(), L["q_a_norm"], cfg.rms_norm_eps).to(self.dtype) @ L["q_b"].t()
        q = q.float().view(T, nh, cfg.key_length)
        kv = (hd @ L["kv_a"].t()).float()                                   # [T, kv_lora + rope]
        cos, sin = self.cos[pos0:pos0 + T], self.sin[pos0:pos0 + T]
        self.lat[li][pos0:pos0 + T] = _rms(kv[:, :kvl], L["kv_a_norm"], cfg.rms_norm_eps)
        self.kpe[li][pos0:pos0 + T] = _rope_neox(kv[:, kvl:], cos, sin)
        q_nope, q_pe = q[..., :nope], _rope_neox(q[..., nope:], cos, sin)
        S = pos0 + T
        lat, kpe = self.lat[li][:S], self.kpe[li][:S]
        # fold the K up-projection into the query: q_abs[t, h, r] = sum_c k_b[h, r, c] q_nope[t, h, c]
        q_abs = torch.einsum("hrc,thc->thr", L["k_b"].float(), q_nope)
        sc = (torch.einsum("thr,sr->hts", q_abs, lat) + torch.einsum("thd,sd->hts", q_pe, kpe)) * self.scale
        qpos = torch.arange(pos0, S, device=h.device)[:, None]
        sc = sc.masked_fill((torch.arange(S, device=h.device)[None, :] > qpos)[None], float("-inf"))
        ctx = torch.einsum("hts,sr->thr", sc.softmax(-1), lat)              # attention-weighted latent
        out = torch.einsum("hdr,thr->thd", L["v_b"].float(), ctx).reshape(T, nh * vd)
        return (out.to(self.dtype) @ L["o"].t()).float()

    # ------------------------------------------------------------------ FFN
    @staticmethod
    def _glu(x, gate, up, down):
        return (F.silu(x @ gate.t()) * (x @ up.t())) @ down.t()

    def _moe(self, L: dict, h: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        T = h.shape[0]
        logits = h.float() @ L["router"].t()                                # [T, E]
        scores = torch.sigmoid(logits) if cfg.expert_gating_sigmoid else logits.softmax(-1)
        pick = scores if L["probs_b"] is None else scores + L["probs_b"]   # the bias steers selection only
        idx = pick.topk(cfg.expert_used_count, dim=-1).indices              # [T, K]
        w = scores.gather(1, idx)
        if cfg.expert_weights_norm:
            w = w / w.sum(-1, keepdim=True).clamp_min(1e-20)
        w = w * cfg.expert_weights_scale
        hd = h.to(self.dtype)
        out = torch.zeros(T, cfg.hidden_size, dtype=torch.float32, device=h.device)
        flat_e, flat_t = idx.reshape(-1), torch.arange(T, device=h.device).repeat_interleave(cfg.expert_used_count)
        flat_w = w.reshape(-1)
        for e in flat_e.unique().tolist():                                  # grouped by expert over all tokens of the call
            sel = flat_e == e
            t_ids = flat_t[sel]
            y = self._glu(hd[t_ids], L["gate_exps"][e], L["up_exps"][e], L["down_exps"][e]).float()
            out.index_add_(0, t_ids, y * flat_w[sel][:, None])
        if L["gate_sh"] is not None:
            out = out + self._glu(hd, L["gate_sh"], L["up_sh"], L["down_sh"]).float()
        return out

    # ------------------------------------------------------------------ model
    @torch.no_grad()
    def forward(self, tokens) -> torch.Tensor:
        cfg = self.cfg
        tokens = torch.as_tensor(tokens, dtype=torch.long, device=self.device).reshape(-1)
        T, pos0 = tokens.numel(), self.pos
        if pos0 + T > self.max_seq:
            raise ValueError(f"{pos0 + T} positions exceed max_seq {self.max_seq}")
        x = self.tok[tokens].float()
        for li, L in enumerate(self.layers):
            x = x + self._attention(li, L, _rms(x, L["attn_norm"], cfg.rms_norm_eps), pos0)
            h = _rms(x, L["ffn_norm"], cfg.rms_norm_eps)
            if "router" in L:
                x = x + self._moe(L, h)
            else:
                x = x + self._glu(h.to(self.dtype), L["gate"], L["up"], L["down"]).float()
        self.pos += T
        return (_rms(x, self.out_norm, cfg.rms_norm_eps).to(self.dtype) @ self.out.t()).float()

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int = 32, stop_ids=()) -> List[int]:
        """Greedy generation: one batched pass over the prompt, then one token per step."""
        self.reset()
        stop = set(int(s) for s in stop_ids)
        if self.cfg.eos_token_id >= 0:
            stop.add(self.cfg.eos_token_id)
        logits = self.forward(prompt)
        out: List[int] = []
        for _ in range(max_new_tokens):
            t = int(logits[-1].argmax())
            if t in stop:
                break
            out.append(t)
            logits = self.forward([t])
        return out
