"""Load Hugging Face checkpoints without the ``transformers`` package.

    from prometorch_b200.transformers_compat import AutoModel, AutoTokenizer
    model = AutoModel.from_pretrained("./my_hf_model_dir", device="cuda", dtype=torch.bfloat16)
    hidden = model(input_ids)                       # [batch, tokens, hidden]

What a directory needs: ``config.json``; ``model.safetensors`` (or its sharded index, or ``pytorch_model.bin``);
``tokenizer.json`` (or ``vocab.json`` + ``merges.txt``, or ``vocab.txt``).  Supported architectures, as in the
reference's shim (python/promethorch/transformers_compat.py:406-690): ``BertModel`` (post-LN encoder, learned positions,
GELU), ``GPT2Model`` (pre-LN decoder, learned positions, ``Conv1D`` weights stored ``[in, out]``), ``LlamaModel``
(RoPE, RMSNorm, SwiGLU, grouped-query attention).  The reference runs these through numpy round trips; here they are
``torch.nn.Module``s whose linear layers, norms and attention go to the sm_100a kernels when the tensors are CUDA bf16
(tcgen05 GEMM, fused RMSNorm, FlashAttention) and to plain torch ops otherwise.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .io.safetensors import load_checkpoint_dir


# ------------------------------------------------------------------------------------------ helpers
def _linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16:
        from .ops.gemm import linear
        return linear(x, w, b)
    return F.linear(x, w, b)


def _attention(q, k, v, causal: bool) -> torch.Tensor:
    """q [B, T, H, D], k / v [B, T, Hk, D] -> [B, T, H, D]."""
    from .ops.attention import flash_attention
    return flash_attention(q, k, v, causal=causal)


def _strip_prefix(sd: Dict[str, torch.Tensor], prefixes) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        for p in prefixes:
            if k.startswith(p):
                k = k[len(p):]
                break
        out[k] = v
    return out


class _ModelBase(nn.Module):
    prefixes: tuple = ()

    def __init__(self, config: dict):
        super().__init__()
        self.config = dict(config)

    def load_hf_state(self, state: Dict[str, torch.Tensor]):
        sd = _strip_prefix(state, self.prefixes)
        own = self.state_dict()
        missing = [k for k in own if k not in sd and not k.endswith("_buf")]
        if missing:
            raise KeyError(f"{type(self).__name__}: checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        with torch.no_grad():
            for k, t in own.items():
                if k in sd:
                    src = sd[k]
                    if src.shape != t.shape:
                        raise ValueError(f"{k}: checkpoint shape {tuple(src.shape)} != model shape {tuple(t.shape)}")
                    t.copy_(src.to(t.dtype))
        return self


# ------------------------------------------------------------------------------------------ BERT
class _BertLayer(nn.Module):
    def __init__(self, D, H, I, eps):
        super().__init__()
        self.H = H
        self.attention = nn.ModuleDict(dict(
            self=nn.ModuleDict(dict(query=nn.Linear(D, D), key=nn.Linear(D, D), value=nn.Linear(D, D))),
            output=nn.ModuleDict(dict(dense=nn.Linear(D, D), LayerNorm=nn.LayerNorm(D, eps=eps)))))
        self.intermediate = nn.ModuleDict(dict(dense=nn.Linear(D, I)))
        self.output = nn.ModuleDict(dict(dense=nn.Linear(I, D), LayerNorm=nn.LayerNorm(D, eps=eps)))

    def forward(self, x):
        B, T, D = x.shape
        s, o = self.attention["self"], self.attention["output"]
        q = _linear(x, s["query"].weight, s["query"].bias).view(B, T, self.H, -1)
        k = _linear(x, s["key"].weight, s["key"].bias).view(B, T, self.H, -1)
        v = _linear(x, s["value"].weight, s["value"].bias).view(B, T, self.H, -1)
        a = _attention(q, k, v, causal=False).reshape(B, T, D)
        x = o["LayerNorm"](_linear(a, o["dense"].weight, o["dense"].bias) + x)
        h = F.gelu(_linear(x, self.intermediate["dense"].weight, self.intermediate["dense"].bias))
        return self.output["LayerNorm"](_linear(h, self.output["dense"].weight, self.output["dense"].bias) + x)


class BertModel(_ModelBase):
    """Encoder; ``forward(input_ids, token_type_ids=None)`` returns the last hidden state."""
    prefixes = ("bert.",)

    def __init__(self, config: dict):
        super().__init__(config)
        D, H, I = config["hidden_size"], config["num_attention_heads"], config["intermediate_size"]
        eps = config.get("layer_norm_eps", 1e-12)
        self.embeddings = nn.ModuleDict(dict(
            word_embeddings=nn.Embedding(config["vocab_size"], D),
            position_embeddings=nn.Embedding(config.get("max_position_embeddings", 512), D),
            token_type_embeddings=nn.Embedding(config.get("type_vocab_size", 2), D),
            LayerNorm=nn.LayerNorm(D, eps=eps)))
        self.encoder = nn.ModuleDict(dict(layer=nn.ModuleList(_BertLayer(D, H, I, eps) for _ in range(config["num_hidden_layers"]))))

    def forward(self, input_ids: torch.Tensor, token_type_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, T = input_ids.shape
        e = self.embeddings
        pos = torch.arange(T, device=input_ids.device)
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(input_ids)
        x = e["LayerNorm"](e["word_embeddings"](input_ids) + e["position_embeddings"](pos)[None] + e["token_type_embeddings"](tt))
        for layer in self.encoder["layer"]:
            x = layer(x)
        return x


# ------------------------------------------------------------------------------------------ GPT-2
class _Conv1D(nn.Module):
    """GPT-2's linear layer: weight stored ``[in, out]``."""

    def __init__(self, nin, nout):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(nin, nout))
        self.bias = nn.Parameter(torch.zeros(nout))
        self._wt = None

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16:
            if self._wt is None or self._wt.device != self.weight.device:
                self._wt = self.weight.detach().t().contiguous()             # K-major copy for the GEMM, made once
            return _linear(x, self._wt, self.bias)
        return x @ self.weight + self.bias


class _GPT2Block(nn.Module):
    def __init__(self, D, H, eps, inner):
        super().__init__()
        self.H = H
        self.ln_1, self.ln_2 = nn.LayerNorm(D, eps=eps), nn.LayerNorm(D, eps=eps)
        self.attn = nn.ModuleDict(dict(c_attn=_Conv1D(D, 3 * D), c_proj=_Conv1D(D, D)))
        self.mlp = nn.ModuleDict(dict(c_fc=_Conv1D(D, inner), c_proj=_Conv1D(inner, D)))

    def forward(self, x):
        B, T, D = x.shape
        q, k, v = self.attn["c_attn"](self.ln_1(x)).split(D, dim=-1)
        sh = (B, T, self.H, D // self.H)
        a = _attention(q.reshape(sh), k.reshape(sh), v.reshape(sh), causal=True).reshape(B, T, D)
        x = x + self.attn["c_proj"](a)
        return x + self.mlp["c_proj"](F.gelu(self.mlp["c_fc"](self.ln_2(x)), approximate="tanh"))


class GPT2Model(_ModelBase):
    prefixes = ("transformer.",)

    def __init__(self, config: dict):
        super().__init__(config)
        D, H = config["n_embd"], config["n_head"]
        eps = config.get("layer_norm_epsilon", 1e-5)
        self.wte = nn.Embedding(config["vocab_size"], D)
        self.wpe = nn.Embedding(config.get("n_positions", 1024), D)
        self.h = nn.ModuleList(_GPT2Block(D, H, eps, config.get("n_inner") or 4 * D) for _ in range(config["n_layer"]))
        self.ln_f = nn.LayerNorm(D, eps=eps)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        T = input_ids.shape[1]
        x = self.wte(input_ids) + self.wpe(torch.arange(T, device=input_ids.device))[None]
        for blk in self.h:
            x = blk(x)
        return self.ln_f(x)


# ------------------------------------------------------------------------------------------ Llama
class _RMSNorm(nn.Module):
    def __init__(self, D, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(D))
        self.eps = eps

    def forward(self, x):
        from .ops.fused_ops import rms_norm
        return rms_norm(x, self.weight, self.eps)


class _LlamaLayer(nn.Module):
    def __init__(self, D, H, Hk, I, eps):
        super().__init__()
        self.H, self.Hk, self.Dh = H, Hk, D // H
        self.self_attn = nn.ModuleDict(dict(q_proj=nn.Linear(D, H * self.Dh, bias=False), k_proj=nn.Linear(D, Hk * self.Dh, bias=False),
                                            v_proj=nn.Linear(D, Hk * self.Dh, bias=False), o_proj=nn.Linear(H * self.Dh, D, bias=False)))
        self.mlp = nn.ModuleDict(dict(gate_proj=nn.Linear(D, I, bias=False), up_proj=nn.Linear(D, I, bias=False),
                                      down_proj=nn.Linear(I, D, bias=False)))
        self.input_layernorm, self.post_attention_layernorm = _RMSNorm(D, eps), _RMSNorm(D, eps)

    def forward(self, x, cos, sin):
        B, T, D = x.shape
        a = self.self_attn
        h = self.input_layernorm(x)
        q = _linear(h, a["q_proj"].weight).view(B, T, self.H, self.Dh)
        k = _linear(h, a["k_proj"].weight).view(B, T, self.Hk, self.Dh)
        v = _linear(h, a["v_proj"].weight).view(B, T, self.Hk, self.Dh)
        q, k = _rotate_half(q, cos, sin), _rotate_half(k, cos, sin)
        x = x + _linear(_attention(q, k, v, causal=True).reshape(B, T, -1), a["o_proj"].weight)
        h = self.post_attention_layernorm(x)
        m = self.mlp
        return x + _linear(F.silu(_linear(h, m["gate_proj"].weight)) * _linear(h, m["up_proj"].weight), m["down_proj"].weight)


def _rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding on pairs (j, j + D/2); x [B, T, H, D], cos / sin [T, D/2]."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        from .ops.fused_ops import rope
        return rope(x.contiguous(), cos, sin, neox=True)
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


class LlamaModel(_ModelBase):
    prefixes = ("model.",)

    def __init__(self, config: dict):
        super().__init__(config)
        D, H = config["hidden_size"], config["num_attention_heads"]
        Hk = config.get("num_key_value_heads") or H
        eps = config.get("rms_norm_eps", 1e-5)
        self.embed_tokens = nn.Embedding(config["vocab_size"], D)
        self.layers = nn.ModuleList(_LlamaLayer(D, H, Hk, config["intermediate_size"], eps) for _ in range(config["num_hidden_layers"]))
        self.norm = _RMSNorm(D, eps)
        self.theta, self.Dh = float(config.get("rope_theta", 10000.0)), D // H

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        T = input_ids.shape[1]
        inv = 1.0 / (self.theta ** (torch.arange(0, self.Dh, 2, dtype=torch.float64) / self.Dh))
        ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
        cos, sin = ang.cos().float().to(input_ids.device), ang.sin().float().to(input_ids.device)
        x = self.embed_tokens(input_ids)
        for layer in self.layers:
            x = layer(x, cos, sin)
        return self.norm(x)


_ARCH_REGISTRY = {"BertModel": BertModel, "BertForMaskedLM": BertModel, "BertForSequenceClassification": BertModel,
                  "GPT2Model": GPT2Model, "GPT2LMHeadModel": GPT2Model, "LlamaModel": LlamaModel, "LlamaForCausalLM": LlamaModel}


def _detect_architecture(config: dict) -> str:
    for a in config.get("architectures") or []:
        if a in _ARCH_REGISTRY:
            return a
    mt = str(config.get("model_type", "")).lower()
    if mt == "bert":
        return "BertModel"
    if mt in ("gpt2", "openai-gpt"):
        return "GPT2Model"
    if mt == "llama":
        return "LlamaModel"
    raise ValueError(f"Unsupported architecture {config.get('architectures')!r} (model_type={mt!r}). "
                     f"Supported: {sorted(set(_ARCH_REGISTRY))}")


class AutoConfig:
    @staticmethod
    def from_pretrained(model_dir: str) -> dict:
        path = os.path.join(model_dir, "config.json")
        if not os.path.isfile(path):
            raise FileNotFoundError(f"config.json not found in {model_dir}")
        with open(path, encoding="utf-8") as fp:
            return json.load(fp)


class AutoModel:
    """``AutoModel.from_pretrained(dir)`` returns a ``BertModel`` / ``GPT2Model`` / ``LlamaModel`` holding the checkpoint."""

    @staticmethod
    def from_pretrained(model_dir: str, device=None, dtype=None) -> _ModelBase:
        config = AutoConfig.from_pretrained(model_dir)
        cls = _ARCH_REGISTRY[_detect_architecture(config)]
        state = load_checkpoint_dir(model_dir)
        if not state:
            raise FileNotFoundError(f"no model.safetensors, sharded index or pytorch_model.bin in {model_dir}")
        model = cls(config).load_hf_state(state)
        if device is not None or dtype is not None:
            model = model.to(device=device, dtype=dtype)
        return model.eval()


# ------------------------------------------------------------------------------------------ tokenizer
class _SimpleTokenizer:
    """``encode`` / ``decode`` for the three common layouts: byte-level BPE (``tokenizer.json`` with merges, or
    ``vocab.json`` + ``merges.txt``), WordPiece (``vocab.txt`` or a WordPiece ``tokenizer.json``)."""

    def __init__(self, kind: str, impl, special: Optional[Dict[str, int]] = None):
        self.kind, self.impl, self.special = kind, impl, special or {}

    def encode(self, text: str) -> List[int]:
        if self.kind == "bpe":
            return self.impl.encode(text, add_bos=False)
        return self.impl.encode(text)

    def decode(self, ids: List[int]) -> str:
        return self.impl.decode(list(ids))

    @property
    def vocab_size(self) -> int:
        return self.impl.vocab_size if hasattr(self.impl, "vocab_size") else len(self.impl)


class _WordPiece:
    def __init__(self, vocab: Dict[str, int], unk: str = "[UNK]", lower: bool = True):
        self.vocab, self.unk, self.lower = vocab, unk, lower
        self.inv = {i: t for t, i in vocab.items()}

    @property
    def vocab_size(self):
        return len(self.vocab)

    def encode(self, text: str) -> List[int]:
        import re
        ids = []
        for word in re.findall(r"\w+|[^\w\s]", text.lower() if self.lower else text):
            start, pieces = 0, []
            while start < len(word):
                end, cur = len(word), None
                while end > start:
                    sub = ("##" if start else "") + word[start:end]
                    if sub in self.vocab:
                        cur = sub
                        break
                    end -= 1
                if cur is None:
                    pieces = [self.unk]
                    break
                pieces.append(cur)
                start = end
            ids.extend(self.vocab.get(p, self.vocab.get(self.unk, 0)) for p in pieces)
        return ids

    def decode(self, ids) -> str:
        out = ""
        for i in ids:
            t = self.inv.get(int(i), self.unk)
            out += t[2:] if t.startswith("##") else (" " if out else "") + t
        return out


class AutoTokenizer:
    @staticmethod
    def from_pretrained(model_dir: str) -> _SimpleTokenizer:
        from .serve.llm import load_hf_tokenizer
        tj, vt = os.path.join(model_dir, "tokenizer.json"), os.path.join(model_dir, "vocab.txt")
        if os.path.exists(tj):
            with open(tj, encoding="utf-8") as f:
                model = json.load(f).get("model", {})
            if model.get("type") == "WordPiece" or (model.get("vocab") and not model.get("merges") and "[UNK]" in model["vocab"]):
                return _SimpleTokenizer("wordpiece", _WordPiece(model["vocab"], model.get("unk_token", "[UNK]")))
        bpe = load_hf_tokenizer(model_dir)
        if bpe is not None:
            return _SimpleTokenizer("bpe", bpe)
        if os.path.exists(vt):
            with open(vt, encoding="utf-8") as f:
                vocab = {ln.rstrip("\n"): i for i, ln in enumerate(f)}
            return _SimpleTokenizer("wordpiece", _WordPiece(vocab))
        raise FileNotFoundError(f"no tokenizer.json, vocab.json + merges.txt or vocab.txt in {model_dir}")


__all__ = ["AutoConfig", "AutoModel", "AutoTokenizer", "BertModel", "GPT2Model", "LlamaModel"]
