"""Transformer hyper-parameters parsed from GGUF metadata.

Field names follow the reference's ``TransformerConfig``
(torch/io/gguf_model.h:57-325): ``<arch>.embedding_length`` becomes
``hidden_size`` and so on.  Architecture flags: qwen3/gemma3 carry a per-head
RMSNorm on Q and K, the qwen/gemma/phi families rotate NeoX-style pairs
``(i, i + d/2)`` while llama/mistral rotate interleaved pairs ``(2i, 2i+1)``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

NEOX_ARCHS = {
    "qwen", "qwen2", "qwen3", "qwen2moe", "qwen3moe", "gemma", "gemma2", "gemma3", "gemma3n",
    "phi2", "phi3", "phimoe", "stablelm", "starcoder2", "falcon", "gptneox", "deepseek2",
}


@dataclass
class TransformerConfig:
    architecture: str = "llama"
    model_name: str = ""
    vocab_size: int = 0
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    intermediate_size: int = 0
    head_dim: int = 0
    context_length: int = 8192
    rope_freq_base: float = 10000.0
    rope_scale: float = 1.0
    rope_swa_freq_base: float = 10000.0
    swa_window: int = 0
    swa_pattern: int = 0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    scale_embeddings: bool = False
    gemma_norm_add_one: bool = False
    has_qk_norm: bool = False
    ffn_gelu: bool = False
    has_post_norm: bool = False
    rope_neox: bool = False
    rope_yarn: bool = False
    yarn_factor: float = 1.0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    yarn_orig_ctx: int = 0
    rope_attn_factor: float = 1.0
    rope_factors_short: Optional[List[float]] = None     # phi-3 LongRoPE: inv_freq[i] /= factor[i]
    rope_factors_long: Optional[List[float]] = None
    rope_orig_ctx: int = 0                                # sequences up to this length use the short factors
    bos_token_id: int = -1
    eos_token_id: int = -1
    extra_stop_ids: List[int] = field(default_factory=list)

    def rope_factors_for(self, seq_len: int) -> Optional[List[float]]:
        """LongRoPE selector (the reference's rule, torch/io/gguf_model.h:285-296): the short factors while the sequence
        fits the original context, the long ones beyond it; None for models without factor tensors."""
        if self.rope_factors_short is None and self.rope_factors_long is None:
            return None
        if self.rope_orig_ctx <= 0 or seq_len <= self.rope_orig_ctx:
            return self.rope_factors_short
        return self.rope_factors_long if self.rope_factors_long is not None else self.rope_factors_short

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    @classmethod
    def from_gguf(cls, reader) -> "TransformerConfig":
        a = reader.arch()
        g = reader.get_arch
        c = cls(architecture=a, model_name=reader.get("general.name", ""))
        c.hidden_size = int(g("embedding_length", 0))
        c.num_layers = int(g("block_count", 0))
        c.num_heads = int(g("attention.head_count", 0))
        c.num_kv_heads = int(g("attention.head_count_kv", c.num_heads))
        c.intermediate_size = int(g("feed_forward_length", 0))
        c.context_length = int(g("context_length", 8192))
        c.rope_freq_base = float(g("rope.freq_base", 10000.0))
        c.rms_norm_eps = float(g("attention.layer_norm_rms_epsilon", 1e-6))
        key_len = int(g("attention.key_length", 0))
        c.head_dim = key_len if key_len > 0 else (c.hidden_size // max(c.num_heads, 1))
        scaling = g("rope.scaling.type", "")
        factor = float(g("rope.scaling.factor", 1.0))
        if scaling == "linear":
            c.rope_scale = factor
        elif scaling == "yarn":
            c.rope_yarn = True
            c.yarn_factor = factor
            c.yarn_beta_fast = float(g("rope.scaling.yarn_beta_fast", 32.0))
            c.yarn_beta_slow = float(g("rope.scaling.yarn_beta_slow", 1.0))
            c.yarn_orig_ctx = int(g("rope.scaling.original_context_length", 0))
        c.rope_attn_factor = float(g("rope.scaling.attn_factor", 1.0))
        c.rope_orig_ctx = int(g("rope.scaling.original_context_length", 0))
        for which in ("short", "long"):
            name = f"rope_factors_{which}.weight"
            if name in reader.tensors:
                setattr(c, f"rope_factors_{which}", [float(v) for v in reader.load(name).reshape(-1).tolist()])
        c.swa_window = int(g("attention.sliding_window", 0))
        c.swa_pattern = int(g("attention.sliding_window_pattern", 0))
        if "token_embd.weight" in reader.tensors:
            c.vocab_size = int(reader.tensors["token_embd.weight"].shape[0])
        else:
            toks = reader.get("tokenizer.ggml.tokens")
            c.vocab_size = len(toks) if toks is not None else int(g("vocab_size", 0))
        c.tie_word_embeddings = "output.weight" not in reader.tensors
        if a.startswith("gemma"):
            c.scale_embeddings = True
            c.tie_word_embeddings = True
            c.ffn_gelu = True
        if a == "gemma3":
            c.has_qk_norm = True
            c.has_post_norm = True
            if c.swa_window and not c.swa_pattern:
                c.swa_pattern = 6
        if a in ("qwen3", "qwen3moe"):
            c.has_qk_norm = True
        c.rope_neox = a in NEOX_ARCHS
        c.bos_token_id = int(reader.get("tokenizer.ggml.bos_token_id", -1))
        c.eos_token_id = int(reader.get("tokenizer.ggml.eos_token_id", -1))
        return c


def layer_matrix_sources(reader, cfg: "TransformerConfig", layer: int):
    """Where the seven matrices of a decoder layer live in the file: ``{q, k, v, o, gate, up, down} -> (tensor name,
    (row0, row1) or None)``.  phi-3 / phi-2 / starcoder2 files store Q, K and V merged as ``attn_qkv`` and gate and up
    merged as an ``ffn_up`` of twice the FFN width (gate rows first); the merged tensors are addressed by row ranges,
    as the reference splits them (torch/io/gguf_model.h:1624-1653)."""
    p = f"blk.{layer}."
    src = {"o": (p + "attn_output.weight", None), "down": (p + "ffn_down.weight", None)}
    if reader.has_tensor(p + "attn_q.weight"):
        for k in ("q", "k", "v"):
            src[k] = (p + f"attn_{k}.weight", None)
    elif reader.has_tensor(p + "attn_qkv.weight"):
        Q, KV = cfg.q_dim, cfg.kv_dim
        n = p + "attn_qkv.weight"
        src.update(q=(n, (0, Q)), k=(n, (Q, Q + KV)), v=(n, (Q + KV, Q + 2 * KV)))
    else:
        raise KeyError(f"layer {layer}: neither attn_q nor attn_qkv")
    up = p + "ffn_up.weight"
    if reader.has_tensor(p + "ffn_gate.weight"):
        src.update(gate=(p + "ffn_gate.weight", None), up=(up, None))
    elif reader.has_tensor(up) and reader.tensors[up].shape[0] == 2 * cfg.intermediate_size:
        I = cfg.intermediate_size
        src.update(gate=(up, (0, I)), up=(up, (I, 2 * I)))
    else:
        raise KeyError(f"layer {layer}: no ffn_gate and ffn_up is not a merged gate+up")
    return src


# Shapes named by the benchmark configs.
def qwen3_4b_config() -> TransformerConfig:
    return TransformerConfig(
        architecture="qwen3", model_name="qwen3-4b-shape", vocab_size=151936, hidden_size=2560,
        num_layers=36, num_heads=32, num_kv_heads=8, intermediate_size=9728, head_dim=128,
        context_length=40960, rope_freq_base=1e6, rms_norm_eps=1e-6, has_qk_norm=True, rope_neox=True)


def tiny_gemma3_config(layers: int = 3, hidden: int = 1024, heads: int = 8, kv_heads: int = 4, inter: int = 2048, vocab: int = 2048,
                       head_dim: int = 128, window: int = 0) -> TransformerConfig:
    """A small model with gemma3's structure: post-attention / post-FFN norms, QK-norm, GELU-gated FFN, scaled and tied
    embeddings, optional sliding-window layers (every 6th layer global)."""
    return TransformerConfig(
        architecture="gemma3", model_name="gemma3-tiny", vocab_size=vocab, hidden_size=hidden, num_layers=layers, num_heads=heads,
        num_kv_heads=kv_heads, intermediate_size=inter, head_dim=head_dim, context_length=4096, rope_freq_base=1e6, rms_norm_eps=1e-6,
        has_qk_norm=True, has_post_norm=True, ffn_gelu=True, scale_embeddings=True, tie_word_embeddings=True, rope_neox=True,
        swa_window=window, swa_pattern=6 if window else 0)


def tiny_qwen3_config(layers: int = 2, hidden: int = 512, heads: int = 8, kv_heads: int = 2,
                      inter: int = 1024, vocab: int = 1024, head_dim: int = 128) -> TransformerConfig:
    return TransformerConfig(
        architecture="qwen3", model_name="qwen3-tiny", vocab_size=vocab, hidden_size=hidden,
        num_layers=layers, num_heads=heads, num_kv_heads=kv_heads, intermediate_size=inter,
        head_dim=head_dim, context_length=4096, rope_freq_base=1e6, rms_norm_eps=1e-6,
        has_qk_norm=True, rope_neox=True)
