"""Synthetic GGUF models: random-init weights quantised with the Q4_K_M recipe.

There is no network access for real checkpoints, so benchmarks and tests use a
file of the named *shape*: weights drawn from N(0, 0.02), quantised to Q4_K
with Q6_K for ``output.weight``, ``attn_v`` and ``ffn_down`` (the Q4_K_M
convention the benchmark config names), F32 norms.  Tensor and metadata names
are the ones the reference's loader expects (torch/io/gguf_model.h:122-181,
6770-6887), so the file is a drop-in for any GGUF consumer.
"""
from __future__ import annotations

from typing import Optional

import torch

from .config import TransformerConfig
from .gguf import GGUFWriter, T_F32, T_I32, T_STR
from .gguf_quant import GGMLType, quantize


def _tokens_for(vocab: int):
    """A printable byte-level style vocabulary: 256 byte tokens then ``<tok_i>``."""
    toks = []
    for i in range(vocab):
        if i < 256:
            toks.append(f"<0x{i:02X}>")
        else:
            toks.append(f"▁t{i}")
    return toks


def write_synthetic_gguf(path: str, cfg: TransformerConfig, seed: int = 0, device: Optional[str] = None,
                         std: float = 0.02, q_main: GGMLType = GGMLType.Q4_K,
                         q_more: GGMLType = GGMLType.Q6_K, with_tokenizer: bool = True) -> str:
    """Write a random-weight model of shape ``cfg`` to ``path``.

    Quantisation runs on ``device`` (a GPU turns the 4 B-parameter shape around
    in seconds); each tensor is produced, quantised, copied to the host and
    written before the next one is generated, so peak memory stays at one tensor.
    """
    if device is None:
        device = "cuda" if torch.cuda.is_available() else "cpu"
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    a = cfg.architecture
    w = GGUFWriter(path)
    w.add("general.architecture", a)
    w.add("general.name", cfg.model_name or f"{a}-synthetic")
    w.add("general.alignment", 32)
    w.add(f"{a}.embedding_length", cfg.hidden_size)
    w.add(f"{a}.block_count", cfg.num_layers)
    w.add(f"{a}.attention.head_count", cfg.num_heads)
    w.add(f"{a}.attention.head_count_kv", cfg.num_kv_heads)
    w.add(f"{a}.feed_forward_length", cfg.intermediate_size)
    w.add(f"{a}.context_length", cfg.context_length)
    w.add(f"{a}.rope.freq_base", float(cfg.rope_freq_base))
    w.add(f"{a}.attention.layer_norm_rms_epsilon", float(cfg.rms_norm_eps))
    w.add(f"{a}.attention.key_length", cfg.head_dim)
    w.add(f"{a}.attention.value_length", cfg.head_dim)
    if cfg.swa_window:
        w.add(f"{a}.attention.sliding_window", int(cfg.swa_window))
        if cfg.swa_pattern:
            w.add(f"{a}.attention.sliding_window_pattern", int(cfg.swa_pattern))
    if with_tokenizer:
        toks = _tokens_for(cfg.vocab_size)
        w.add("tokenizer.ggml.model", "llama")
        w.add("tokenizer.ggml.tokens", toks, elem_type=T_STR)
        w.add("tokenizer.ggml.scores", [0.0] * len(toks), elem_type=T_F32)
        w.add("tokenizer.ggml.token_type", [6 if i < 256 else 1 for i in range(len(toks))], elem_type=T_I32)
        w.add("tokenizer.ggml.bos_token_id", 1)
        w.add("tokenizer.ggml.eos_token_id", 2)
        w.add("tokenizer.ggml.add_bos_token", False)

    def rnd(rows, cols, qt):
        def make():
            x = torch.randn(rows, cols, generator=gen, device=device, dtype=torch.float32) * std
            return quantize(x, qt).cpu()
        return make

    def norm(n):
        def make():
            x = 1.0 + 0.05 * torch.randn(n, generator=gen, device=device, dtype=torch.float32)
            return quantize(x, GGMLType.F32).cpu()
        return make

    H, Q, KV, I, V = cfg.hidden_size, cfg.q_dim, cfg.kv_dim, cfg.intermediate_size, cfg.vocab_size
    w.add_tensor("token_embd.weight", (V, H), q_main, rnd(V, H, q_main))
    for i in range(cfg.num_layers):
        p = f"blk.{i}."
        w.add_tensor(p + "attn_norm.weight", (H,), GGMLType.F32, norm(H))
        w.add_tensor(p + "attn_q.weight", (Q, H), q_main, rnd(Q, H, q_main))
        w.add_tensor(p + "attn_k.weight", (KV, H), q_main, rnd(KV, H, q_main))
        w.add_tensor(p + "attn_v.weight", (KV, H), q_more, rnd(KV, H, q_more))
        if cfg.has_qk_norm:
            w.add_tensor(p + "attn_q_norm.weight", (cfg.head_dim,), GGMLType.F32, norm(cfg.head_dim))
            w.add_tensor(p + "attn_k_norm.weight", (cfg.head_dim,), GGMLType.F32, norm(cfg.head_dim))
        w.add_tensor(p + "attn_output.weight", (H, Q), q_main, rnd(H, Q, q_main))
        if cfg.has_post_norm:
            w.add_tensor(p + "post_attention_norm.weight", (H,), GGMLType.F32, norm(H))
        w.add_tensor(p + "ffn_norm.weight", (H,), GGMLType.F32, norm(H))
        w.add_tensor(p + "ffn_gate.weight", (I, H), q_main, rnd(I, H, q_main))
        w.add_tensor(p + "ffn_up.weight", (I, H), q_main, rnd(I, H, q_main))
        w.add_tensor(p + "ffn_down.weight", (H, I), q_more, rnd(H, I, q_more))
        if cfg.has_post_norm:
            w.add_tensor(p + "post_ffw_norm.weight", (H,), GGMLType.F32, norm(H))
    w.add_tensor("output_norm.weight", (H,), GGMLType.F32, norm(H))
    if not cfg.tie_word_embeddings:
        w.add_tensor("output.weight", (V, H), q_more, rnd(V, H, q_more))
    return w.write()
