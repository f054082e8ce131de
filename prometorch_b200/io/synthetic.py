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
                         q_more: GGMLType = GGMLType.Q6_K, with_tokenizer: bool = True, merged: bool = False,
                         rope_factors=None, rope_orig_ctx: int = 0) -> str:
    """Write a random-weight model of shape ``cfg`` to ``path``.

    Quantisation runs on ``device`` (a GPU turns the 4 B-parameter shape around
    in seconds); each tensor is produced, quantised, copied to the host and
    written before the next one is generated, so peak memory stays at one tensor.

    ``merged=True`` stores Q/K/V as one ``attn_qkv`` and gate/up as one ``ffn_up`` of twice the FFN width, the way
    phi-3 files do (both parts then use ``q_main``); ``rope_factors=(short, long)`` adds LongRoPE factor tensors.
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
    if rope_orig_ctx:
        w.add(f"{a}.rope.scaling.original_context_length", int(rope_orig_ctx))
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
        if merged:
            w.add_tensor(p + "attn_qkv.weight", (Q + 2 * KV, H), q_main, rnd(Q + 2 * KV, H, q_main))
        else:
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
        if merged:
            w.add_tensor(p + "ffn_up.weight", (2 * I, H), q_main, rnd(2 * I, H, q_main))
        else:
            w.add_tensor(p + "ffn_gate.weight", (I, H), q_main, rnd(I, H, q_main))
            w.add_tensor(p + "ffn_up.weight", (I, H), q_main, rnd(I, H, q_main))
        w.add_tensor(p + "ffn_down.weight", (H, I), q_more, rnd(H, I, q_more))
        if cfg.has_post_norm:
            w.add_tensor(p + "post_ffw_norm.weight", (H,), GGMLType.F32, norm(H))
    w.add_tensor("output_norm.weight", (H,), GGMLType.F32, norm(H))
    if rope_factors is not None:
        for which, vals in zip(("short", "long"), rope_factors):
            t = torch.tensor(list(vals), dtype=torch.float32)
            w.add_tensor(f"rope_factors_{which}.weight", (t.numel(),), GGMLType.F32, (lambda t=t: quantize(t, GGMLType.F32).cpu()))
    if not cfg.tie_word_embeddings:
        w.add_tensor("output.weight", (V, H), q_more, rnd(V, H, q_more))
    return w.write()


def write_synthetic_deepseek2(path: str, *, vocab: int = 320, hidden: int = 256, layers: int = 3, heads: int = 4,
                              kv_lora: int = 64, qk_nope: int = 32, rope_dim: int = 32, v_dim: int = 32, inter: int = 512,
                              experts: int = 8, used: int = 2, shared: int = 1, expert_ff: int = 128, leading_dense: int = 1,
                              q_lora: int = 0, yarn: bool = True, seed: int = 0, std: float = 0.05,
                              qtype: GGMLType = GGMLType.Q8_0) -> str:
    """A small random deepseek2 file (multi-head latent attention + mixture of experts) with llama.cpp's tensor names
    and metadata keys; ``attn_k_b`` is stored ``[heads, kv_lora, qk_nope]`` and ``attn_v_b`` ``[heads, v_dim, kv_lora]``
    as that conversion does."""
    gen = torch.Generator().manual_seed(seed)
    a = "deepseek2"
    w = GGUFWriter(path)
    w.add("general.architecture", a)
    w.add("general.name", "deepseek2-synthetic")
    w.add("general.alignment", 32)
    for k, v in (("embedding_length", hidden), ("block_count", layers), ("attention.head_count", heads),
                 ("attention.head_count_kv", 1), ("feed_forward_length", inter), ("context_length", 4096),
                 ("attention.kv_lora_rank", kv_lora), ("attention.key_length", kv_lora + rope_dim),
                 ("attention.value_length", kv_lora), ("attention.key_length_mla", qk_nope + rope_dim),
                 ("attention.value_length_mla", v_dim), ("rope.dimension_count", rope_dim), ("expert_count", experts),
                 ("expert_used_count", used), ("expert_shared_count", shared), ("expert_feed_forward_length", expert_ff),
                 ("leading_dense_block_count", leading_dense), ("expert_gating_func", 2)):
        w.add(f"{a}.{k}", int(v))
    if q_lora:
        w.add(f"{a}.attention.q_lora_rank", int(q_lora))
    w.add(f"{a}.rope.freq_base", 10000.0)
    w.add(f"{a}.attention.layer_norm_rms_epsilon", 1e-6)
    w.add(f"{a}.expert_weights_scale", 1.0)
    w.add(f"{a}.expert_weights_norm", True)
    if yarn:
        w.add(f"{a}.rope.scaling.type", "yarn")
        w.add(f"{a}.rope.scaling.factor", 4.0)
        w.add(f"{a}.rope.scaling.original_context_length", 64)
        w.add(f"{a}.rope.scaling.yarn_log_multiplier", 0.1)
    toks = _tokens_for(vocab)
    w.add("tokenizer.ggml.model", "llama")
    w.add("tokenizer.ggml.tokens", toks, elem_type=T_STR)
    w.add("tokenizer.ggml.scores", [0.0] * len(toks), elem_type=T_F32)
    w.add("tokenizer.ggml.token_type", [6 if i < 256 else 1 for i in range(len(toks))], elem_type=T_I32)
    w.add("tokenizer.ggml.bos_token_id", 1)
    w.add("tokenizer.ggml.eos_token_id", 2)
    w.add("tokenizer.ggml.add_bos_token", False)

    def rnd(*shape, qt=qtype):
        def make():
            return quantize(torch.randn(*shape, generator=gen) * std, qt)
        return make

    def norm(n):
        return lambda: quantize(1.0 + 0.05 * torch.randn(n, generator=gen), GGMLType.F32)

    def add(name, shape, qt=qtype):
        w.add_tensor(name, shape, qt, rnd(*shape, qt=qt))
    H, key = hidden, qk_nope + rope_dim
    add("token_embd.weight", (vocab, H))
    for i in range(layers):
        p = f"blk.{i}."
        w.add_tensor(p + "attn_norm.weight", (H,), GGMLType.F32, norm(H))
        if q_lora:
            add(p + "attn_q_a.weight", (q_lora, H))
            w.add_tensor(p + "attn_q_a_norm.weight", (q_lora,), GGMLType.F32, norm(q_lora))
            add(p + "attn_q_b.weight", (heads * key, q_lora))
        else:
            add(p + "attn_q.weight", (heads * key, H))
        add(p + "attn_kv_a_mqa.weight", (kv_lora + rope_dim, H))
        w.add_tensor(p + "attn_kv_a_norm.weight", (kv_lora,), GGMLType.F32, norm(kv_lora))
        add(p + "attn_k_b.weight", (heads, kv_lora, qk_nope))
        add(p + "attn_v_b.weight", (heads, v_dim, kv_lora))
        add(p + "attn_output.weight", (H, heads * v_dim))
        w.add_tensor(p + "ffn_norm.weight", (H,), GGMLType.F32, norm(H))
        if i < leading_dense:
            add(p + "ffn_gate.weight", (inter, H))
            add(p + "ffn_up.weight", (inter, H))
            add(p + "ffn_down.weight", (H, inter))
        else:
            add(p + "ffn_gate_inp.weight", (experts, H), GGMLType.F32)
            add(p + "ffn_gate_exps.weight", (experts, expert_ff, H))
            add(p + "ffn_up_exps.weight", (experts, expert_ff, H))
            add(p + "ffn_down_exps.weight", (experts, H, expert_ff))
            if shared:
                add(p + "ffn_gate_shexp.weight", (shared * expert_ff, H))
                add(p + "ffn_up_shexp.weight", (shared * expert_ff, H))
                add(p + "ffn_down_shexp.weight", (H, shared * expert_ff))
    w.add_tensor("output_norm.weight", (H,), GGMLType.F32, norm(H))
    add("output.weight", (vocab, H))
    return w.write()
