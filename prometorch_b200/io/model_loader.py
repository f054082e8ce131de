"""One loader for every weight container the server may be pointed at.

``detect_format`` sniffs magic bytes (GGUF, ZIP-based ``.pt``, pickle, PTOR, the safetensors length + ``{`` header) before it
trusts an extension; ``load_model`` returns a :class:`ModelWeights` with per-tensor metadata, the architecture and the
shape parameters inferred from the tensor names and shapes, and reads tensor data lazily with ``read_tensor``.  Mirrors
the reference's ``promeserve/model_loader.h`` (``detect_format`` :170-227, ``infer_architecture`` :998-1058,
``infer_config_from_tensors`` :1060-1141, ``load_model`` :1197-1249); ONNX initialisers are out of scope here.
"""
from __future__ import annotations

import json
import os
import re
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

FORMATS = ("gguf", "safetensors", "pytorch", "ptor", "hf_dir", "unknown")


@dataclass
class TensorInfo:
    name: str
    dtype: str = "unknown"
    shape: List[int] = field(default_factory=list)
    file: str = ""

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= int(d)
        return n


@dataclass
class ModelConfig:
    hidden_size: int = 0
    num_layers: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    head_dim: int = 0
    context_length: int = 0
    rms_norm_eps: float = 1e-6
    rope_freq_base: float = 10000.0
    tie_word_embeddings: bool = False
    extra: Dict[str, str] = field(default_factory=dict)


@dataclass
class ModelWeights:
    architecture: str = ""
    format: str = "unknown"
    source_path: str = ""
    tensors: Dict[str, TensorInfo] = field(default_factory=dict)
    config: ModelConfig = field(default_factory=ModelConfig)
    files: List[str] = field(default_factory=list)

    def total_parameters(self) -> int:
        return sum(t.numel() for t in self.tensors.values())


def detect_format(path: str) -> str:
    """``gguf`` / ``safetensors`` / ``pytorch`` / ``ptor`` / ``hf_dir`` / ``unknown``; content first, extension second."""
    if os.path.isdir(path):
        return "hf_dir" if os.path.isfile(os.path.join(path, "config.json")) else "unknown"
    try:
        with open(path, "rb") as f:
            head = f.read(9)
    except OSError:
        return "unknown"
    if len(head) < 4:
        return "unknown"
    if head[:4] == b"GGUF":
        return "gguf"
    if head[:4] == b"PTOR":
        return "ptor"
    if len(head) >= 9:                                    # before the pickle test: a header length may start with byte 0x80
        (n,) = struct.unpack("<Q", head[:8])
        if 2 <= n < 100 * 1024 * 1024 and n <= os.path.getsize(path) - 8 and head[8:9] == b"{":
            return "safetensors"
    if head[:4] == b"PK\x03\x04" or (head[0] == 0x80 and head[1] in (2, 3, 4, 5)):
        return "pytorch"
    ext = os.path.splitext(path)[1].lower()
    return {".safetensors": "safetensors", ".gguf": "gguf", ".bin": "pytorch", ".pt": "pytorch", ".pth": "pytorch", ".ptor": "ptor"}.get(ext, "unknown")


def infer_architecture(names) -> str:
    """From tensor names: Hugging Face and GGUF naming of the families the runtime knows."""
    names = list(names)
    joined = "\n".join(names)
    if re.search(r"\bblk\.\d+\.attn_q\.weight", joined):
        return "llama"                                    # GGUF layout; the file's own metadata names the exact family
    if "encoder.layer.0.attention.self.query.weight" in joined:
        return "bert"
    if re.search(r"(^|\.)h\.0\.attn\.c_attn\.weight", joined, re.M):
        return "gpt2"
    if re.search(r"layers\.0\.self_attn\.q_proj\.weight", joined):
        if re.search(r"layers\.0\.self_attn\.q_norm\.weight", joined):
            return "qwen3"
        if re.search(r"layers\.0\.self_attn\.q_proj\.bias", joined):
            return "qwen2"
        if re.search(r"layers\.0\.pre_feedforward_layernorm\.weight", joined):
            return "gemma2"
        return "llama"
    if re.search(r"layers\.0\.self_attn\.qkv_proj\.weight", joined):
        return "phi3"
    return "unknown"


def infer_config_from_tensors(mw: ModelWeights):
    """Fill the shape parameters that the tensor shapes determine (embedding, projections, layer count)."""
    c, t = mw.config, mw.tensors

    def shape(*cands):
        for k in cands:
            for pre in ("", "model.", "transformer.", "bert."):
                if pre + k in t:
                    return t[pre + k].shape
        return None
    emb = shape("embed_tokens.weight", "wte.weight", "embeddings.word_embeddings.weight", "token_embd.weight")
    if emb:
        c.vocab_size, c.hidden_size = int(emb[0]), int(emb[1])
    layer_ids = {int(m.group(1)) for n in t for m in [re.search(r"(?:layers|h|layer|blk)\.(\d+)\.", n)] if m}
    c.num_layers = max(layer_ids) + 1 if layer_ids else 0
    q = shape("layers.0.self_attn.q_proj.weight", "blk.0.attn_q.weight")
    k = shape("layers.0.self_attn.k_proj.weight", "blk.0.attn_k.weight")
    up = shape("layers.0.mlp.up_proj.weight", "blk.0.ffn_up.weight", "h.0.mlp.c_fc.weight", "encoder.layer.0.intermediate.dense.weight")
    if up:
        c.intermediate_size = int(up[1] if "h.0.mlp.c_fc.weight" in "".join(t) and up[0] == c.hidden_size else up[0])
    qn = shape("layers.0.self_attn.q_norm.weight", "blk.0.attn_q_norm.weight")
    if qn:
        c.head_dim = int(qn[0])
    if q and c.hidden_size:
        if not c.head_dim:
            c.head_dim = 128 if int(q[0]) % 128 == 0 and c.hidden_size >= 2048 else 64 if int(q[0]) % 64 == 0 else int(q[0])
        c.num_heads = int(q[0]) // c.head_dim
        if k:
            c.num_kv_heads = int(k[0]) // c.head_dim
    c.tie_word_embeddings = not any(n.endswith("lm_head.weight") or n == "output.weight" for n in t)


def _apply_hf_config(mw: ModelWeights, cfg: dict):
    c = mw.config
    c.hidden_size = int(cfg.get("hidden_size", cfg.get("n_embd", c.hidden_size)))
    c.num_layers = int(cfg.get("num_hidden_layers", cfg.get("n_layer", c.num_layers)))
    c.num_heads = int(cfg.get("num_attention_heads", cfg.get("n_head", c.num_heads)))
    c.num_kv_heads = int(cfg.get("num_key_value_heads", c.num_heads))
    c.intermediate_size = int(cfg.get("intermediate_size", cfg.get("n_inner") or c.intermediate_size))
    c.vocab_size = int(cfg.get("vocab_size", c.vocab_size))
    c.head_dim = int(cfg.get("head_dim", c.hidden_size // c.num_heads if c.num_heads else 0))
    c.context_length = int(cfg.get("max_position_embeddings", cfg.get("n_positions", c.context_length)))
    c.rms_norm_eps = float(cfg.get("rms_norm_eps", c.rms_norm_eps))
    c.rope_freq_base = float(cfg.get("rope_theta", c.rope_freq_base))
    c.tie_word_embeddings = bool(cfg.get("tie_word_embeddings", c.tie_word_embeddings))
    if cfg.get("model_type"):
        mw.architecture = str(cfg["model_type"])


def find_shard_files(path: str) -> List[str]:
    """The files of a sharded checkpoint: what ``model.safetensors.index.json`` lists, else ``*-00001-of-0000N.*`` siblings."""
    d = path if os.path.isdir(path) else os.path.dirname(os.path.abspath(path))
    idx = os.path.join(d, "model.safetensors.index.json")
    if os.path.isfile(idx):
        with open(idx) as f:
            return [os.path.join(d, s) for s in sorted(set(json.load(f)["weight_map"].values()))]
    single = os.path.join(d, "model.safetensors")
    if os.path.isdir(path) and os.path.isfile(single):
        return [single]
    m = re.match(r"(.*)-(\d{5})-of-(\d{5})(\..*)$", os.path.basename(path))
    if m:
        return [os.path.join(d, f"{m.group(1)}-{i:05d}-of-{m.group(3)}{m.group(4)}") for i in range(1, int(m.group(3)) + 1)]
    return [path]


def load_model(path: str) -> ModelWeights:
    """Metadata of every tensor of ``path`` (a file of any known format, or a Hugging Face directory)."""
    fmt = detect_format(path)
    mw = ModelWeights(format=fmt, source_path=path)
    if fmt == "unknown":
        raise ValueError(f"{path}: unknown model format")
    if fmt == "gguf":
        from .gguf import GGUFReader
        r = GGUFReader(path)
        mw.files = [path]
        for name, ti in r.tensors.items():
            mw.tensors[name] = TensorInfo(name, getattr(ti.qtype, "name", str(ti.qtype)).lower(), [int(x) for x in ti.shape], path)
        arch = r.get("general.architecture", "") or "llama"
        mw.architecture = str(arch)
        infer_config_from_tensors(mw)
        g = lambda k, d=0: r.get(f"{arch}.{k}", d)
        c = mw.config
        c.num_heads = int(g("attention.head_count", c.num_heads) or c.num_heads)
        c.num_kv_heads = int(g("attention.head_count_kv", c.num_kv_heads or c.num_heads) or c.num_heads)
        c.context_length = int(g("context_length", 0) or 0)
        c.rope_freq_base = float(g("rope.freq_base", c.rope_freq_base) or c.rope_freq_base)
        c.rms_norm_eps = float(g("attention.layer_norm_rms_epsilon", c.rms_norm_eps) or c.rms_norm_eps)
        if c.num_heads and not c.head_dim:
            c.head_dim = int(g("attention.key_length", 0) or (c.hidden_size // c.num_heads))
        return mw
    if fmt in ("safetensors", "hf_dir"):
        from .safetensors import SafeTensorsFile
        files = find_shard_files(path) if (fmt == "hf_dir" or re.search(r"-\d{5}-of-\d{5}\.", os.path.basename(path))) else [path]
        files = [f for f in files if os.path.isfile(f) and detect_format(f) == "safetensors"]
        if fmt == "hf_dir" and not files:
            legacy = os.path.join(path, "pytorch_model.bin")
            if os.path.isfile(legacy):
                return _finish_dir(load_model(legacy), path)
        mw.files = files
        for fpath in files:
            with SafeTensorsFile(fpath) as f:
                for name in f.keys():
                    meta = f.info(name)
                    mw.tensors[name] = TensorInfo(name, meta["dtype"].lower(), [int(x) for x in meta["shape"]], fpath)
        mw.architecture = infer_architecture(mw.tensors)
        infer_config_from_tensors(mw)
        return _finish_dir(mw, path if fmt == "hf_dir" else os.path.dirname(os.path.abspath(path)))
    from ..serialization import load as load_ptor, load_pytorch
    sd = load_ptor(path) if fmt == "ptor" else load_pytorch(path)
    if isinstance(sd, dict) and "state_dict" in sd and isinstance(sd["state_dict"], dict):
        sd = sd["state_dict"]
    if torch.is_tensor(sd):
        sd = {"tensor": sd}
    mw.files = [path]
    for name, t in sd.items():
        if torch.is_tensor(t):
            mw.tensors[name] = TensorInfo(name, str(t.dtype).replace("torch.", ""), list(t.shape), path)
    mw.architecture = infer_architecture(mw.tensors)
    infer_config_from_tensors(mw)
    return mw


def _finish_dir(mw: ModelWeights, directory: str) -> ModelWeights:
    cj = os.path.join(directory, "config.json")
    if os.path.isfile(cj):
        with open(cj) as f:
            _apply_hf_config(mw, json.load(f))
    return mw


def read_tensor(mw: ModelWeights, name: str) -> torch.Tensor:
    """The data of one tensor (GGUF tensors come back dequantised to fp32)."""
    info = mw.tensors[name]
    if mw.format == "gguf":
        from .gguf import GGUFReader
        return GGUFReader(info.file).load(name)
    if mw.format in ("safetensors", "hf_dir") and detect_format(info.file) == "safetensors":
        from .safetensors import SafeTensorsFile
        with SafeTensorsFile(info.file) as f:
            return f.get_tensor(name)
    from ..serialization import load as load_ptor, load_pytorch
    sd = load_ptor(info.file) if detect_format(info.file) == "ptor" else load_pytorch(info.file)
    sd = sd.get("state_dict", sd) if isinstance(sd, dict) else {"tensor": sd}
    return sd[name]
