"""Model I/O: GGUF container, GGML block formats, tokenizer, chat templates, Ollama store resolver and the
quantised decode model."""
from .config import TransformerConfig, qwen3_4b_config, tiny_qwen3_config
from .gguf import GGUFReader, GGUFWriter
from .gguf_quant import GGMLType, dequantize, quantize
from .tokenizer import GGUFTokenizer
from .chat import apply_chat_template, render_messages, strip_think
from .ollama import list_models, resolve_model
from .synthetic import write_synthetic_gguf
from .model_loader import ModelWeights, detect_format, load_model, read_tensor  # noqa: F401
from . import safetensors  # noqa: F401
from .gguf import TensorInfo as GGUFTensorInfo  # noqa: F401
from .speculative import LowRankOutputProj, NgramDraft, SlidingWindowAttention, SpecStats, speculative_generate  # noqa: F401
from ..utils.profiler import InferenceProfiler  # noqa: F401
from dataclasses import dataclass as _dataclass


@_dataclass
class GGUFTPConfig:
    """Which slice of a model a rank holds under tensor parallelism (the fields ``GGUFModel(tp_rank=, tp_world=)`` takes)."""
    rank: int = 0
    world: int = 1

    def kwargs(self):
        return {"tp_rank": self.rank, "tp_world": self.world}


def __getattr__(name):
    if name == "GGUFModel":
        from .gguf_model import GGUFModel
        return GGUFModel
    if name in ("QuantizedWeight", "PackedWeight"):        # a matrix repacked for the decode kernels
        from .gguf_model import PackedWeight
        return PackedWeight
    raise AttributeError(name)
