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


def __getattr__(name):
    if name == "GGUFModel":
        from .gguf_model import GGUFModel
        return GGUFModel
    raise AttributeError(name)
