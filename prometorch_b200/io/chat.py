"""Chat prompt templates per architecture: ChatML (qwen2/qwen3, ``/no_think`` option), phi-3, gemma,
llama-3 and mistral ``[INST]`` — the formats of torch/io/gguf_model.h:4178-4239.  The default system
prompt and the ``PT_SYSTEM_PROMPT`` / ``PT_NO_THINK`` switches are kept (``PROMETHORCH_*`` spellings too)."""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional

DEFAULT_SYSTEM = "You are a helpful assistant."


def _env(name: str) -> Optional[str]:
    for k in (f"PROMETHORCH_{name}", f"PT_{name}"):
        if k in os.environ:
            return os.environ[k]
    return None


def apply_chat_template(prompt: str, architecture: str, model_name: str = "", system: Optional[str] = None,
                        no_think: Optional[bool] = None) -> str:
    sys = system if system is not None else (_env("SYSTEM_PROMPT") if _env("SYSTEM_PROMPT") is not None else DEFAULT_SYSTEM)
    if no_think is None:
        no_think = (_env("NO_THINK") or "") [:1] == "1"
    a = architecture
    if a in ("qwen3", "qwen2"):
        if no_think and a == "qwen3":
            text = "/no_think" if not sys else sys + "\n/no_think"
            sb = f"<|im_start|>system\n{text}<|im_end|>\n"
        else:
            sb = f"<|im_start|>system\n{sys}<|im_end|>\n" if sys else ""
        return f"{sb}<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"
    if a in ("phi3", "phi2"):
        sb = f"<|system|>\n{sys}<|end|>\n" if sys else ""
        return f"{sb}<|user|>\n{prompt}<|end|>\n<|assistant|>\n"
    if a in ("gemma3", "gemma2", "gemma"):
        user = prompt if not sys else f"{sys}\n\n{prompt}"
        return f"<start_of_turn>user\n{user}<end_of_turn>\n<start_of_turn>model\n"
    if a == "llama":
        if "mistral" in model_name.lower():
            return f"<s>[INST] {prompt} [/INST]" if not sys else f"<s>[INST] <<SYS>>\n{sys}\n<</SYS>>\n\n{prompt} [/INST]"
        sb = f"<|start_header_id|>system<|end_header_id|>\n\n{sys}<|eot_id|>" if sys else ""
        return (f"<|begin_of_text|>{sb}<|start_header_id|>user<|end_header_id|>\n\n{prompt}<|eot_id|>"
                f"<|start_header_id|>assistant<|end_header_id|>\n\n")
    return prompt


def render_messages(messages: List[Dict[str, str]], architecture: str, model_name: str = "") -> str:
    """A list of ``{role, content}`` messages -> one prompt.  System messages become the system block; earlier
    turns are replayed in the architecture's format; the result ends with the assistant header."""
    system = "\n".join(m["content"] for m in messages if m.get("role") == "system") or None
    turns = [m for m in messages if m.get("role") in ("user", "assistant", "tool")]
    if not turns:
        return apply_chat_template("", architecture, model_name, system)
    if architecture in ("qwen3", "qwen2"):
        sys = system if system is not None else DEFAULT_SYSTEM
        out = f"<|im_start|>system\n{sys}<|im_end|>\n" if sys else ""
        for m in turns:
            role = "user" if m["role"] == "tool" else m["role"]
            out += f"<|im_start|>{role}\n{m['content']}<|im_end|>\n"
        return out + "<|im_start|>assistant\n"
    # other formats: fold the history into the last user prompt
    hist = "\n".join(f"{m['role']}: {m['content']}" for m in turns[:-1])
    last = turns[-1]["content"]
    return apply_chat_template(f"{hist}\n{last}" if hist else last, architecture, model_name, system)


_THINK = re.compile(r"<think>.*?</think>\s*", re.S)


def strip_think(text: str) -> str:
    """Remove ``<think>...</think>`` blocks (torch/io/gguf_model.h:5100-5118)."""
    return _THINK.sub("", text)
