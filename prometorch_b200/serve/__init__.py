"""Serving: PromeServe (Ollama-compatible REST, :mod:`.server`), ``LLMEngine`` (request queue over one GGUF model) and
the continuous-batching engine over a paged KV cache for Hugging Face Llama directories (:mod:`.llm`: ``PagedLLMEngine``,
``EngineServer``; the server's ``PagedBackend`` uses it).

``python -m prometorch_b200.serve --port 11434 --device cuda --model NAME --workers N --queue-depth N --timeout-ms MS``
starts the server (same flags as the reference's ``promeserve`` binary, promeserve/main.cpp:40-105)."""
from __future__ import annotations

import collections
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from . import llm
from .llm import GenerationConfig, LlamaConfig, LlamaWeights, PagedKVCache, load_safetensors, save_safetensors
from .llm import LLMEngine as PagedLLMEngine
from .llm import EngineServer  # noqa: F401
from .server import PagedBackend  # noqa: F401
from .server import ApiHandlers, GGUFBackend, HttpServer, ModelBackend, PromeServe, ServerConfig, StreamWriter, VERSION


@dataclass
class Request:
    rid: int
    prompt_ids: List[int]
    max_tokens: int = 32
    temperature: float = 0.0
    top_k: int = 0
    out: List[int] = field(default_factory=list)
    done: bool = False


class LLMEngine:
    """``submit_request / step / poll_responses`` over one model (torch/serve/llm.h:299-420).  Requests are served
    in arrival order; each ``step()`` advances the oldest unfinished request by one scheduling quantum."""

    def __init__(self, backend: ModelBackend, quantum: int = 16):
        self.backend, self.quantum = backend, quantum
        self.queue: Deque[Request] = collections.deque()
        self.finished: Dict[int, Request] = {}
        self._next = 0

    def submit_request(self, prompt, max_tokens: int = 32, temperature: float = 0.0, top_k: int = 0) -> int:
        ids = self.backend.encode(prompt) if isinstance(prompt, str) else list(prompt)
        r = Request(self._next, ids, max_tokens, temperature, top_k)
        self._next += 1
        self.queue.append(r)
        return r.rid

    def step(self) -> int:
        if not self.queue:
            return 0
        r = self.queue.popleft()

        def on_token(t):
            r.out.append(t)
            return len(r.out) < r.max_tokens
        self.backend.generate(r.prompt_ids, {"num_predict": r.max_tokens, "temperature": r.temperature, "top_k": r.top_k or 40,
                                             "repeat_penalty": 1.0}, on_token)
        r.done = True
        self.finished[r.rid] = r
        return len(r.out)

    def poll_responses(self) -> Dict[int, List[int]]:
        out = {rid: r.out for rid, r in self.finished.items()}
        self.finished = {}
        return out

    def generate(self, prompts, max_tokens: int = 32, temperature: float = 0.0, top_k: int = 0) -> List[str]:
        rids = [self.submit_request(p, max_tokens, temperature, top_k) for p in prompts]
        res: Dict[int, List[int]] = {}
        while self.queue:
            self.step()
            res.update(self.poll_responses())
        return ["".join(self.backend.decode_token(t) for t in res[r]) for r in rids]
