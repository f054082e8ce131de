"""PromeServe: an Ollama-compatible HTTP server in front of the native decode engine.

Routes and wire format follow promeserve/api_handlers.h:351-394 and http_server.h of the reference:
``GET /`` (the chat page of ``serve/web`` for a browser, liveness text otherwise), ``GET /api/version``, ``GET /api/tags``, ``GET /api/ps`` (loaded models and counters), ``POST /api/show``,
``POST /api/generate``, ``POST /api/chat``, ``POST /api/embeddings`` (501), ``HEAD``/``OPTIONS`` with CORS.
Streaming responses are chunked ``application/x-ndjson``: one object per token
(``{"model","created_at","response","done":false}`` or, for chat, ``"message":{"role","content"}``) and a
final object with ``total_duration, load_duration, prompt_eval_count, prompt_eval_duration, eval_count,
eval_duration`` in nanoseconds.  Back-pressure: a bounded queue in front of ``worker_threads`` workers;
when it is full the reply is ``503`` with ``Retry-After: 1``.  Per-request timeout: an in-stream
``{"error":"timeout","done":true}``.  One generation runs on the GPU at a time (the engine lock), as in
the reference; what differs is the engine behind it — greedy requests never copy logits to the host, and
sampling runs on the device.
"""
from __future__ import annotations

import json
import queue
import socket
import threading
import time
from dataclasses import dataclass, field
from datetime import datetime, timezone
from http import HTTPStatus
from typing import Callable, Dict, List, Optional

VERSION = "0.1.0-promeserve"


@dataclass
class ServerConfig:
    host: str = "127.0.0.1"             # loopback by default; pass 0.0.0.0 to serve other machines
    port: int = 11434
    worker_threads: int = 4
    max_queue_depth: int = 128
    server_timeout_ms: int = 60000
    device: str = "cuda"
    model: Optional[str] = None
    model_dirs: List[str] = field(default_factory=list)
    max_seq: int = 4096
    max_loaded_models: int = 2          # models resident on the GPU at once; the least recently used one is dropped
    max_body_bytes: int = 8 << 20       # larger request bodies are answered 413
    allow_model_paths: bool = False     # let a request name a model by filesystem path (off: names only)
    web_root: Optional[str] = None      # folder whose index.html answers a browser's GET /; None = the page shipped in serve/web


def _now() -> str:
    return datetime.now(timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.%fZ")


class StreamWriter:
    """Chunked-transfer NDJSON writer over a raw socket file."""

    def __init__(self, wfile):
        self.w = wfile
        self.open = True

    def write(self, obj) -> bool:
        if not self.open:
            return False
        data = (json.dumps(obj, ensure_ascii=False) + "\n").encode("utf-8")
        try:
            self.w.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
            self.w.flush()
            return True
        except (BrokenPipeError, ConnectionResetError, OSError):
            self.open = False
            return False

    def finish(self):
        if self.open:
            try:
                self.w.write(b"0\r\n\r\n")
                self.w.flush()
            except OSError:
                pass
            self.open = False


CORS = {"Access-Control-Allow-Origin": "*", "Access-Control-Allow-Methods": "POST, GET, OPTIONS",
        "Access-Control-Allow-Headers": "Content-Type, Authorization"}


class ModelBackend:
    """What the handlers need from a model.  ``GGUFBackend`` binds the native engine; tests use a fake."""

    name = "model"
    architecture = "llama"
    format = "gguf"
    model_name = ""
    size = 0
    parameter_size = ""

    def encode(self, text: str) -> List[int]:
        raise NotImplementedError

    def decode_token(self, tid: int) -> str:
        raise NotImplementedError

    def generate(self, prompt_ids: List[int], options: Dict, on_token: Callable[[int], bool]):
        """Run prefill + decode; call ``on_token(id)`` per generated token (return False to stop).
        Returns ``(prompt_eval_seconds, eval_seconds)``."""
        raise NotImplementedError


class GGUFBackend(ModelBackend):
    def close(self):
        self.model.close()

    def __init__(self, path: str, name: str, device: str = "cuda", max_seq: int = 4096):
        import os
        from ..io.gguf_model import GGUFModel
        from ..io.tokenizer import GGUFTokenizer
        self.model = GGUFModel(path, device=device, max_seq=max_seq, want_logits=True)
        self.tokenizer = GGUFTokenizer.from_reader(self.model.reader)
        self.name, self.path = name, path
        self.architecture, self.model_name = self.model.cfg.architecture, self.model.cfg.model_name
        self.size = os.path.getsize(path)
        n = sum(t.nbytes for t in self.model.reader.tensors.values())
        self.parameter_size = f"{n / 0.5625 / 1e9:.1f}B"
        self.stop_ids = {self.model.cfg.eos_token_id} - {-1}
        for t in ("<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>"):
            if t in self.tokenizer.vocab:
                self.stop_ids.add(self.tokenizer.vocab[t])

    def encode(self, text):
        return self.tokenizer.encode(text)

    def decode_token(self, tid):
        return self.tokenizer.decode([tid], strip_leading_space=False)

    def generate(self, prompt_ids, options, on_token):
        m = self.model
        n_new = int(options.get("num_predict", 128))
        room = m.max_seq - len(prompt_ids) - 1
        n_new = max(0, min(n_new, room))
        t0 = time.perf_counter()
        if len(prompt_ids) > 1:
            if m.supports_prefill and len(prompt_ids) - 1 >= 8:
                m.prefill(prompt_ids[:-1])      # one batched pass over the prompt (tcgen05 GEMMs + FlashAttention); returns when it is done
            else:
                m.run_script(prompt_ids[:-1], 1)
        t1 = time.perf_counter()
        m.generate(prompt_ids[-1:], max_new_tokens=n_new, temperature=float(options.get("temperature", 0.7)),
                   top_k=int(options.get("top_k", 40)), top_p=float(options.get("top_p", 0.9)),
                   repeat_penalty=float(options.get("repeat_penalty", 1.05)), stop_ids=self.stop_ids, on_token=on_token,
                   _pos0=len(prompt_ids) - 1, _history=prompt_ids)
        return t1 - t0, time.perf_counter() - t1


class OracleBackend(ModelBackend):
    """A GGUF file on the fp32 CPU oracle (``models/gguf_oracle.py``): what ``--device cpu`` serves.  For checking and for
    machines without a GPU; sampling runs on the host."""

    def __init__(self, path: str, name: str, max_seq: int = 4096):
        import os
        from ..io.tokenizer import GGUFTokenizer
        from ..models.gguf_oracle import OracleModel
        self.model = OracleModel(path, device="cpu", max_seq=max_seq)
        self.max_seq = max_seq
        self.tokenizer = GGUFTokenizer.from_reader(self.model.reader)
        self.name, self.path = name, path
        self.architecture, self.model_name = self.model.cfg.architecture, self.model.cfg.model_name
        self.size = os.path.getsize(path)
        n = sum(t.nbytes for t in self.model.reader.tensors.values())
        self.parameter_size = f"{n / 0.5625 / 1e9:.1f}B"
        self.stop_ids = {self.model.cfg.eos_token_id} - {-1}
        for t in ("<|im_end|>", "<|eot_id|>", "<end_of_turn>", "<|end|>", "<|endoftext|>"):
            if t in self.tokenizer.vocab:
                self.stop_ids.add(self.tokenizer.vocab[t])

    def encode(self, text):
        return self.tokenizer.encode(text)

    def decode_token(self, tid):
        return self.tokenizer.decode([tid], strip_leading_space=False)

    def generate(self, prompt_ids, options, on_token):
        import torch
        from ..ops.sampling import sample_logits
        m = self.model
        n_new = max(0, min(int(options.get("num_predict", 128)), self.max_seq - len(prompt_ids) - 1))
        gen = torch.Generator().manual_seed(int(options.get("seed", 42)))
        t0 = time.perf_counter()
        m.reset()
        logits = m.forward(prompt_ids)
        t1 = time.perf_counter()
        history = list(prompt_ids)
        for _ in range(n_new):
            nxt = sample_logits(logits[-1], float(options.get("temperature", 0.7)), int(options.get("top_k", 40)), float(options.get("top_p", 0.9)),
                                float(options.get("repeat_penalty", 1.05)), history, gen)
            history.append(nxt)
            if on_token(nxt) is False or nxt in self.stop_ids:
                break
            logits = m.forward([nxt])
        return t1 - t0, time.perf_counter() - t1

    def close(self):
        pass


class PagedBackend(ModelBackend):
    """A Hugging Face Llama directory served by the continuous-batching engine (``serve/llm.py``).  ``concurrent``:
    the handlers do not serialise generations for this backend, so requests that arrive together share decode
    batches (the reference's server takes one generation at a time, promeserve/api_handlers.h:769-790)."""
    concurrent = True
    architecture = "llama"
    format = "safetensors"

    def __init__(self, model_dir: str, name: str, device: str = "cuda", max_active: int = 16, max_pages: int = 2048):
        import os
        import torch
        from .llm import EngineServer, LLMEngine
        dev = "cpu" if (device == "cuda" and not torch.cuda.is_available()) else device
        self.engine = LLMEngine(device=dev, max_pages=max_pages, max_active=max_active)
        if not self.engine.load(model_dir) or not self.engine.loaded:
            raise KeyError(f"'{model_dir}' is not a loadable Hugging Face Llama directory")
        self.server = EngineServer(self.engine)
        self.name, self.path, self.model_name = name, model_dir, os.path.basename(os.path.normpath(model_dir))
        self.size = sum(os.path.getsize(os.path.join(model_dir, f)) for f in os.listdir(model_dir) if f.endswith(".safetensors"))
        n = sum(t.numel() for L in self.engine.weights.layers for t in L.values()) + self.engine.weights.tok_emb.numel()
        self.parameter_size = f"{n / 1e9:.1f}B"

    def encode(self, text):
        return self.engine._encode(text)

    def decode_token(self, tid):
        return self.engine.tokenizer.decode([tid])

    def embed(self, text: str):
        """Sentence embedding of ``text`` (list of floats), computed on the engine's thread between decode steps."""
        return self.server.call(lambda eng: eng.embed(text).cpu().tolist())

    def generate(self, prompt_ids, options, on_token):
        from .llm import GenerationConfig
        cfg = GenerationConfig(max_new_tokens=int(options.get("num_predict", 128)), temperature=float(options.get("temperature", 0.7)),
                               top_k=int(options.get("top_k", 40)), top_p=float(options.get("top_p", 0.9)),
                               repetition_penalty=float(options.get("repeat_penalty", 1.05)))
        # the scheduler thread only queues the ids; this (HTTP worker) thread runs the caller's hook, so a slow
        # client socket never stalls the decode batches of the other requests
        import queue
        q: "queue.Queue" = queue.Queue()
        stop = {"flag": False}

        def hook(tok: int) -> bool:
            q.put(tok)
            return not stop["flag"]
        h = self.server.submit(list(prompt_ids), cfg, hook)
        while not (h.event.is_set() and q.empty()):
            try:
                tok = q.get(timeout=0.05)
            except queue.Empty:
                continue
            if not stop["flag"] and not on_token(tok):
                stop["flag"] = True                               # the client is gone or timed out: end the request now,
                rid = h.request_id                                # not after one more decode pass
                try:
                    self.server.call(lambda eng: eng.cancel(rid), timeout=30.0)
                except TimeoutError:
                    pass                                          # the hook's False ends it at the next token anyway
        t_end = time.perf_counter()
        t_first = h.t_first if h.t_first is not None else t_end
        return t_first - h.t_submit, t_end - t_first


class ApiHandlers:
    def __init__(self, config: ServerConfig, backends: Optional[Dict[str, ModelBackend]] = None,
                 loader: Optional[Callable[[str], ModelBackend]] = None):
        self.config = config
        self.backends: Dict[str, ModelBackend] = dict(backends or {})
        self.loader = loader
        self.generate_mutex = threading.Lock()
        self.load_mutex = threading.Lock()
        self.pinned = set(self.backends)          # backends handed in by the host program are never evicted
        self.tools_max_iters = 5
        self.stats = {"requests": 0, "tokens_generated": 0, "prompt_tokens": 0, "timeouts": 0}

    # ------------------------------------------------------------------ model management
    def _lookup(self, name: str) -> Optional[ModelBackend]:
        if name in self.backends:
            self.backends[name] = self.backends.pop(name)       # most recently used goes last
            return self.backends[name]
        base = name.split(":")[0]
        for k, b in self.backends.items():
            if k.split(":")[0] == base:
                return b
        return None

    def ensure_model(self, name: str) -> ModelBackend:
        b = self._lookup(name)
        if b is not None:
            return b
        if self.loader is None:
            raise KeyError(f"model '{name}' not found")
        with self.load_mutex:                    # one load at a time; a second request for the same name finds it cached
            b = self._lookup(name)
            if b is not None:
                return b
            loaded = [k for k in self.backends if k not in self.pinned]
            while loaded and len(loaded) >= max(1, self.config.max_loaded_models):
                with self.generate_mutex:        # never drop a model in the middle of its generation
                    old = self.backends.pop(loaded.pop(0))
                    close = getattr(old, "close", None)
                    if close:
                        close()
            b = self.loader(name)
            self.backends[name] = b
            return b

    def tags(self):
        from ..io.ollama import list_models
        seen, models = set(), []
        for name, b in self.backends.items():
            seen.add(name)
            models.append({"name": name, "model": name, "modified_at": _now(), "size": b.size, "digest": "",
                           "details": {"family": b.architecture, "format": b.format, "parameter_size": b.parameter_size}})
        try:
            for m in list_models(extra_dirs=self.config.model_dirs):
                if m["name"] not in seen:
                    models.append({"name": m["name"], "model": m["name"], "modified_at": _now(), "size": m["size"], "digest": "",
                                   "details": {"family": "", "format": "gguf", "parameter_size": ""}})
        except Exception:
            pass
        return {"models": models}

    def ps(self):
        """Loaded models and the server's counters (Ollama's ``/api/ps`` shape, plus ``stats``)."""
        models = [{"name": name, "model": name, "size": b.size, "digest": "", "expires_at": "", "size_vram": int(getattr(b, "size_vram", b.size)),
                   "details": {"family": b.architecture, "format": b.format, "parameter_size": b.parameter_size}}
                  for name, b in self.backends.items()]
        return {"models": models, "stats": dict(self.stats)}

    def show(self, body):
        b = self.ensure_model(body.get("model") or body.get("name") or "")
        return {"modelfile": "", "parameters": "", "template": "", "details": {"family": b.architecture, "format": b.format,
                                                                                 "parameter_size": b.parameter_size},
                "model_info": {"general.architecture": b.architecture, "general.name": b.model_name}}

    # ------------------------------------------------------------------ generation
    def _options(self, body):
        o = {"num_predict": 128, "temperature": 0.7, "top_k": 40, "top_p": 0.9, "repeat_penalty": 1.05}
        o.update(body.get("options") or {})
        return o

    def _run(self, backend: ModelBackend, prompt: str, options, emit: Callable[[str], bool], deadline: float):
        """Tokenise, generate, stream pieces through ``emit``; returns the stats dict and whether it timed out."""
        ids = backend.encode(prompt) or [0]
        pieces: List[str] = []
        state = {"n": 0, "timeout": False}

        def on_token(tid: int) -> bool:
            if time.time() > deadline:
                state["timeout"] = True
                return False
            state["n"] += 1
            piece = backend.decode_token(tid)
            pieces.append(piece)
            return emit(piece)

        import contextlib
        with (contextlib.nullcontext() if getattr(backend, "concurrent", False) else self.generate_mutex):
            pe, ev = backend.generate(ids, options, on_token)
        with self.load_mutex:
            self.stats["requests"] += 1
            self.stats["tokens_generated"] += state["n"]
            self.stats["prompt_tokens"] += len(ids)
            self.stats["timeouts"] += int(state["timeout"])
        stats = {"total_duration": int((pe + ev) * 1e9), "load_duration": 0, "prompt_eval_count": len(ids),
                 "prompt_eval_duration": int(pe * 1e9), "eval_count": state["n"], "eval_duration": int(ev * 1e9)}
        return "".join(pieces), stats, state["timeout"]

    def generate(self, body, writer: Optional[StreamWriter]):
        from ..io.chat import apply_chat_template
        model = body.get("model", "")
        backend = self.ensure_model(model)
        prompt = body.get("prompt", "")
        if not body.get("raw", False) and "<|im_start|>" not in prompt and "[INST]" not in prompt and "<|start_header_id|>" not in prompt:
            prompt = apply_chat_template(prompt, backend.architecture, backend.model_name, body.get("system"))
        deadline = time.time() + self.config.server_timeout_ms / 1e3

        def emit(piece):
            if writer is None:
                return True
            return writer.write({"model": model, "created_at": _now(), "response": piece, "done": False})
        text, stats, timed_out = self._run(backend, prompt, self._options(body), emit, deadline)
        if timed_out:
            final = {"error": "timeout", "done": True}
        else:
            final = {"model": model, "created_at": _now(), "response": "" if writer is not None else text, "done": True, **stats}
        if writer is not None:
            writer.write(final)
            writer.finish()
        return final

    def chat(self, body, writer: Optional[StreamWriter]):
        from ..io.chat import render_messages
        model = body.get("model", "")
        backend = self.ensure_model(model)
        messages = list(body.get("messages") or [])
        tools = body.get("tools") or []
        if tools:
            desc = json.dumps(tools)
            messages = [{"role": "system", "content": "You may call a tool by answering with a JSON object "
                         '{"tool_call": {"name": ..., "arguments": {...}}}. Tools: ' + desc}] + messages
        deadline = time.time() + self.config.server_timeout_ms / 1e3

        def emit(piece):
            if writer is None:
                return True
            return writer.write({"model": model, "created_at": _now(), "message": {"role": "assistant", "content": piece}, "done": False})
        prompt = render_messages(messages, backend.architecture, backend.model_name)
        text, stats, timed_out = self._run(backend, prompt, self._options(body), emit, deadline)
        msg = {"role": "assistant", "content": "" if writer is not None else text}
        call = self._parse_tool_call(text) if tools else None
        if call is not None:
            msg["tool_calls"] = [{"function": call}]
        final = {"error": "timeout", "done": True} if timed_out else {"model": model, "created_at": _now(), "message": msg, "done": True, **stats}
        if writer is not None:
            writer.write(final)
            writer.finish()
        return final

    @staticmethod
    def _parse_tool_call(text: str):
        i = text.find('{"tool_call"')
        if i < 0:
            return None
        depth = 0
        for j in range(i, len(text)):
            depth += text[j] == "{"
            depth -= text[j] == "}"
            if depth == 0:
                try:
                    return json.loads(text[i:j + 1])["tool_call"]
                except (ValueError, KeyError):
                    return None
        return None


class HttpServer:
    """Blocking accept loop + fixed worker pool + bounded queue (503 when full)."""

    def __init__(self, config: ServerConfig, handlers: ApiHandlers):
        self.config, self.handlers = config, handlers
        self.q: "queue.Queue" = queue.Queue(maxsize=config.max_queue_depth)
        self.sock: Optional[socket.socket] = None
        self.threads: List[threading.Thread] = []
        self.running = False
        self.port = config.port

    def start(self):
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((self.config.host, self.config.port))
        self.port = self.sock.getsockname()[1]
        self.sock.listen(128)
        self.running = True
        for _ in range(self.config.worker_threads):
            t = threading.Thread(target=self._worker, daemon=True)
            t.start()
            self.threads.append(t)
        t = threading.Thread(target=self._accept, daemon=True)
        t.start()
        self.threads.append(t)
        return self

    def stop(self):
        self.running = False
        try:
            self.sock.close()
        except OSError:
            pass
        for _ in range(self.config.worker_threads):
            try:
                self.q.put_nowait(None)
            except queue.Full:
                pass

    def _accept(self):
        while self.running:
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            try:
                self.q.put_nowait(conn)
            except queue.Full:
                try:
                    conn.sendall(b"HTTP/1.1 503 Service Unavailable\r\nRetry-After: 1\r\nContent-Length: 0\r\nConnection: close\r\n\r\n")
                finally:
                    conn.close()

    def _worker(self):
        while True:
            conn = self.q.get()
            if conn is None:
                return
            try:
                conn.settimeout(self.config.server_timeout_ms / 1e3)
                self._handle(conn)
            except Exception:
                pass
            finally:
                try:
                    conn.close()
                except OSError:
                    pass

    # ------------------------------------------------------------------ HTTP
    @staticmethod
    def _read_request(rfile, max_body: int = 8 << 20):
        line = rfile.readline(65536).decode("latin1").strip()
        if not line:
            return None
        method, path, _ = (line.split(" ") + ["", ""])[:3]
        headers = {}
        while True:
            h = rfile.readline(65536).decode("latin1")
            if h in ("\r\n", "\n", ""):
                break
            k, _, v = h.partition(":")
            headers[k.strip().lower()] = v.strip()
        try:
            n = int(headers.get("content-length", "0") or 0)
        except ValueError:
            n = -1
        if n < 0 or n > max_body:
            return method.upper(), path.split("?")[0], headers, None       # the caller answers 413
        body = rfile.read(n) if n else b""
        return method.upper(), path.split("?")[0], headers, body

    def _web_page(self) -> Optional[bytes]:
        """index.html of the configured folder, or None when there is none (read per request: the page can be edited live)."""
        import os
        root = self.config.web_root or os.path.join(os.path.dirname(os.path.abspath(__file__)), "web")
        try:
            with open(os.path.join(root, "index.html"), "rb") as f:
                return f.read()
        except OSError:
            return None

    @staticmethod
    def _send(wfile, status: int, body: bytes, ctype="application/json", extra=None):
        reason = HTTPStatus(status).phrase
        hdr = {"Content-Type": ctype, "Content-Length": str(len(body)), "Connection": "close", **CORS, **(extra or {})}
        wfile.write(f"HTTP/1.1 {status} {reason}\r\n".encode() + "".join(f"{k}: {v}\r\n" for k, v in hdr.items()).encode() + b"\r\n" + body)
        wfile.flush()

    def _handle(self, conn):
        rfile, wfile = conn.makefile("rb"), conn.makefile("wb")
        req = self._read_request(rfile, self.config.max_body_bytes)
        if req is None:
            return
        method, path, headers, raw = req
        H = self.handlers
        if raw is None:
            return self._send(wfile, 413, json.dumps({"error": "request body too large"}).encode())
        if "chunked" in headers.get("transfer-encoding", "").lower():
            return self._send(wfile, 400, json.dumps({"error": "chunked request bodies are not supported: send Content-Length"}).encode())
        if method == "OPTIONS":
            return self._send(wfile, 204, b"")
        if method == "HEAD":
            return self._send(wfile, 200 if path in ("/", "/api/version", "/api/tags") else 404, b"")
        if method == "GET" and path in ("/", "/index.html"):
            # a browser gets the chat page (the reference serves promeserve/web/index.html, api_handlers.h:400-430); other clients the liveness text
            page = self._web_page() if (path != "/" or "text/html" in headers.get("accept", "")) else None
            if page is not None:
                return self._send(wfile, 200, page, "text/html; charset=utf-8")
            if path != "/":
                return self._send(wfile, 404, json.dumps({"error": "not found"}).encode())
            return self._send(wfile, 200, b"PromeServe is running", "text/plain")
        if method == "GET" and path == "/api/version":
            return self._send(wfile, 200, json.dumps({"version": VERSION}).encode())
        if method == "GET" and path == "/api/tags":
            return self._send(wfile, 200, json.dumps(H.tags()).encode())
        if method == "GET" and path == "/api/ps":
            return self._send(wfile, 200, json.dumps(H.ps()).encode())
        if method == "POST" and path in ("/api/embeddings", "/api/embed"):
            # backends that can embed (the paged engine) answer; for the others this stays 501 as in the reference
            try:
                req = json.loads(raw or b"{}")
                backend = H.ensure_model(req.get("model", ""))
            except Exception:                                         # noqa: BLE001
                backend = None
            if backend is None or not hasattr(backend, "embed"):
                return self._send(wfile, 501, json.dumps({"error": "embeddings are not implemented"}).encode())
            text = req.get("prompt") if req.get("prompt") is not None else req.get("input", "")
            try:
                if isinstance(text, list):
                    out = {"model": req.get("model", ""), "embeddings": [backend.embed(str(t)) for t in text]}
                else:
                    out = {"model": req.get("model", ""), "embedding": backend.embed(str(text))}
            except Exception as e:                                    # noqa: BLE001
                return self._send(wfile, 500, json.dumps({"error": str(e)}).encode())
            return self._send(wfile, 200, json.dumps(out).encode(), "application/json")
        if method == "POST" and path in ("/api/generate", "/api/chat", "/api/show"):
            try:
                body = json.loads(raw.decode("utf-8") or "{}")
            except ValueError:
                return self._send(wfile, 400, json.dumps({"error": "invalid JSON"}).encode())
            try:
                if path == "/api/show":
                    return self._send(wfile, 200, json.dumps(H.show(body)).encode())
                H.ensure_model(body.get("model", ""))
            except KeyError as e:
                return self._send(wfile, 404, json.dumps({"error": str(e).strip("'\"")}).encode())
            fn = H.generate if path == "/api/generate" else H.chat
            if body.get("stream", True):
                wfile.write(b"HTTP/1.1 200 OK\r\nContent-Type: application/x-ndjson\r\nTransfer-Encoding: chunked\r\nConnection: close\r\n" +
                            "".join(f"{k}: {v}\r\n" for k, v in CORS.items()).encode() + b"\r\n")
                wfile.flush()
                w = StreamWriter(wfile)
                try:
                    fn(body, w)
                except Exception as e:       # errors travel in-stream
                    w.write({"error": str(e), "done": True})
                    w.finish()
                return
            try:
                return self._send(wfile, 200, json.dumps(fn(body, None)).encode())
            except Exception as e:
                return self._send(wfile, 500, json.dumps({"error": str(e)}).encode())
        return self._send(wfile, 404, json.dumps({"error": "not found"}).encode())


class PromeServe:
    def __init__(self, config: Optional[ServerConfig] = None, backends: Optional[Dict[str, ModelBackend]] = None):
        self.config = config or ServerConfig()

        def loader(name: str) -> ModelBackend:
            from ..io.ollama import resolve_model
            import os
            path = None
            if self.config.allow_model_paths:
                if os.path.isdir(name) and os.path.isfile(os.path.join(name, "config.json")):
                    return PagedBackend(name, name, self.config.device)  # a Hugging Face directory: the paged engine serves it
                path = name if os.path.isfile(name) else None
            elif os.path.isabs(name) or ".." in name.replace("\\", "/").split("/") or "/" in name or "\\" in name:
                # a request names models, not files: only model_dirs and the Ollama store are searched
                raise KeyError(f"model '{name}' not found (paths are not accepted as model names)")
            if path is None:
                for d in self.config.model_dirs:
                    stem = os.path.join(d, name.split(":")[0])
                    if os.path.isfile(stem + ".gguf"):
                        path = stem + ".gguf"
                    elif os.path.isfile(os.path.join(stem, "config.json")):
                        return PagedBackend(stem, name, self.config.device)
            if path is None:
                try:
                    path = resolve_model(name)
                except FileNotFoundError as e:
                    raise KeyError(str(e))
            if self.config.device == "cpu":
                return OracleBackend(path, name, self.config.max_seq)
            return GGUFBackend(path, name, self.config.device, self.config.max_seq)
        self.handlers = ApiHandlers(self.config, backends, loader)
        self.http = HttpServer(self.config, self.handlers)

    def start(self):
        if self.config.model:
            self.handlers.ensure_model(self.config.model)
        self.http.start()
        return self

    def stop(self):
        self.http.stop()

    @property
    def port(self):
        return self.http.port
