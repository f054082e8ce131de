"""Continuous-batching engine for Hugging Face Llama checkpoints with a paged KV cache.

Same public surface as the reference's ``LLMEngine`` (torch/serve/llm.h:33-57 for the request types, :299-334 for the
64-token page pool, :352-437 for ``load / set_weights / generate / submit_request / step / poll_responses``).  The
reference walks its active requests one after another on the CPU; here one ``step()`` is

* a prompt pass for each newly admitted request (tcgen05 GEMMs, FlashAttention over the prompt, rotary + page write
  in ``paged_rope_write_kernel``), and
* ONE batched decode pass for all other active requests: a ``[B, hidden]`` activation runs through the layer GEMMs,
  ``paged_attn_decode_kernel`` reads each request's pages through the page table, and the sampler picks the next ids
  on the device.

Pages come from one pool shared by all requests and go back to it when a request finishes.  CPU tensors take the
plain torch path of every op, which is how the scheduling logic is tested without a GPU.
"""
from __future__ import annotations

import collections
import json
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Union

import torch
import torch.nn.functional as F

from ..ops import paged as P

PAGE = P.PAGE


@dataclass
class GenerationConfig:
    max_new_tokens: int = 128
    temperature: float = 0.8
    top_p: float = 0.9
    top_k: int = 50
    repetition_penalty: float = 1.1
    stop_tokens: List[int] = field(default_factory=list)


@dataclass
class Request:
    request_id: int = 0
    prompt: Union[str, Sequence[int]] = ""
    config: GenerationConfig = field(default_factory=GenerationConfig)
    on_token: Optional[Callable[[int], bool]] = None     # called with every generated id; returning False ends the request


@dataclass
class Response:
    request_id: int = 0
    output: str = ""
    token_ids: List[int] = field(default_factory=list)
    tokens_generated: int = 0
    throughput_tok_per_s: float = 0.0


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    bos_token_id: int = 1
    eos_token_id: int = 2
    tie_word_embeddings: bool = False

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_json(cls, path: str) -> "LlamaConfig":
        with open(path) as f:
            d = json.load(f)
        c = cls()
        for k in cls.__dataclass_fields__:
            if k in d and d[k] is not None:
                v = d[k]
                if k == "eos_token_id" and isinstance(v, list):
                    v = v[0]
                setattr(c, k, type(getattr(c, k))(v))
        if "num_key_value_heads" not in d:
            c.num_key_value_heads = c.num_attention_heads
        return c


from ..io.safetensors import load_checkpoint_dir, load_file as load_safetensors, save_file as save_safetensors  # noqa: E402,F401


# ------------------------------------------------------------------------------------------ weights
class LlamaWeights:
    """Weights in the layout the engine runs: q/k/v packed into one matrix, gate/up packed into one."""

    def __init__(self, cfg: LlamaConfig):
        self.cfg = cfg
        self.tok_emb: Optional[torch.Tensor] = None
        self.layers: List[Dict[str, torch.Tensor]] = []
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head: Optional[torch.Tensor] = None

    @classmethod
    def random(cls, cfg: LlamaConfig, seed: int = 0, dtype=torch.float32, device="cpu") -> "LlamaWeights":
        """Random weights of the right scales (benchmarks and tests); drawn on ``device`` so a large model never sits in
        host memory."""
        g = torch.Generator(device=device).manual_seed(seed)
        D, I, H, Hk, Dh = cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim

        def r(*s, scale):
            return (torch.randn(*s, generator=g, device=device) * scale).to(dtype)

        def norm_w():
            return (1 + 0.1 * torch.randn(D, generator=g, device=device)).to(dtype)
        w = cls(cfg)
        w.tok_emb = r(cfg.vocab_size, D, scale=1.0)
        for _ in range(cfg.num_hidden_layers):
            w.layers.append(dict(attn_norm=norm_w(), wqkv=r((H + 2 * Hk) * Dh, D, scale=D ** -0.5), wo=r(D, H * Dh, scale=(H * Dh) ** -0.5),
                                 ffn_norm=norm_w(), w_gate_up=r(2 * I, D, scale=D ** -0.5), w_down=r(D, I, scale=I ** -0.5)))
        w.final_norm = norm_w()
        w.lm_head = r(cfg.vocab_size, D, scale=D ** -0.5)
        return w

    @classmethod
    def from_state_dict(cls, cfg: LlamaConfig, sd: Dict[str, torch.Tensor]) -> "LlamaWeights":
        """Hugging Face names: ``model.layers.N.self_attn.{q,k,v,o}_proj.weight`` and so on."""
        w = cls(cfg)
        if "embed_tokens.weight" in sd and "model.embed_tokens.weight" not in sd:          # a bare LlamaModel checkpoint
            sd = {("model." + k if not k.startswith("lm_head") else k): v for k, v in sd.items()}
        w.tok_emb = sd["model.embed_tokens.weight"]
        for l in range(cfg.num_hidden_layers):
            p = f"model.layers.{l}."
            w.layers.append(dict(
                attn_norm=sd[p + "input_layernorm.weight"],
                wqkv=torch.cat([sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"]]),
                wo=sd[p + "self_attn.o_proj.weight"], ffn_norm=sd[p + "post_attention_layernorm.weight"],
                w_gate_up=torch.cat([sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"]]), w_down=sd[p + "mlp.down_proj.weight"]))
        w.final_norm = sd["model.norm.weight"]
        w.lm_head = sd.get("lm_head.weight", w.tok_emb)
        return w

    def state_dict(self) -> Dict[str, torch.Tensor]:
        c = self.cfg
        H, Hk, Dh, I = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.intermediate_size
        sd = {"model.embed_tokens.weight": self.tok_emb, "model.norm.weight": self.final_norm, "lm_head.weight": self.lm_head}
        for l, L in enumerate(self.layers):
            p = f"model.layers.{l}."
            q, k, v = L["wqkv"].split([H * Dh, Hk * Dh, Hk * Dh])
            g, u = L["w_gate_up"].split([I, I])
            sd.update({p + "input_layernorm.weight": L["attn_norm"], p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k,
                       p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": L["wo"],
                       p + "post_attention_layernorm.weight": L["ffn_norm"], p + "mlp.gate_proj.weight": g,
                       p + "mlp.up_proj.weight": u, p + "mlp.down_proj.weight": L["w_down"]})
        return sd

    def to(self, device, dtype) -> "LlamaWeights":
        w = LlamaWeights(self.cfg)
        mv = lambda t: t.to(device=device, dtype=dtype).contiguous()
        w.tok_emb, w.final_norm, w.lm_head = mv(self.tok_emb), mv(self.final_norm), mv(self.lm_head)
        w.layers = [{k: mv(v) for k, v in L.items()} for L in self.layers]
        return w


class ByteTokenizer:
    """Fallback when a checkpoint directory has no tokenizer files: one id per UTF-8 byte (offset 3)."""
    bos_id, eos_id = 1, 2

    def encode(self, text: str, add_bos: bool = True) -> List[int]:
        return ([self.bos_id] if add_bos else []) + [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids) -> str:
        return bytes(i - 3 for i in ids if 3 <= i < 259).decode("utf-8", errors="replace")


def load_hf_tokenizer(model_dir: str):
    """``vocab.json`` + ``merges.txt``, or the ``model`` section of ``tokenizer.json`` (byte-level BPE,
    torch/serve/llm.h:94-297)."""
    from ..io.tokenizer import GGUFTokenizer
    vocab, merges = None, None
    vj, mt, tj = (os.path.join(model_dir, n) for n in ("vocab.json", "merges.txt", "tokenizer.json"))
    if os.path.exists(vj) and os.path.exists(mt):
        with open(vj, encoding="utf-8") as f:
            vocab = json.load(f)
        with open(mt, encoding="utf-8") as f:
            merges = [ln.rstrip("\n") for ln in f if ln.strip() and not ln.startswith("#version")]
    elif os.path.exists(tj):
        with open(tj, encoding="utf-8") as f:
            m = json.load(f).get("model", {})
        vocab = m.get("vocab")
        merges = [x if isinstance(x, str) else " ".join(x) for x in m.get("merges", [])]
    if not vocab:
        return None
    tokens = [""] * (max(vocab.values()) + 1)
    for t, i in vocab.items():
        tokens[i] = t
    return GGUFTokenizer(tokens, "gpt2", merges=merges)


# ------------------------------------------------------------------------------------------ KV pool
class PagedKVCache:
    """One pool of 64-token pages shared by all requests; a page id addresses the same slot in every layer."""

    def __init__(self, num_layers: int, num_kv_heads: int, head_dim: int, max_pages: int, device, dtype, spare: bool = False):
        n = max_pages + (1 if spare else 0)                # the spare page (id max_pages) is never handed out
        self.k = [torch.zeros(n, num_kv_heads, PAGE, head_dim, device=device, dtype=dtype) for _ in range(num_layers)]
        self.v = [torch.zeros(n, num_kv_heads, PAGE, head_dim, device=device, dtype=dtype) for _ in range(num_layers)]
        self.max_pages = max_pages
        self.spare_page = max_pages if spare else -1
        self.free_pages: Deque[int] = collections.deque(range(max_pages))

    def alloc_page(self) -> int:
        return self.free_pages.popleft() if self.free_pages else -1

    def free_page(self, p: int):
        self.free_pages.append(p)

    @property
    def pages_in_use(self) -> int:
        return self.max_pages - len(self.free_pages)


@dataclass
class RequestState:
    request_id: int
    config: GenerationConfig
    input_ids: List[int]
    prompt_len: int
    t_start: float
    prompt_ids: List[int] = field(default_factory=list)
    row: int = -1                        # row of the page table while active
    pages: List[int] = field(default_factory=list)
    kv_position: int = 0
    output_ids: List[int] = field(default_factory=list)
    prefill_done: bool = False
    done: bool = False
    sampler: object = None
    on_token: Optional[Callable[[int], bool]] = None
    ngram_hist: Optional[List[int]] = None               # speculative decoding: history and its n-gram index
    ngram_index: Optional[Dict[tuple, int]] = None
    ngram_done: int = 0


class LLMEngine:
    """``submit_request`` queues a prompt, ``step`` advances every active request by one token (the prompt pass for
    new ones), ``poll_responses`` hands back what finished."""

    def __init__(self, device=None, max_pages: int = 1024, max_active: int = 8, dtype=None, seed: int = 0, use_graphs: bool = True,
                 spec_tokens: int = 0):
        self.device = torch.device(device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu"))
        self.dtype = dtype if dtype is not None else (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.max_pages, self.max_active = max_pages, max_active
        self.cfg: Optional[LlamaConfig] = None
        self.weights: Optional[LlamaWeights] = None
        self.tokenizer = ByteTokenizer()
        self.kv: Optional[PagedKVCache] = None
        self.pending: Deque[RequestState] = collections.deque()
        self.active: List[RequestState] = []
        self.done: List[Response] = []
        self.loaded = False
        self._next_id = 0
        self._gen = torch.Generator().manual_seed(seed)
        self.steps = 0
        self.tokens_generated = 0
        self.launch_log: List[int] = []          # batch size of every decode pass (tests and metrics read it)
        self.use_graphs = use_graphs
        self._graphs: Dict[tuple, tuple] = {}
        # speculative decoding for greedy requests: up to `spec_tokens` ids proposed by an n-gram look-up in the request's
        # own history are verified in the same decode pass (one extra batch row per proposed id)
        self.spec_tokens = spec_tokens
        self.max_prompt_tokens = 16384           # tokens of new requests that share one prompt pass
        self.spec_drafted = self.spec_accepted = 0

    # -------------------------------------------------------------------------------------- loading
    def load(self, model_dir: str) -> bool:
        """A Hugging Face directory: ``config.json``, ``model.safetensors`` (or the shards its index lists), tokenizer."""
        cj = os.path.join(model_dir, "config.json")
        if not os.path.exists(cj):
            return False
        cfg = LlamaConfig.from_json(cj)
        sd = load_checkpoint_dir(model_dir)
        tok = load_hf_tokenizer(model_dir)
        if tok is not None:
            self.tokenizer = tok
        if not sd:
            self.cfg = cfg
            return True                           # weights may still arrive through set_weights()
        self.set_weights(LlamaWeights.from_state_dict(cfg, sd))
        return True

    def set_weights(self, w: LlamaWeights):
        self.cfg = w.cfg
        self.weights = w.to(self.device, self.dtype)
        c = self.cfg
        self.cos, self.sin = P.rope_tables(c.max_position_embeddings, c.head_dim, c.rope_theta, self.device)
        self.kv = PagedKVCache(c.num_hidden_layers, c.num_key_value_heads, c.head_dim, self.max_pages, self.device, self.dtype, spare=True)
        self.pt_stride = (c.max_position_embeddings + PAGE - 1) // PAGE
        # one row per active request plus a spare one whose single page absorbs the writes of padding rows
        self.page_table = torch.zeros(self.max_active + 1, self.pt_stride, dtype=torch.int32, device=self.device)
        self.page_table[self.max_active].fill_(self.kv.spare_page)
        self.free_rows = list(range(self.max_active))
        self._graphs = {}
        self.loaded = True

    # -------------------------------------------------------------------------------------- public API
    def generate(self, prompt, config: Optional[GenerationConfig] = None) -> Response:
        rid = self._next_id
        self.submit_request(Request(rid, prompt, config or GenerationConfig()))
        mine = None
        while mine is None:
            self.step()
            keep = []
            for r in self.done:
                if r.request_id == rid:
                    mine = r
                else:
                    keep.append(r)
            self.done = keep
            if mine is None and self.num_active() == 0:
                return Response(request_id=rid)
        return mine

    def stream(self, prompt, config: Optional[GenerationConfig] = None):
        """Generator over the ids of one request as they are produced (other queued requests keep advancing with it)."""
        rid = self._next_id
        fresh: List[int] = []
        self.submit_request(Request(rid, prompt, config or GenerationConfig(), lambda t: fresh.append(t) or True))
        while True:
            alive = any(s.request_id == rid for s in self.active) or any(s.request_id == rid for s in self.pending)
            if not alive and not fresh:
                break
            if alive:
                self.step()
            while fresh:
                yield fresh.pop(0)
        self.done = [r for r in self.done if r.request_id != rid]

    def submit_request(self, req: Request):
        ids = self._encode(req.prompt)
        self._next_id = max(self._next_id, req.request_id + 1)
        limit = self.cfg.max_position_embeddings - 1
        ids = ids[-limit:] if len(ids) > limit else ids
        self.pending.append(RequestState(req.request_id, req.config, list(ids), len(ids), time.perf_counter(), prompt_ids=list(ids),
                                         on_token=req.on_token))
        self._admit_pending()

    def cancel(self, request_id: int) -> bool:
        """Drop a queued request or end a running one at the next step (its pages go back to the pool; it still gets a
        response with what it produced).  Returns whether the id was found."""
        for s in list(self.pending):
            if s.request_id == request_id:
                self.pending.remove(s)
                self.done.append(Response(request_id=request_id))
                return True
        for s in self.active:
            if s.request_id == request_id:
                s.done = True
                if not s.prefill_done:                     # never ran: nothing to decode, and no prompt pass either
                    s.prefill_done = True
                self._collect_done()
                return True
        return False

    def stats(self) -> Dict[str, float]:
        """Counters for logs and dashboards."""
        return {"active": len(self.active), "pending": len(self.pending), "steps": self.steps,
                "pages_in_use": self.kv.pages_in_use if self.kv is not None else 0, "pages_total": self.max_pages,
                "tokens_generated": self.tokens_generated, "graphs": len(self._graphs),
                "spec_drafted": self.spec_drafted, "spec_accepted": self.spec_accepted}

    def poll_responses(self) -> List[Response]:
        out, self.done = self.done, []
        return out

    def num_active(self) -> int:
        return len(self.active) + len(self.pending)

    @torch.no_grad()
    def step(self):
        self._admit_pending()
        if not self.active:
            return
        self.steps += 1
        fresh = [s for s in self.active if not s.prefill_done]
        running = [s for s in self.active if s.prefill_done and not s.done]
        ready: List[RequestState] = []
        for s in fresh:
            if not self._ensure_pages(s, s.prompt_len - 1):
                if len(self.active) > 1:                       # wait for a running request to give its pages back
                    self.active.remove(s)
                    self.free_rows.append(s.row)
                    self.pending.appendleft(s)
                    self._held = True
                else:
                    self._finish(s)                            # the pool cannot hold this prompt at all
                continue
            ready.append(s)
        while ready:                                           # prompt passes: as many new requests as the token cap allows
            chunk, total = [], 0
            while ready and (not chunk or total + ready[0].prompt_len <= self.max_prompt_tokens):
                total += ready[0].prompt_len
                chunk.append(ready.pop(0))
            logits = self._forward_prompts(chunk)
            for i, s in enumerate(chunk):
                s.kv_position = s.prompt_len
                s.prefill_done = True
                self._emit(s, self._sample([s], logits[i:i + 1])[0])
        running = [s for s in running if self._ensure_pages(s, s.kv_position) or self._finish(s)]
        if running and self.spec_tokens > 0:
            self._step_speculative(running)
        elif running:                                          # one batched decode pass for everyone else
            logits = self._forward_decode(running)
            for s, t in zip(running, self._sample(running, logits)):
                s.kv_position += 1
                self._emit(s, t)
        finished = any(s.done for s in self.active)
        self._collect_done()
        # the kernels' status word (a page id or position outside its extent) costs a device round trip to read: look at it
        # when a request finishes and every 32 steps, not after every token
        if self.device.type == "cuda" and (finished or self.steps % 32 == 0):
            P.check_status(self.device)

    # -------------------------------------------------------------------------------------- speculative decoding
    def _draft(self, s: RequestState, k: int) -> List[int]:
        """Prompt look-up: find the latest earlier occurrence of the last 3 (then 2, then 1) ids in the request's own
        history and propose the ids that followed it (the reference drafts the same way on the CPU,
        torch/io/speculative_draft.h).  The request keeps an index from n-gram to the position after its latest
        occurrence, extended by the ids that arrived since the last call, so a look-up costs O(new ids)."""
        hist = s.prompt_ids + s.output_ids if s.ngram_hist is None else s.ngram_hist
        if s.ngram_hist is None:
            s.ngram_hist, s.ngram_index, s.ngram_done = hist, {}, 0
        else:
            hist.extend(s.output_ids[len(hist) - len(s.prompt_ids):])
        L = len(hist)
        for q in range(s.ngram_done, L - 1):                  # n-grams that end before the last id
            for n in (1, 2, 3):
                if q + 1 >= n:
                    s.ngram_index[tuple(hist[q + 1 - n:q + 1])] = q + 1
        s.ngram_done = max(s.ngram_done, L - 1)
        for n in (3, 2, 1):
            if L > n:
                at = s.ngram_index.get(tuple(hist[L - n:]))
                if at is not None:
                    return hist[at:at + k]
        return []

    def _step_speculative(self, running: List[RequestState]):
        """One decode pass in which a greedy request contributes 1 + d rows: its last id and d proposed ids at the next
        positions (row j attends to the cache up to its own position, so the rows are causal among themselves).  Row j
        is valid when all proposals before it matched the model's own choice; the request advances by 1 + matches."""
        rows, spans = [], []
        for s in running:
            greedy = s.config.temperature <= 0.0 and s.config.repetition_penalty == 1.0
            draft = self._draft(s, self.spec_tokens) if greedy else []
            room = min(s.config.max_new_tokens - len(s.output_ids) - 1, self.cfg.max_position_embeddings - 2 - s.kv_position)
            draft = draft[:max(room, 0)]
            while draft and not self._ensure_pages(s, s.kv_position + len(draft)):
                draft.pop()
            spans.append((s, len(rows), draft, greedy))
            for j, t in enumerate([s.input_ids[-1]] + draft):
                rows.append([t, s.kv_position + j, s.row, s.kv_position + j + 1])
        self.launch_log.append(len(running))
        logits = self._forward_rows(rows, min_rows=len(running) * (self.spec_tokens + 1))
        choice = logits.argmax(-1).tolist()
        for s, start, draft, greedy in spans:
            if not greedy:
                s.kv_position += 1
                self._emit(s, self._sample([s], logits[start:start + 1])[0])
                continue
            j = 0
            while True:
                tok = int(choice[start + j])
                s.kv_position += 1
                self._emit(s, tok)
                if s.done or j >= len(draft) or draft[j] != tok:
                    break
                j += 1
            self.spec_drafted += len(draft)
            self.spec_accepted += j

    # -------------------------------------------------------------------------------------- scheduling
    def _encode(self, prompt) -> List[int]:
        """Text goes through the tokenizer and starts with the BOS id; a list of ids is taken as it is."""
        if not isinstance(prompt, str):
            return [int(i) for i in prompt]
        try:
            ids = list(self.tokenizer.encode(prompt, add_bos=False))
        except TypeError:                                      # a tokenizer without the add_bos switch
            ids = list(self.tokenizer.encode(prompt))
        bos = self.cfg.bos_token_id
        if not ids or ids[0] != bos:
            ids = [bos] + ids
        return [min(max(int(i), 0), self.cfg.vocab_size - 1) for i in ids]

    def _admit_pending(self):
        if getattr(self, "_held", False) and self.active:      # a prompt is waiting for pages: admit nothing new
            return
        self._held = False
        while self.pending and self.loaded and self.free_rows and len(self.active) < self.max_active:
            s = self.pending.popleft()
            s.row = self.free_rows.pop()
            self.active.append(s)

    def _ensure_pages(self, s: RequestState, pos: int) -> bool:
        """Make sure the pages up to the one that holds ``pos`` exist; False when the pool is empty."""
        need = pos // PAGE + 1
        fresh = []
        while len(s.pages) + len(fresh) < need:
            p = self.kv.alloc_page()
            if p < 0:
                for q in fresh:
                    self.kv.free_page(q)
                return False
            fresh.append(p)
        if fresh:
            lo = len(s.pages)
            s.pages.extend(fresh)
            self.page_table[s.row, lo:lo + len(fresh)] = torch.tensor(fresh, dtype=torch.int32, device=self.device)
        return True

    def _emit(self, s: RequestState, tok: int):
        self.tokens_generated += 1
        s.output_ids.append(tok)
        s.input_ids = [tok]
        c = s.config
        if tok == self.cfg.eos_token_id or tok in c.stop_tokens or len(s.output_ids) >= c.max_new_tokens or \
                s.kv_position + 1 >= self.cfg.max_position_embeddings:
            s.done = True
        if s.on_token is not None and not s.on_token(tok):
            s.done = True

    def _finish(self, s: RequestState) -> bool:
        s.done = True
        return False

    def _collect_done(self):
        keep = []
        for s in self.active:
            if not s.done:
                keep.append(s)
                continue
            for p in s.pages:
                self.kv.free_page(p)
            s.pages = []
            self.free_rows.append(s.row)
            dt = max(time.perf_counter() - s.t_start, 1e-9)
            text = self.tokenizer.decode(s.output_ids)
            self.done.append(Response(s.request_id, text, list(s.output_ids), len(s.output_ids), len(s.output_ids) / dt))
        self.active = keep

    # -------------------------------------------------------------------------------------- model
    def _linear(self, x, w):
        if x.is_cuda:
            from ..ops.gemm import linear
            return linear(x, w)
        return F.linear(x, w)

    def _norm(self, x, w):
        from ..ops.fused_ops import rms_norm
        return rms_norm(x, w, self.cfg.rms_norm_eps)

    def _mlp(self, x, L):
        from ..ops.fused_ops import swiglu
        return self._linear(swiglu(self._linear(x, L["w_gate_up"])), L["w_down"])

    def _forward_prompt(self, s: RequestState) -> torch.Tensor:
        """All prompt tokens of one request; fills its pages; returns the logits of the last position ``[1, V]``."""
        return self._forward_prompts([s])

    @torch.no_grad()
    def embed(self, prompt) -> torch.Tensor:
        """Mean of the final-norm hidden states over the prompt's tokens, L2-normalised ``[hidden]`` fp32 (a sentence
        embedding from the decoder; the reference's server answers 501 to ``/api/embeddings``).  Call it from the thread
        that runs the engine, between steps; it borrows a page-table row and returns its pages when it is done."""
        ids = self._encode(prompt)[: self.cfg.max_position_embeddings - 1]
        if not self.free_rows:
            raise RuntimeError("embed: every page-table row is in use")
        s = RequestState(-1, GenerationConfig(), list(ids), len(ids), time.perf_counter(), prompt_ids=list(ids))
        s.row = self.free_rows.pop()
        try:
            if not self._ensure_pages(s, s.prompt_len - 1):
                raise RuntimeError("embed: the page pool cannot hold this prompt now")
            h = self._forward_prompts([s], hidden=True).float().mean(0)
            return h / h.norm().clamp_min(1e-12)
        finally:
            for p in s.pages:
                self.kv.free_page(p)
            self.free_rows.append(s.row)

    def _forward_prompts(self, batch: List[RequestState], hidden: bool = False) -> torch.Tensor:
        """The prompt pass of several new requests at once: their tokens are concatenated, so every projection is one
        GEMM over all of them; attention runs per request (requests of equal length share a call).  Fills the pages;
        returns the logits of each request's last position ``[len(batch), V]``."""
        from ..ops.attention import flash_attention
        c, w = self.cfg, self.weights
        H, Hk, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        dev = self.device
        lens = [s.prompt_len for s in batch]
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + n)
        ids = torch.tensor([t for s in batch for t in s.input_ids], dtype=torch.long)
        pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in lens])
        req = torch.cat([torch.full((n,), s.row, dtype=torch.int32) for s, n in zip(batch, lens)])
        ids, pos, req = ids.to(dev), pos.to(dev), req.to(dev)
        groups: Dict[int, List[int]] = {}
        for i, n in enumerate(lens):
            groups.setdefault(n, []).append(i)
        consecutive = all(g == list(range(g[0], g[0] + len(g))) for g in groups.values())
        x = w.tok_emb[ids]
        for l, L in enumerate(w.layers):
            qkv = self._linear(self._norm(x, L["attn_norm"]), L["wqkv"]).contiguous()
            k = P.paged_rope_write(qkv, H, Hk, Dh, pos, req, self.page_table, self.cos, self.sin, self.kv.k[l], self.kv.v[l], want_k=True)
            a = torch.empty(qkv.shape[0], H * Dh, dtype=qkv.dtype, device=dev)
            for n, members in groups.items():
                runs = [members] if consecutive else [[i] for i in members]      # equal lengths side by side: one call
                for run in runs:
                    lo, hi, nb = offs[run[0]], offs[run[-1] + 1], len(run)
                    q = qkv[lo:hi, :H * Dh].reshape(nb, n, H, Dh)
                    v = qkv[lo:hi, (H + Hk) * Dh:].reshape(nb, n, Hk, Dh)
                    a[lo:hi] = flash_attention(q, k[lo:hi].view(nb, n, Hk, Dh), v, causal=True).reshape(nb * n, H * Dh)
            x = x + self._linear(a, L["wo"])
            x = x + self._mlp(self._norm(x, L["ffn_norm"]), L)
        if hidden:                                             # the embedding path: every position after the final norm
            return self._norm(x, w.final_norm)
        last = x[torch.tensor([o - 1 for o in offs[1:]], device=dev)]
        return self._linear(self._norm(last, w.final_norm), w.lm_head).float()

    def _decode_layers(self, meta: torch.Tensor, nsplit: int) -> torch.Tensor:
        """The device work of a decode pass.  ``meta [B, 4]`` int32: token id, position, page-table row, cached length."""
        from ..ops.gemm import linear_add_rms_norm, linear_swiglu
        c, w = self.cfg, self.weights
        H, Hk, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        B = meta.shape[0]
        ids, pos, rows, lens = meta[:, 0].long(), meta[:, 1].contiguous(), meta[:, 2].long(), meta[:, 3].contiguous()
        table = self.page_table[rows]                          # [B, pt_stride] rows in batch order
        req = torch.arange(B, dtype=torch.int32, device=meta.device)
        x = w.tok_emb[ids]
        h = self._norm(x, w.layers[0]["attn_norm"])
        for l, L in enumerate(w.layers):
            q = P.qkv_rope_write(h, L["wqkv"], H, Hk, Dh, pos, req, table, self.cos, self.sin, self.kv.k[l], self.kv.v[l])
            a = P.paged_attention_decode(q, H, Hk, Dh, lens, table, self.kv.k[l], self.kv.v[l], nsplit=nsplit)
            h, x = linear_add_rms_norm(a, L["wo"], x, L["ffn_norm"], c.rms_norm_eps)
            nxt = w.layers[l + 1]["attn_norm"] if l + 1 < len(w.layers) else w.final_norm
            h, x = linear_add_rms_norm(linear_swiglu(h, L["w_gate_up"]), L["w_down"], x, nxt, c.rms_norm_eps)
        return self._linear(h, w.lm_head).float()

    def _forward_decode(self, batch: List[RequestState]) -> torch.Tensor:
        """One new token for every request of the batch; returns logits ``[B, V]``.  On a GPU the pass is a CUDA graph
        per (batch bucket, split count): the batch is padded to the bucket with rows that write to a spare page."""
        self.launch_log.append(len(batch))
        return self._forward_rows([[s.input_ids[-1], s.kv_position, s.row, s.kv_position + 1] for s in batch])

    def _forward_rows(self, rows: List[List[int]], min_rows: int = 0) -> torch.Tensor:
        """``rows``: [token id, position, page-table row, cached length] per batch row; returns logits ``[len(rows), V]``.
        ``min_rows`` keeps the graph bucket stable when the row count varies from pass to pass (speculative decoding)."""
        dev = self.device
        B = len(rows)
        rows = list(rows)
        max_len = max(r[3] for r in rows)
        Hk = self.cfg.num_key_value_heads
        if dev.type != "cuda" or not self.use_graphs:
            meta = torch.tensor(rows, dtype=torch.int32)
            meta = (meta.pin_memory() if dev.type == "cuda" else meta).to(dev, non_blocking=True)
            return self._decode_layers(meta, P.pick_splits(B, Hk, max_len))
        Bb = 1
        while Bb < max(B, min_rows):
            Bb *= 2
        nsplit = P.pick_splits(Bb, Hk, max_len)
        rows += [[0, 0, self.max_active, 1]] * (Bb - B)        # padding: the spare row of the page table
        key = (Bb, nsplit)
        if key not in self._graphs:
            self._graphs[key] = self._capture(Bb, nsplit, rows)
        graph, meta_dev, meta_host, logits = self._graphs[key]
        meta_host.copy_(torch.tensor(rows, dtype=torch.int32))
        meta_dev.copy_(meta_host, non_blocking=True)
        graph.replay()
        return logits[:B]

    def _capture(self, Bb: int, nsplit: int, rows):
        dev = self.device
        meta_host = torch.tensor(rows, dtype=torch.int32).pin_memory()
        meta_dev = meta_host.to(dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):                          # warm-up outside the capture (allocations, status words)
            self._decode_layers(meta_dev, nsplit)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits = self._decode_layers(meta_dev, nsplit)
        return graph, meta_dev, meta_host, logits

    # -------------------------------------------------------------------------------------- sampling
    def _sample(self, batch: List[RequestState], logits: torch.Tensor) -> List[int]:
        """Greedy requests share one arg-max; the others go through the device sampler (top-k <= 64) or tensor ops."""
        from ..ops.sampling import MAX_DEVICE_TOP_K, DeviceSampler, sample_batch, sample_logits
        out: List[Optional[int]] = [None] * len(batch)
        greedy = [i for i, s in enumerate(batch) if s.config.temperature <= 0.0 and s.config.repetition_penalty == 1.0]
        if greedy:
            am = logits[greedy].argmax(-1).tolist()
            for i, t in zip(greedy, am):
                out[i] = int(t)
        waiting = []                                           # indices of the requests that go through the device sampler
        for i, s in enumerate(batch):
            if out[i] is not None:
                continue
            g = s.config
            row = logits[i].contiguous()
            if logits.is_cuda and 1 <= g.top_k <= MAX_DEVICE_TOP_K:
                if s.sampler is None:
                    s.sampler = DeviceSampler(self.cfg.vocab_size, self.device, max_history=self.cfg.max_position_embeddings,
                                              seed=int(torch.randint(0, 2 ** 31 - 1, (1,), generator=self._gen)))
                    s.sampler.reset(s.prompt_ids + s.output_ids)
                waiting.append(i)
            else:
                hist = s.prompt_ids + s.output_ids
                out[i] = sample_logits(row, g.temperature, g.top_k, g.top_p, g.repetition_penalty,
                                       hist if g.repetition_penalty != 1.0 else None, generator=self._gen if not row.is_cuda else None)
        if waiting:                                            # three launches and one synchronisation for all of them
            rows = logits[waiting].contiguous() if len(waiting) != len(batch) else logits.contiguous()
            cfgs = [(batch[i].config.temperature, batch[i].config.top_k, batch[i].config.top_p, batch[i].config.repetition_penalty)
                    for i in waiting]
            for i, t in zip(waiting, sample_batch([batch[i].sampler for i in waiting], rows, cfgs)):
                out[i] = int(t)
        return [int(t) for t in out]


class EngineServer:
    """Runs an :class:`LLMEngine` on a thread of its own so that many callers (HTTP workers) share its decode batches:
    ``submit`` is thread-safe and returns at once, the scheduler thread admits the request at the next step, calls its
    ``on_token`` for every generated id and sets the returned handle's event when the request is finished."""

    class Handle:
        def __init__(self):
            import threading
            self.event = threading.Event()
            self.request_id = -1
            self.response: Optional[Response] = None
            self.t_submit = time.perf_counter()
            self.t_first: Optional[float] = None

        def wait(self, timeout: Optional[float] = None) -> Optional[Response]:
            self.event.wait(timeout)
            return self.response

    def __init__(self, engine: LLMEngine):
        import threading
        self.engine = engine
        self._cv = threading.Condition()
        self._inbox: List[tuple] = []
        self._calls: List[tuple] = []
        self._handles: Dict[int, "EngineServer.Handle"] = {}
        self._next = 0
        self._stop = False
        self.max_batch_seen = 0
        self._thread = threading.Thread(target=self._run, name="llm-engine", daemon=True)
        self._thread.start()

    def submit(self, prompt, config: GenerationConfig, on_token: Optional[Callable[[int], bool]] = None) -> "EngineServer.Handle":
        h = EngineServer.Handle()

        def hook(tok: int) -> bool:
            if h.t_first is None:
                h.t_first = time.perf_counter()
            return on_token(tok) if on_token is not None else True
        with self._cv:
            rid = self._next
            self._next += 1
            h.request_id = rid
            self._handles[rid] = h
            self._inbox.append(Request(rid, prompt, config, hook))
            self._cv.notify()
        return h

    def call(self, fn, timeout: Optional[float] = 60.0):
        """Run ``fn(engine)`` on the scheduler thread between two steps and return its result (or raise what it raised)."""
        import threading
        box = {"done": threading.Event()}
        with self._cv:
            self._calls.append((fn, box))
            self._cv.notify()
        if not box["done"].wait(timeout):
            raise TimeoutError("the engine thread did not get to the call in time")
        if "error" in box:
            raise box["error"]
        return box.get("value")

    def close(self):
        with self._cv:
            self._stop = True
            self._cv.notify()
        self._thread.join(10)

    def _run(self):
        eng = self.engine
        if eng.device.type == "cuda":
            torch.cuda.set_device(eng.device)
        while True:
            with self._cv:
                while not self._stop and not self._inbox and not self._calls and eng.num_active() == 0:
                    self._cv.wait()
                if self._stop:
                    return
                inbox, self._inbox = self._inbox, []
                calls, self._calls = self._calls, []
            for fn, box in calls:
                try:
                    box["value"] = fn(eng)
                except Exception as e:                                # noqa: BLE001
                    box["error"] = e
                box["done"].set()
            for req in inbox:
                try:
                    eng.submit_request(req)
                except Exception:                                    # a bad prompt ends that request, not the thread
                    eng.done.append(Response(request_id=req.request_id))
            if eng.num_active():
                try:
                    eng.step()
                except Exception:
                    for s in eng.active + list(eng.pending):          # fail what is in flight, keep serving
                        eng.done.append(Response(request_id=s.request_id, token_ids=list(s.output_ids), tokens_generated=len(s.output_ids)))
                    eng.active, eng.pending = [], collections.deque()
                    eng.free_rows = list(range(eng.max_active))
                    if eng.kv is not None:
                        eng.kv.free_pages = collections.deque(range(eng.kv.max_pages))
                if eng.launch_log:
                    self.max_batch_seen = max(self.max_batch_seen, eng.launch_log[-1])
                    del eng.launch_log[:-1]
            for r in eng.poll_responses():
                with self._cv:
                    h = self._handles.pop(r.request_id, None)
                if h is not None:
                    h.response = r
                    h.event.set()


# the reference's class names for the same things (torch/serve/llm.h)
KVCache = PagedKVCache
LlamaLayerWeights = Dict[str, torch.Tensor]          # one layer of LlamaWeights.layers: attn_norm, wqkv, wo, ffn_norm, w_gate_up, w_down


class ByteBPETokenizer:
    """Byte-level BPE from ``vocab.json`` + ``merges.txt`` or ``tokenizer.json`` of a checkpoint directory; falls back to one id
    per byte when the directory has neither."""

    def __init__(self, model_dir: str = None):
        self.inner = load_hf_tokenizer(model_dir) if model_dir else None
        self.fallback = ByteTokenizer()

    @property
    def vocab_size(self) -> int:
        return self.inner.vocab_size if self.inner is not None else 259

    def encode(self, text: str) -> List[int]:
        return self.inner.encode(text) if self.inner is not None else self.fallback.encode(text)

    def decode(self, ids) -> str:
        return self.inner.decode(list(ids)) if self.inner is not None else self.fallback.decode(ids)
