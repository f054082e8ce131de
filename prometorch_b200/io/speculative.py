"""Speculative decoding: a low-rank output projection, and a draft model verified in batched passes.

*Low-rank output projection* (the reference's ``LowRankOutputProj``): pick the next token without computing every logit
exactly.

``W[vocab, hidden]`` is approximated once by ``U[vocab, r] @ V[r, hidden]`` (randomised range finder with two power
iterations, then an SVD of the small projected matrix).  A decode step computes ``z = V x`` and the approximate logits
``U z``, takes the ``candidate_k`` best, computes those few logits EXACTLY from the quantised rows and returns the
exact best of them: the result equals the full arg-max whenever the true winner is among the candidates.  Traffic per
token is ``vocab * r`` (bf16) instead of the whole quantised matrix.

Same contract as the reference's ``LowRankOutputProj`` (torch/io/speculative_decode.h:72-500: ``init_from_float``,
``init_from_quantized``, ``decode_greedy``, ``decode_sample`` with softmax over the exact candidates); the factorisation
and both passes are tensor programs here and run on the model's device.

*Draft model* (:func:`speculative_generate`): a small GGUF model proposes ``k`` greedy tokens with its decode engine, the
target model scores all of them in ONE batched prompt pass (tcgen05 GEMMs + FlashAttention, logits at every position) and
keeps the longest agreeing prefix plus its own next token.  The output is the target's greedy continuation under the
batched pass; rejected positions of either KV cache are simply overwritten later.
"""
from __future__ import annotations

from typing import Optional

import torch

from .gguf_quant import GGMLType, dequantize


class LowRankOutputProj:
    def __init__(self, rank: int = 256, candidate_k: int = 64, dtype=torch.float32):
        self.rank, self.candidate_k, self.dtype = int(rank), int(candidate_k), dtype
        self.U: Optional[torch.Tensor] = None       # [vocab, r]  (left factor times the singular values)
        self.V: Optional[torch.Tensor] = None       # [r, hidden]
        self.S: Optional[torch.Tensor] = None       # singular values (diagnostics)
        self._raw = None                            # quantised rows for the exact pass, or
        self._W = None                              # a float matrix
        self._qtype, self._cols = None, 0
        self.last_candidates: Optional[torch.Tensor] = None
        self.last_exact: Optional[torch.Tensor] = None

    @property
    def valid(self) -> bool:
        return self.U is not None

    @torch.no_grad()
    def init_from_float(self, W: torch.Tensor, rank: Optional[int] = None, seed: int = 42, keep_exact: bool = True):
        vocab, hidden = W.shape
        r = min(int(rank or self.rank), vocab, hidden)
        l = min(r + 20, hidden)
        g = torch.Generator(device="cpu").manual_seed(seed)
        Wf = W.float()
        omega = torch.randn(hidden, l, generator=g).to(Wf.device)
        Q, _ = torch.linalg.qr(Wf @ omega)                         # range of W, [vocab, l]
        for _ in range(2):                                         # power iterations sharpen the spectrum
            Z, _ = torch.linalg.qr(Wf.t() @ Q)
            Q, _ = torch.linalg.qr(Wf @ Z)
        B = Q.t() @ Wf                                             # [l, hidden]
        Ub, S, Vt = torch.linalg.svd(B, full_matrices=False)
        self.U = ((Q @ Ub[:, :r]) * S[:r]).to(self.dtype).contiguous()
        self.V = Vt[:r].to(self.dtype).contiguous()
        self.S, self.rank = S[:r].clone(), r
        if keep_exact and self._raw is None:
            self._W = W
        return self

    @torch.no_grad()
    def init_from_quantized(self, raw: torch.Tensor, qtype, cols: int, rank: Optional[int] = None, device=None, chunk: int = 16384):
        """``raw``: the matrix's rows as stored in the GGUF file (uint8 ``[vocab, row_bytes]``).  The float copy used for
        the factorisation is dropped afterwards; the exact pass dequantises only the candidate rows."""
        self._qtype, self._cols = GGMLType(qtype), int(cols)
        dev = torch.device(device) if device is not None else raw.device
        self._raw = raw.to(dev)
        W = torch.cat([dequantize(self._raw[i:i + chunk], self._qtype, cols) for i in range(0, raw.shape[0], chunk)])
        return self.init_from_float(W, rank, keep_exact=False)

    def _exact(self, idx: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        rows = dequantize(self._raw[idx], self._qtype, self._cols) if self._raw is not None else self._W[idx].float()
        return rows @ x.float()

    @torch.no_grad()
    def candidates(self, x: torch.Tensor) -> torch.Tensor:
        approx = self.U @ (self.V @ x.to(self.dtype))
        return approx.float().topk(min(self.candidate_k, approx.numel())).indices

    @torch.no_grad()
    def decode_greedy(self, x: torch.Tensor) -> int:
        if not self.valid:
            return -1
        idx = self.candidates(x)
        exact = self._exact(idx, x)
        self.last_candidates, self.last_exact = idx, exact
        return int(idx[exact.argmax()])

    @torch.no_grad()
    def decode_sample(self, x: torch.Tensor, temperature: float = 1.0, top_k: int = 40, generator=None) -> int:
        """Softmax over the exact logits of the best ``top_k`` candidates."""
        if not self.valid:
            return -1
        if temperature <= 0:
            return self.decode_greedy(x)
        idx = self.candidates(x)
        exact = self._exact(idx, x)
        self.last_candidates, self.last_exact = idx, exact
        k = min(int(top_k), exact.numel()) if top_k > 0 else exact.numel()
        v, j = exact.topk(k)
        p = torch.softmax(v / temperature, dim=0)
        return int(idx[j[torch.multinomial(p, 1, generator=generator)]])


@torch.no_grad()
def speculative_generate(target, draft, prompt, max_new_tokens: int = 64, k: int = 4, stop_ids=()):
    """Greedy generation of ``target`` (a ``GGUFModel`` with batched prefill) sped up by ``draft`` (a smaller
    ``GGUFModel`` over the same vocabulary).  Returns ``(tokens, stats)`` with ``stats = {"target_passes", "accepted",
    "proposed"}``."""
    if not target.supports_prefill:
        raise NotImplementedError("the target model has no batched prompt pass")
    prompt = [int(t) for t in prompt]
    stop = set(int(s) for s in stop_ids)
    out = []
    stats = {"target_passes": 0, "accepted": 0, "proposed": 0}
    # the target scores the whole prompt once; its arg-max at the last position is the first new token
    logits = target.prefill(prompt, 0, return_logits=True)
    stats["target_passes"] += 1
    nxt = int(logits[-1].argmax())
    for pos, t in enumerate(prompt):                       # the draft's cache follows the same tokens
        draft.forward_decode(t, pos)
    n_ctx = len(prompt)                                    # positions whose KV both models hold
    while len(out) < max_new_tokens and nxt not in stop:
        out.append(nxt)
        if len(out) >= max_new_tokens or n_ctx + k + 1 >= min(target.max_seq, draft.max_seq):
            break
        # draft proposes k tokens after `nxt`
        prop, t = [], nxt
        for i in range(k):
            t = draft.forward_decode(t, n_ctx + i)
            prop.append(t)
        stats["proposed"] += k
        # target scores [nxt, prop[0], ..., prop[k-1]] in one pass: row i predicts the token after position n_ctx + i
        lg = target.prefill([nxt] + prop, n_ctx, return_logits=True)
        stats["target_passes"] += 1
        choice = lg.argmax(-1).tolist()
        a = 0
        while a < k and prop[a] == choice[a]:
            a += 1
        stats["accepted"] += a
        hit_stop = False
        for tok in prop[:a]:
            if tok in stop or len(out) >= max_new_tokens:
                hit_stop = True
                break
            out.append(tok)
        if hit_stop:
            break
        nxt = choice[a]
        if a == k:                                         # the draft has not seen its own last proposal yet
            draft.forward_decode(prop[-1], n_ctx + k)
        n_ctx += a + 1
    return out[:max_new_tokens], stats


# ---------------------------------------------------------------------------------------------- n-gram draft and statistics
from dataclasses import dataclass as _dataclass  # noqa: E402
from typing import Dict as _Dict, List as _List, Sequence as _Sequence, Tuple as _Tuple  # noqa: E402


@_dataclass
class SpecStats:
    """Counters of a speculative run (torch/io/speculative_decode.h): proposals made, proposals the target agreed with, and
    target passes taken."""
    proposed: int = 0
    accepted: int = 0
    target_passes: int = 0

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.proposed if self.proposed else 0.0

    def tokens_per_pass(self, generated: int) -> float:
        return generated / self.target_passes if self.target_passes else 0.0


class NgramDraft:
    """A draft "model" that needs no weights: it proposes the ids that followed the most recent earlier occurrence of the
    last ``n`` ids (longest n first) in the sequence so far.  The index is kept incrementally, so a proposal costs a few
    dictionary look-ups (torch/io/speculative_draft.h; the batching engine uses the same scheme, serve/llm.py)."""

    def __init__(self, max_n: int = 3, min_n: int = 1):
        self.max_n, self.min_n = max_n, min_n
        self.hist: _List[int] = []
        self.index: _Dict[_Tuple[int, ...], int] = {}
        self.done = 0

    def reset(self, history: _Sequence[int] = ()):
        self.hist, self.index, self.done = list(history), {}, 0

    def append(self, token: int):
        self.hist.append(int(token))

    def _update(self):
        L = len(self.hist)
        for q in range(self.done, L - 1):                        # n-grams that end before the last id
            for n in range(self.min_n, self.max_n + 1):
                if q + 1 - n >= 0:
                    self.index[tuple(self.hist[q + 1 - n:q + 1])] = q + 1
        self.done = max(self.done, L - 1)

    def propose(self, k: int) -> _List[int]:
        """Up to ``k`` ids that followed the latest earlier match of the current suffix; empty when nothing matches."""
        self._update()
        L = len(self.hist)
        for n in range(min(self.max_n, L), self.min_n - 1, -1):
            at = self.index.get(tuple(self.hist[L - n:]))
            if at is not None:
                return self.hist[at:at + k]
        return []


class SlidingWindowAttention:
    """Decode attention over the last ``window`` positions plus one summary position per KV head: the running mean of the
    keys and of the values that left the window (a lossy approximation for long contexts, torch/io/sliding_window_attn.h).
    ``window = 0`` is full attention.  One instance per layer; ``step(q, k, v)`` takes the new token's ``q [H, D]``,
    ``k [Hk, D]``, ``v [Hk, D]`` and returns the attention output ``[H, D]``."""

    def __init__(self, n_heads: int, n_kv_heads: int, head_dim: int, window: int = 512):
        self.H, self.Hk, self.D, self.window = n_heads, n_kv_heads, head_dim, window
        self.k: _List[torch.Tensor] = []
        self.v: _List[torch.Tensor] = []
        self.k_summary = torch.zeros(n_kv_heads, head_dim)
        self.v_summary = torch.zeros(n_kv_heads, head_dim)
        self.n_summarized = 0

    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        self.k.append(k.float())
        self.v.append(v.float())
        if self.window and len(self.k) > self.window:            # the oldest position moves into the running means
            ko, vo = self.k.pop(0), self.v.pop(0)
            self.n_summarized += 1
            self.k_summary += (ko - self.k_summary) / self.n_summarized
            self.v_summary += (vo - self.v_summary) / self.n_summarized
        K, V = torch.stack(self.k, 1), torch.stack(self.v, 1)    # [Hk, T, D]
        if self.n_summarized:
            K, V = torch.cat([self.k_summary[:, None], K], 1), torch.cat([self.v_summary[:, None], V], 1)
        g = self.H // self.Hk
        qh = q.float().view(self.Hk, g, self.D)
        s = torch.einsum("kgd,ktd->kgt", qh, K) / self.D ** 0.5
        return torch.einsum("kgt,ktd->kgd", torch.softmax(s, -1), V).reshape(self.H, self.D).to(q.dtype)
