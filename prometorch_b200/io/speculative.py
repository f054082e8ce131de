"""Low-rank speculative output projection: pick the next token without computing every logit exactly.

``W[vocab, hidden]`` is approximated once by ``U[vocab, r] @ V[r, hidden]`` (randomised range finder with two power
iterations, then an SVD of the small projected matrix).  A decode step computes ``z = V x`` and the approximate logits
``U z``, takes the ``candidate_k`` best, computes those few logits EXACTLY from the quantised rows and returns the
exact best of them: the result equals the full arg-max whenever the true winner is among the candidates.  Traffic per
token is ``vocab * r`` (bf16) instead of the whole quantised matrix.

Same contract as the reference's ``LowRankOutputProj`` (torch/io/speculative_decode.h:72-500: ``init_from_float``,
``init_from_quantized``, ``decode_greedy``, ``decode_sample`` with softmax over the exact candidates); the factorisation
and both passes are tensor programs here and run on the model's device.
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
