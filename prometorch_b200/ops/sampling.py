"""Token sampling on the device: repetition penalty, temperature, top-k, top-p.

The reference copies the full logits vector to the host and sorts there
(torch/io/gguf_model.h:7658-7748), which makes sampling 1.84x slower than
greedy decoding.  Here everything stays on the GPU and only the chosen id (4
bytes) crosses PCIe.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _native as N

MAX_DEVICE_TOP_K = 64


@N.register_decls
def _decls(L):
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    if hasattr(L, "ptb_sample_logits"):
        L.ptb_sample_logits.argtypes = [vp, ci, vp, ci, ci, cf, cf, ci, cf, cf, vp, vp, vp, vp]
        L.ptb_sample_logits.restype = ci
    if hasattr(L, "ptb_sample_logits_batch"):
        L.ptb_sample_logits_batch.argtypes = [vp, ci, ci, vp, vp]
        L.ptb_sample_logits_batch.restype = ci
        L.ptb_sample_batch_param_bytes.argtypes = [ci]
        L.ptb_sample_batch_param_bytes.restype = C.c_longlong


class SampleRequest(C.Structure):
    """Mirrors ``PtbSampleRequest`` (csrc/ptb200_types.h)."""
    _fields_ = [("logits", C.c_void_p), ("history", C.c_void_p), ("scratch", C.c_void_p), ("out", C.c_void_p), ("n_hist", C.c_int),
                ("hist_cap", C.c_int), ("top_k", C.c_int), ("pad", C.c_int), ("repeat_penalty", C.c_float), ("temperature", C.c_float),
                ("top_p", C.c_float), ("u", C.c_float)]


_BATCH_PARAMS = {}


def sample_batch(samplers, logits: torch.Tensor, configs) -> list:
    """Sample one id for each of ``len(samplers)`` requests in three launches (grid row = request) and one host
    synchronisation.  ``logits``: ``[n, V]`` fp32 contiguous; ``configs``: per request ``(temperature, top_k, top_p,
    repeat_penalty)``.  Every :class:`DeviceSampler` keeps its own history and scratch, as with :meth:`DeviceSampler.sample`."""
    n = len(samplers)
    if n == 0:
        return []
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous() and logits.shape[0] == n
    dev = logits.device
    V = logits.shape[1]
    reqs = (SampleRequest * n)()
    for i, (s, (temperature, top_k, top_p, repeat_penalty)) in enumerate(zip(samplers, configs)):
        assert 1 <= top_k <= MAX_DEVICE_TOP_K and s.V == V
        if not s._u:
            s._u = torch.rand(4096, generator=s.gen).tolist()
        r = reqs[i]
        r.logits, r.history, r.scratch, r.out = logits[i].data_ptr(), s.hist.data_ptr(), s.scratch.data_ptr(), s.out.data_ptr()
        r.n_hist, r.hist_cap, r.top_k = s.n_hist, s.hist.numel(), int(top_k)
        r.repeat_penalty, r.temperature, r.top_p, r.u = float(repeat_penalty), float(temperature), float(top_p), float(s._u.pop())
    key = (dev.index, n)
    need = int(N.lib().ptb_sample_batch_param_bytes(n))
    if key not in _BATCH_PARAMS or _BATCH_PARAMS[key].numel() < need:
        _BATCH_PARAMS[key] = torch.empty(need, dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    N.check(min(0, N.lib().ptb_sample_logits_batch(C.addressof(reqs), n, V, _BATCH_PARAMS[key].data_ptr(), st)), "sample_logits_batch")
    for s in samplers:
        if s.n_hist < s.hist.numel():
            s.n_hist += 1                                     # the kernel appended its choice
    return torch.stack([s.out for s in samplers])[:, 0].tolist()


class DeviceSampler:
    """One-launch sampling for a fixed vocabulary: repetition penalty, temperature, top-k (<= 64), top-p and the
    inverse-CDF draw run in ``sample_kernel`` (csrc/sampling.cu); only the chosen id crosses to the host.  The
    history lives on the device and grows by one id per call."""

    def __init__(self, vocab: int, device, max_history: int = 1 << 16, seed: int = 42):
        self.V, self.device = vocab, torch.device(device)
        self.hist = torch.zeros(max_history, dtype=torch.int32, device=self.device)
        self.n_hist = 0
        self.scratch = torch.zeros(64 + 4096 * 4 + 4096 * 8 + vocab * 4 + 256, dtype=torch.uint8, device=self.device)
        self.out = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.gen = torch.Generator().manual_seed(seed)
        self._u = []

    def reset(self, history: Sequence[int] = ()):
        h = torch.as_tensor(list(history)[-self.hist.numel():], dtype=torch.int32)
        self.n_hist = h.numel()
        self.hist[:self.n_hist].copy_(h)

    def push(self, tid: int):
        """Append an id that did not come from :meth:`sample` (the kernel appends its own choice)."""
        if self.n_hist < self.hist.numel():
            self.hist[self.n_hist] = int(tid)
            self.n_hist += 1

    def sample_async(self, logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repeat_penalty: float = 1.0,
                     u: Optional[float] = None, ctrl_token_ptr: int = 0) -> torch.Tensor:
        """Launch the sampling kernels and return the device tensor ``[id, probability bits]`` without waiting for it, so
        that a batch of samplers costs one host synchronisation."""
        assert logits.is_cuda and logits.dtype == torch.float32 and logits.is_contiguous() and 1 <= top_k <= MAX_DEVICE_TOP_K
        if u is None:
            if not self._u:
                self._u = torch.rand(4096, generator=self.gen).tolist()
            u = self._u.pop()
        st = torch.cuda.current_stream(self.device).cuda_stream
        N.check(min(0, N.lib().ptb_sample_logits(logits.data_ptr(), logits.numel(), self.hist.data_ptr(), self.n_hist, self.hist.numel(),
                                                 float(repeat_penalty), float(temperature), int(top_k), float(top_p), float(u),
                                                 self.scratch.data_ptr(), self.out.data_ptr(), ctrl_token_ptr or None, st)),
                "sample_logits")
        if self.n_hist < self.hist.numel():
            self.n_hist += 1                                  # the kernel appended its choice
        return self.out

    def sample(self, logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repeat_penalty: float = 1.0,
               u: Optional[float] = None, ctrl_token_ptr: int = 0) -> int:
        return int(self.sample_async(logits, temperature, top_k, top_p, repeat_penalty, u, ctrl_token_ptr)[0])


def sample_reference(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, repeat_penalty: float, history, u: float) -> int:
    """The kernel's algorithm in plain fp32 tensor ops (oracle): penalty, top-k by (value desc, id asc), softmax at
    temperature, shortest prefix reaching ``top_p``, inverse-CDF draw with ``u``."""
    x = logits.float().clone().cpu()
    if repeat_penalty != 1.0 and len(history):
        idx = torch.as_tensor(sorted(set(int(t) for t in history)), dtype=torch.long)
        v = x[idx]
        x[idx] = torch.where(v > 0, v / repeat_penalty, v * repeat_penalty)
    order = sorted(range(x.numel()), key=lambda i: (-float(x[i]), i))[:top_k] if x.numel() <= 4096 else None
    if order is None:
        vals, ids = torch.topk(x, top_k)
        order = [int(i) for i in ids]
        order.sort(key=lambda i: (-float(x[i]), i))
    vals = x[order]
    if temperature <= 0:
        return order[0]
    e = torch.exp(vals / temperature - vals[0] / temperature)
    z = float(e.sum())
    n_keep, kept = top_k, z
    if 0.0 < top_p < 1.0:
        n_keep, kept = 0, 0.0
        for i in range(top_k):
            if kept >= top_p * z:
                break
            kept += float(e[i])
            n_keep += 1
    target, cum = u * kept, 0.0
    for i in range(n_keep):
        cum += float(e[i])
        if target < cum:
            return order[i]
    return order[n_keep - 1]


def sample_logits(logits: torch.Tensor, temperature: float = 0.7, top_k: int = 40, top_p: float = 0.9,
                  repeat_penalty: float = 1.0, history: Optional[Sequence[int]] = None,
                  generator: Optional[torch.Generator] = None) -> int:
    x = logits.float().clone()
    if repeat_penalty != 1.0 and history:
        idx = torch.as_tensor(sorted(set(int(t) for t in history)), device=x.device, dtype=torch.long)
        v = x[idx]
        x[idx] = torch.where(v > 0, v / repeat_penalty, v * repeat_penalty)
    if temperature <= 0.0:
        return int(x.argmax())
    x = x / temperature
    if top_k and top_k < x.numel():
        vals, ids = torch.topk(x, top_k)
    else:
        vals, ids = torch.sort(x, descending=True)
    probs = torch.softmax(vals, dim=-1)
    if 0.0 < top_p < 1.0:
        cum = probs.cumsum(-1)
        keep = cum - probs < top_p          # always keeps the first
        probs = torch.where(keep, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    choice = torch.multinomial(probs, 1, generator=generator)
    return int(ids[choice])
