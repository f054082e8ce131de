"""Gradient norm, clipping and the non-finite check as multi-tensor launches.

``clip_grad_norm_(params, max_norm)`` has the reference's contract
(torch/nn/utils/clip_grad.h:29-188: returns the total norm, scales gradients in place when the
norm exceeds ``max_norm``).  On CUDA the norm, the clip coefficient and the non-finite flag stay
on the device: :class:`GradNormClipper` hands the coefficient to the fused optimizer step as a
device scalar, so clipping costs no host synchronisation."""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional

import torch

from .. import _native as N
from .optimizers import TensorTable


class _G:
    """A (tensor, gradient) pair for gradients that do not live in ``.grad`` (bf16 buckets)."""

    def __init__(self, grad):
        self.grad = grad

    def numel(self):
        return self.grad.numel()

    def data_ptr(self):
        return self.grad.data_ptr()


def _grads(params):
    if torch.is_tensor(params):
        params = [params]
    return [p for p in params if p.grad is not None]


def grads_as_params(grads):
    """Wrap bare gradient tensors so the norm/clip helpers accept them."""
    return [_G(g) for g in grads]


class GradNormClipper:
    """Reusable device-side norm/clip state for a fixed parameter list."""

    def __init__(self, params: Iterable[torch.Tensor], max_norm: float = 0.0):
        self.params = [p for p in params]
        self.max_norm = float(max_norm)
        self._tables = {}
        self.out = None           # [norm, coefficient]
        self.found_inf = None

    @torch.no_grad()
    def compute(self, extra_scale: float = 1.0):
        """Launch the norm kernels; returns the device tensor ``[total_norm, clip_coef * extra_scale]``."""
        ps = _grads(self.params)
        if not ps:
            return torch.zeros(2)
        dev = ps[0].grad.device
        lib = N.lib()
        if self.out is None:
            self.out = torch.zeros(2, device=dev)
            self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        self.found_inf.zero_()
        st = torch.cuda.current_stream(dev).cuda_stream
        groups = [[p for p in ps if p.grad.dtype == dt] for dt in (torch.float32, torch.bfloat16)]
        if sum(len(g) for g in groups) != len(ps) or (groups[0] and groups[1]):
            # mixed or unusual dtypes: tensor-op fallback
            norm = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(p.grad.float()) for p in ps]))
            coef = (self.max_norm / (norm + 1e-6)).clamp(max=1.0) if self.max_norm > 0 else torch.ones_like(norm)
            self.out = torch.stack([norm, coef * extra_scale])
            self.found_inf = (~torch.isfinite(norm)).to(torch.int32).reshape(1)
            self._last = ("tensor_ops", list(ps))      # scale_grads() multiplies with tensor ops for this call
            return self.out
        bf16 = bool(groups[1])
        sub = groups[1] if bf16 else groups[0]
        tab = self._tables.setdefault(bf16, TensorTable())
        tab.build(sub, [p.grad for p in sub], [(None, None, None)] * len(sub), [None] * len(sub), dev)
        if getattr(tab, "partial", None) is None or tab.partial.numel() < tab.n_chunks:
            tab.partial = torch.empty(max(tab.n_chunks, 1), device=dev)
        N.check(lib.ptb_multi_tensor_grad_norm(tab.rows.data_ptr(), tab.chunks.data_ptr(), tab.n_chunks, int(bf16),
                                               tab.partial.data_ptr(), self.max_norm, extra_scale, self.out.data_ptr(),
                                               self.found_inf.data_ptr(), st), "grad_norm")
        self._last = (tab, bf16)
        return self.out

    @torch.no_grad()
    def scale_grads(self):
        """Multiply the gradients by the coefficient computed by :meth:`compute` (device-side)."""
        tab, bf16 = self._last
        if tab == "tensor_ops":
            for p in bf16:
                p.grad.mul_(self.out[1].to(p.grad.dtype))
            return
        dev = self.out.device
        st = torch.cuda.current_stream(dev).cuda_stream
        N.check(N.lib().ptb_multi_tensor_scale(tab.rows.data_ptr(), tab.chunks.data_ptr(), tab.n_chunks, int(bf16),
                                               self.out[1:].data_ptr(), st), "grad scale")


@torch.no_grad()
def clip_grad_norm_(parameters, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    ps = _grads(parameters)
    if not ps:
        return torch.tensor(0.0)
    fused = norm_type == 2.0 and all(p.grad.is_cuda and p.grad.is_contiguous() for p in ps) and \
        len({p.grad.dtype for p in ps}) == 1 and ps[0].grad.dtype in (torch.float32, torch.bfloat16)
    if fused:
        c = GradNormClipper(ps, max_norm)
        out = c.compute()
        c.scale_grads()
        return out[0].clone()
    if norm_type == float("inf"):
        total = torch.stack([p.grad.detach().abs().max() for p in ps]).max()
    else:
        total = torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(p.grad.detach().float(), norm_type) for p in ps]), norm_type)
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for p in ps:
        p.grad.mul_(coef.to(p.grad.device))
    return total


@torch.no_grad()
def clip_grad_value_(parameters, clip_value: float):
    for p in _grads(parameters):
        p.grad.clamp_(-clip_value, clip_value)
