"""Gated linear recurrence ``h[t] = g[t] * h[t-1] + x[t]`` along dim 1 of ``[B, T, D]`` tensors (the PIR example's
``parallel_scan``: aten/src/ATen/cuda/CUDAKernels.cu:869-906 forward, ``ParallelScanBackward`` in
torch/csrc/autograd/functions/MathBackward.h).  CUDA tensors run the chunked two-pass scan of ``csrc/scan.cu``, forward
and backward; everything else takes the step-by-step loop below, which is also the oracle of the tests."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native as N


@N.register_decls
def _decls(L):
    vp, ci, cll = C.c_void_p, C.c_int, C.c_longlong
    if hasattr(L, "ptb_linear_scan_fwd"):
        L.ptb_linear_scan_scratch_floats.argtypes = [ci, ci, ci]
        L.ptb_linear_scan_scratch_floats.restype = cll
        L.ptb_linear_scan_fwd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, vp]
        L.ptb_linear_scan_fwd.restype = ci
        L.ptb_linear_scan_bwd.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp]
        L.ptb_linear_scan_bwd.restype = ci


def linear_scan_reference(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """Step by step in fp32 (differentiable through autograd)."""
    gf, xf = g.float(), x.float()
    h = torch.zeros_like(xf[:, 0])
    out = []
    for t in range(x.shape[1]):
        h = gf[:, t] * h + xf[:, t]
        out.append(h)
    return torch.stack(out, 1).to(x.dtype)


def _native_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dim() == 3 and t.dtype in (torch.bfloat16, torch.float32) and hasattr(N.lib(), "ptb_linear_scan_fwd")


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, x):
        g, x = g.contiguous(), x.contiguous()
        B, T, D = x.shape
        h = torch.empty_like(x)
        agg = torch.empty(int(N.lib().ptb_linear_scan_scratch_floats(B, T, D)), dtype=torch.float32, device=x.device)
        st = torch.cuda.current_stream(x.device).cuda_stream
        N.check(N.lib().ptb_linear_scan_fwd(g.data_ptr(), x.data_ptr(), h.data_ptr(), agg.data_ptr(), B, T, D,
                                            int(x.dtype == torch.bfloat16), st), "linear_scan_fwd")
        ctx.save_for_backward(g, h)
        return h

    @staticmethod
    def backward(ctx, dh):
        g, h = ctx.saved_tensors
        dh = dh.contiguous()
        B, T, D = h.shape
        dx, dg = torch.empty_like(h), torch.empty_like(h)
        agg = torch.empty(int(N.lib().ptb_linear_scan_scratch_floats(B, T, D)), dtype=torch.float32, device=h.device)
        st = torch.cuda.current_stream(h.device).cuda_stream
        N.check(N.lib().ptb_linear_scan_bwd(g.data_ptr(), h.data_ptr(), dh.data_ptr(), dx.data_ptr(), dg.data_ptr(), agg.data_ptr(), B, T, D,
                                            int(h.dtype == torch.bfloat16), st), "linear_scan_bwd")
        return dg, dx


def linear_scan(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``h[:, t] = g[:, t] * h[:, t-1] + x[:, t]`` with ``h[:, -1] = 0``; ``g`` and ``x`` are ``[B, T, D]`` of one dtype."""
    if g.shape != x.shape or g.dtype != x.dtype:
        raise ValueError("linear_scan: gates and inputs must agree in shape and dtype")
    if _native_ok(x) and g.is_cuda:
        return _Scan.apply(g, x)
    return linear_scan_reference(g, x)


parallel_scan = linear_scan          # the reference's name for the op
