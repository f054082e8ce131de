"""bf16 GEMM on tcgen05 tensor cores (csrc/gemm_sm100.cuh) and the linear layer built on it.

``gemm_bf16`` exposes the kernel's operand majors directly; ``linear`` is the autograd function
``y = x W^T + b`` whose backward runs the other two products on the same kernel without materialising
a transpose: ``dX = dY W`` reads ``W`` as an N-major operand and ``dW = dY^T X`` reads both operands
M/N-major.  The reference's linear layers go through fp32 cublasSgemm
(torch/csrc/autograd/autograd.h:931-940, aten/src/ATen/cuda/CUDABlas.cu:455-479)."""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from .. import _native as N

EPI_BIAS, EPI_ACCUM, EPI_OUT_F32, EPI_GELU, EPI_SCATTER_ADD, EPI_SCATTER_STORE = 1, 2, 4, 8, 16, 32


@N.register_decls
def _decls(L):
    vp, ci, ll = C.c_void_p, C.c_int, C.c_longlong
    L.ptb_gemm_bf16.argtypes = [vp, ll, ci, vp, ll, ci, vp, ll, ci, ci, ci, vp, ci, vp, ci, vp]
    L.ptb_gemm_bf16.restype = ci
    if hasattr(L, "ptb_gemm_bf16_splitk"):
        L.ptb_gemm_pick_splits.argtypes = [ci, ci, ci, ci]
        L.ptb_gemm_pick_splits.restype = ci
        L.ptb_gemm_bf16_splitk.argtypes = [vp, ll, vp, ll, vp, ll, ci, ci, ci, vp, ci, ci, vp, vp, ci, vp]
        L.ptb_gemm_bf16_splitk.restype = ci
    if hasattr(L, "ptb_gemm_bf16_splitk_add_norm"):
        cf = C.c_float
        L.ptb_gemm_bf16_splitk_add_norm.argtypes = [vp, ll, vp, ll, ci, ci, ci, ci, vp, vp, vp, vp, cf, vp, vp, ci, vp]
        L.ptb_gemm_bf16_splitk_add_norm.restype = ci
        L.ptb_gemm_bf16_splitk_gated.argtypes = [vp, ll, vp, ll, ci, ci, ci, ci, vp, ci, vp, vp, ci, vp]
        L.ptb_gemm_bf16_splitk_gated.restype = ci


_STATUS = {}


def _status(dev):
    if dev not in _STATUS:
        _STATUS[dev] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _STATUS[dev]


def check_status(dev=None):
    """Raise if any GEMM launched on ``dev`` reported a timed-out wait."""
    for d, s in _STATUS.items():
        if dev is None or d == dev:
            if int(s) != 0:
                s.zero_()
                raise N.NativeError("tcgen05 GEMM: a pipeline wait timed out (status %d)" % int(s))


_SPLITK = os.environ.get("PTB_GEMM_SPLITK", "1") != "0"
_SM_COUNT = {}


def _sms(dev) -> int:
    k = torch.device(dev).index or 0
    if k not in _SM_COUNT:
        _SM_COUNT[k] = torch.cuda.get_device_properties(k).multi_processor_count
    return _SM_COUNT[k]


def _rowmajor(t):
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("operand must be a 2-D tensor with a contiguous last dimension")
    return t


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: Optional[torch.Tensor] = None,
              bias: Optional[torch.Tensor] = None, accumulate: bool = False, out_dtype=torch.bfloat16, gelu: bool = False):
    """``C[M,N] (+)= A B^T``.  ``a``: ``[M,K]`` (or ``[K,M]`` with ``a_mn``); ``b``: ``[N,K]`` (or ``[K,N]`` with ``b_mn``)."""
    a, b = _rowmajor(a), _rowmajor(b)
    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16 or not a.is_cuda:
        raise TypeError("gemm_bf16 takes CUDA bf16 operands")
    M, K = (a.shape[1], a.shape[0]) if a_mn else a.shape
    Nn, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    if K != Kb:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an output tensor")
        out = torch.empty(M, Nn, dtype=out_dtype, device=a.device)
    if M <= 128 and not (a_mn or b_mn or accumulate) and out.dtype == torch.bfloat16 and Nn % 4 == 0 and _SPLITK:
        # skinny M (decode batches): swapped operands with a narrow token tile and / or K split over the idle SMs
        splits = N.lib().ptb_gemm_pick_splits(M, Nn, K, _sms(a.device))         # 0: the ordinary kernel is the better choice
        if splits > 0:
            work = torch.empty(splits * M * Nn, dtype=torch.float32, device=a.device)
            st = torch.cuda.current_stream(a.device).cuda_stream
            N.check(N.lib().ptb_gemm_bf16_splitk(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), out.data_ptr(), out.stride(0), M, Nn,
                                                 K, N.ptr(bias.float().contiguous() if bias is not None else None), int(gelu), splits,
                                                 work.data_ptr(), _status(a.device).data_ptr(), 0, st), "gemm_bf16_splitk")
            return out
    flags = (EPI_BIAS if bias is not None else 0) | (EPI_ACCUM if accumulate else 0) | \
        (EPI_OUT_F32 if out.dtype == torch.float32 else 0) | (EPI_GELU if gelu else 0)
    if bias is not None:
        bias = bias.float().contiguous()
    st = torch.cuda.current_stream(a.device).cuda_stream
    N.check(N.lib().ptb_gemm_bf16(a.data_ptr(), a.stride(0), int(a_mn), b.data_ptr(), b.stride(0), int(b_mn), out.data_ptr(),
                                  out.stride(0), M, Nn, K, N.ptr(bias), flags, _status(a.device).data_ptr(), 0, st), "gemm_bf16")
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        y = gemm_bf16(x2, w, bias=bias)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm_bf16(dy2, w, b_mn=True).view(ctx.xshape)          # dX[M,in] = dY[M,out] W[out,in]
        if ctx.needs_input_grad[1]:
            dw = gemm_bf16(dy2, x2, a_mn=True, b_mn=True)                 # dW[out,in] = dY^T X
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x W^T + b``.  CUDA bf16 runs on the tcgen05 kernel; other inputs use ``torch.nn.functional.linear``."""
    if x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0:
        return _Linear.apply(x, weight, bias)
    return torch.nn.functional.linear(x, weight, bias)


def _skinny_splits(x: torch.Tensor, w: torch.Tensor) -> int:
    """Split count for ``x [M, K] @ w[N, K]^T`` when the fused split-K path applies, else 0."""
    if not (_SPLITK and x.is_cuda and x.dim() == 2 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= 128
            and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] % 8 == 0 and w.shape[0] % 8 == 0
            and hasattr(N.lib(), "ptb_gemm_bf16_splitk_add_norm")):
        return 0
    return N.lib().ptb_gemm_pick_splits(x.shape[0], w.shape[0], x.shape[1], _sms(x.device))


def linear_add_rms_norm(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, norm_w: torch.Tensor, eps: float):
    """``h = x W^T + resid``; returns ``(rmsnorm(h) * norm_w, h)``.  For decode-sized batches the sum of the split-K
    partials, the residual add and the norm are one launch after the GEMM (inference path, no autograd)."""
    splits = _skinny_splits(x, w)
    if splits and w.shape[0] <= 8192 and resid.is_contiguous() and norm_w.dtype == torch.bfloat16 and not torch.is_grad_enabled():
        M, K, Nn = x.shape[0], x.shape[1], w.shape[0]
        work = torch.empty(splits * M * Nn, dtype=torch.float32, device=x.device)
        h, y = torch.empty_like(resid), torch.empty_like(resid)
        st = torch.cuda.current_stream(x.device).cuda_stream
        N.check(N.lib().ptb_gemm_bf16_splitk_add_norm(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), M, Nn, K, splits, work.data_ptr(),
                                                      resid.data_ptr(), h.data_ptr(), norm_w.data_ptr(), float(eps), y.data_ptr(),
                                                      _status(x.device).data_ptr(), 0, st), "gemm_bf16_splitk_add_norm")
        return y, h
    from .fused_ops import add_rms_norm
    return add_rms_norm(linear(x, w), resid, norm_w, eps)


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """``act(x Wg^T) * (x Wu^T)`` for the packed weight ``[2 I, K]`` (gate rows first); the split-K sum and the gate
    share a launch for decode-sized batches (inference path, no autograd)."""
    splits = _skinny_splits(x, w_gate_up)
    if splits and not torch.is_grad_enabled():
        M, K, Nn = x.shape[0], x.shape[1], w_gate_up.shape[0]
        work = torch.empty(splits * M * Nn, dtype=torch.float32, device=x.device)
        out = torch.empty(M, Nn // 2, dtype=torch.bfloat16, device=x.device)
        st = torch.cuda.current_stream(x.device).cuda_stream
        N.check(N.lib().ptb_gemm_bf16_splitk_gated(x.data_ptr(), x.stride(0), w_gate_up.data_ptr(), w_gate_up.stride(0), M, Nn, K, splits,
                                                   work.data_ptr(), int(gelu), out.data_ptr(), _status(x.device).data_ptr(), 0, st),
                "gemm_bf16_splitk_gated")
        return out
    from .fused_ops import swiglu
    if x.is_cuda:
        return swiglu(linear(x, w_gate_up), gelu)
    return swiglu(torch.nn.functional.linear(x, w_gate_up), gelu)
