"""Attention front end: ``flash_attention(q, k, v, causal)`` on ``[B, T, heads, D]`` tensors with
grouped-query heads (``heads_q`` a multiple of ``heads_kv``).

CUDA bf16 inputs with D in {64, 128} run the hand-written FlashAttention kernels: the forward on
tcgen05 tensor cores with TMEM accumulators and TMA-fed tiles (csrc/flash_attn_sm100.cu; it also returns the
log-sum-exp), the recompute-based backward with the GQA reduction of dK/dV done inside the kernel
(csrc/flash_attn.cu, which also holds an mma.sync forward selected by PTB_FA_SM100=0).  ``q_offset`` /
``return_lse`` are the hooks a ring/context-parallel wrapper needs: blocks of K/V can be processed
separately and merged by log-sum-exp.  CPU tensors use the plain softmax formulation.  The layout
matches the reference's kernel, which also takes ``[B, N, H, D]`` (aten/src/ATen/native/Attention.h:244-250)."""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native as N


@N.register_decls
def _decls(L):
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    if hasattr(L, "ptb_flash_attn_fwd"):
        L.ptb_flash_attn_fwd.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp]
        L.ptb_flash_attn_fwd.restype = ci
        L.ptb_flash_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp]
        L.ptb_flash_attn_bwd.restype = ci
    if hasattr(L, "ptb_flash_attn_fwd_sm100"):
        L.ptb_flash_attn_fwd_sm100.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp, vp]
        L.ptb_flash_attn_fwd_sm100.restype = ci
    if hasattr(L, "ptb_flash_attn_bwd_sm100"):
        L.ptb_flash_attn_bwd_sm100.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, ci, vp, vp]
        L.ptb_flash_attn_bwd_sm100.restype = ci


def _use_tcgen05() -> bool:
    """The forward runs on tcgen05/TMEM (csrc/flash_attn_sm100.cu) unless PTB_FA_SM100=0 selects the mma.sync kernel."""
    import os
    return os.environ.get("PTB_FA_SM100", "1") != "0" and hasattr(N.lib(), "ptb_flash_attn_fwd_sm100")


def attention_reference(q, k, v, causal=True, q_offset: int = 0, scale: Optional[float] = None):
    """Plain softmax attention in fp32 (oracle and CPU path).  Returns ``(out, lse)``."""
    B, Tq, H, D = q.shape
    Tk, Hk = k.shape[1], k.shape[2]
    g = H // Hk
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    wide = torch.float64 if q.dtype == torch.float64 else torch.float32       # fp32 math, except that double inputs stay double
    qf = q.to(wide).permute(0, 2, 1, 3)
    kf = k.to(wide).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    vf = v.to(wide).permute(0, 2, 1, 3).repeat_interleave(g, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(Tq, device=q.device)[:, None] + q_offset
        ki = torch.arange(Tk, device=q.device)[None, :]
        s = s.masked_fill(ki > qi, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vf)
    return o.permute(0, 2, 1, 3).to(q.dtype), lse


class _Flash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, q_offset, scale):
        B, Tq, H, D = q.shape
        Tk, Hk = k.shape[1], k.shape[2]
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o = torch.empty_like(q)
        lse = torch.empty(B, H, Tq, dtype=torch.float32, device=q.device)
        st = torch.cuda.current_stream(q.device).cuda_stream
        if _use_tcgen05():
            from .gemm import _status
            N.check(N.lib().ptb_flash_attn_fwd_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, Tq, Tk,
                                                     H, Hk, D, int(causal), scale, q_offset, _status(q.device).data_ptr(), st),
                    "flash_attn_fwd_sm100")
        else:
            N.check(N.lib().ptb_flash_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, Tq, Tk, H, Hk,
                                               D, int(causal), scale, q_offset, st), "flash_attn_fwd")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.q_offset, ctx.scale = causal, q_offset, scale
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        B, Tq, H, D = q.shape
        Tk, Hk = k.shape[1], k.shape[2]
        do = do.contiguous()
        import os
        sm100_bwd = os.environ.get("PTB_FA_BWD_SM100", "1") != "0" and hasattr(N.lib(), "ptb_flash_attn_bwd_sm100")
        # the tcgen05 path clears the fp32 dQ accumulator inside its delta pass
        dq32 = (torch.empty if sm100_bwd else torch.zeros)(B, Tq, H, D, dtype=torch.float32, device=q.device)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty(B, H, Tq, dtype=torch.float32, device=q.device)
        st = torch.cuda.current_stream(q.device).cuda_stream
        if sm100_bwd:
            from .gemm import _status
            # few KV heads: split each head's query group over several CTAs until the grid fills the GPU twice over
            gs, base, group = 1, ((Tk + 127) // 128) * Hk * B, H // Hk
            while base * gs < 296 and group % (gs * 2) == 0:
                gs *= 2
            if gs > 1:
                dk = torch.empty((gs,) + tuple(k.shape), dtype=k.dtype, device=k.device)
                dv = torch.empty((gs,) + tuple(v.shape), dtype=v.dtype, device=v.device)
            N.check(N.lib().ptb_flash_attn_bwd_sm100(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                                     delta.data_ptr(), dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, Tq, Tk, H, Hk, D,
                                                     int(ctx.causal), ctx.scale, ctx.q_offset, gs, _status(q.device).data_ptr(), st),
                    "flash_attn_bwd_sm100")
            if gs > 1:
                dk, dv = dk.sum(0, dtype=torch.float32).to(k.dtype), dv.sum(0, dtype=torch.float32).to(v.dtype)
        else:
            N.check(N.lib().ptb_flash_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr(), lse.data_ptr(),
                                               delta.data_ptr(), dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), 0, B, Tq, Tk, H, Hk, D,
                                               int(ctx.causal), ctx.scale, ctx.q_offset, st), "flash_attn_bwd")
        return dq32.to(q.dtype), dk, dv, None, None, None


def flash_attention(q, k, v, causal: bool = True, q_offset: int = 0, scale: Optional[float] = None, return_lse: bool = False):
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if q.is_cuda and q.dtype == torch.bfloat16 and D in (64, 128) and q.shape[2] % k.shape[2] == 0 and \
            hasattr(N.lib(), "ptb_flash_attn_fwd"):
        o, lse = _Flash.apply(q, k, v, causal, q_offset, scale)
    else:
        o, lse = attention_reference(q, k, v, causal, q_offset, scale)
    return (o, lse) if return_lse else o
