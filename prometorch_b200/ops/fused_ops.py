"""Autograd-aware wrappers of the bandwidth-bound training kernels
(csrc/train_kernels.cu): RMSNorm (optionally fused with the residual add),
rotary embedding, gated MLP activation and softmax cross-entropy.

CUDA tensors in bf16/fp32 go to the sm_100a kernels; CPU tensors (unit tests,
the CPU configs) take the same math written with tensor ops.  A CUDA tensor
never silently falls back: an unsupported shape raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.nn.functional as F

from .. import _native as N


@N.register_decls
def _decls(L):
    vp, ci, cf, ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
    L.ptb_rmsnorm_fwd.argtypes = [vp, vp, vp, vp, ll, ci, cf, vp, vp, ci, vp]
    L.ptb_rmsnorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ll, ci, vp, ci, vp]
    L.ptb_rope.argtypes = [vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, ci, vp]
    L.ptb_qkv_rope_split.argtypes = [vp, vp, vp, vp, vp, vp, ll, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    L.ptb_qkv_rope_split.restype = ci
    L.ptb_gated_act_fwd.argtypes = [vp, vp, ll, ci, ci, ci, vp]
    L.ptb_gated_act_bwd.argtypes = [vp, vp, vp, ll, ci, ci, ci, vp]
    L.ptb_xent.argtypes = [vp, vp, vp, vp, vp, ll, ci, ll, cf, ll, ci, vp]
    for n in ("ptb_rmsnorm_fwd", "ptb_rmsnorm_bwd", "ptb_rope", "ptb_gated_act_fwd", "ptb_gated_act_bwd", "ptb_xent"):
        getattr(L, n).restype = ci


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _is_bf16(t):
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise TypeError(f"fused kernels take bf16 or fp32 tensors, got {t.dtype}")


_SM_COUNT = {}


def _sms(dev):
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


# ----------------------------------------------------------------------------- RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, resid):
        shape = x.shape
        H = shape[-1]
        x2 = x.contiguous().view(-1, H)
        w = w.contiguous().to(x.dtype)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        r_in = resid.contiguous().view(-1, H) if resid is not None else None
        r_out = torch.empty_like(x2) if resid is not None else None
        N.check(N.lib().ptb_rmsnorm_fwd(x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, H, eps,
                                        N.ptr(r_in), N.ptr(r_out), _is_bf16(x2), _stream(x)), "rmsnorm_fwd")
        ctx.save_for_backward(r_out if resid is not None else x2, w, rstd)
        ctx.shape, ctx.has_resid = shape, resid is not None
        if resid is not None:
            return y.view(shape), r_out.view(shape)
        return y.view(shape), None

    @staticmethod
    def backward(ctx, dy, dres):
        h, w, rstd = ctx.saved_tensors
        H = h.shape[-1]
        rows = h.shape[0]
        dy2 = dy.contiguous().view(-1, H)
        dres2 = dres.contiguous().view(-1, H) if (ctx.has_resid and dres is not None) else None
        dx = torch.empty_like(h)
        dw = torch.empty_like(w)
        n_ctas = max(1, min((rows + 7) // 8, _sms(h.device) * 2))      # eight rows (warps) per CTA
        part = torch.empty(n_ctas, H, dtype=torch.float32, device=h.device)
        N.check(N.lib().ptb_rmsnorm_bwd(h.data_ptr(), w.data_ptr(), dy2.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                        part.data_ptr(), n_ctas, rows, H, N.ptr(dres2), _is_bf16(h), _stream(h)), "rmsnorm_bwd")
        dx = dx.view(ctx.shape)
        return dx, dw, None, (dx if ctx.has_resid else None)


def _rms_ref(x, w, eps):
    v = x if x.dtype == torch.float64 else x.float()          # fp32 math, except that double inputs stay double
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.to(v.dtype)).to(x.dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` over the last dimension."""
    if not x.is_cuda:
        return _rms_ref(x, weight, eps)
    return _RMSNorm.apply(x, weight, eps, None)[0]


def add_rms_norm(x: torch.Tensor, resid: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """Fused residual add + RMSNorm: returns ``(norm(x + resid), x + resid)``."""
    if not x.is_cuda:
        h = x + resid
        return _rms_ref(h, weight, eps), h
    return _RMSNorm.apply(x, weight, eps, resid)


# ----------------------------------------------------------------------------- RoPE
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, neox, pos_offset):
        B, T, Hh, D = x.shape
        xc = x.contiguous()
        y = torch.empty_like(xc)
        N.check(N.lib().ptb_rope(xc.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, Hh, D, int(neox), 0,
                                 pos_offset, _is_bf16(xc), _stream(x)), "rope")
        ctx.save_for_backward(cos, sin)
        ctx.neox, ctx.pos_offset = neox, pos_offset
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        B, T, Hh, D = dy.shape
        g = dy.contiguous()
        dx = torch.empty_like(g)
        N.check(N.lib().ptb_rope(g.data_ptr(), dx.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, Hh, D, int(ctx.neox), 1,
                                 ctx.pos_offset, _is_bf16(g), _stream(g)), "rope_bwd")
        return dx, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, neox: bool = True, pos_offset: int = 0) -> torch.Tensor:
    """Rotary embedding of ``x [B, T, heads, D]`` with fp32 tables ``[T_max, D/2]``; ``neox`` pairs
    ``(i, i + D/2)``, otherwise ``(2i, 2i+1)``."""
    if x.is_cuda:
        return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous(), neox, pos_offset)
    T = x.shape[1]
    wide = torch.float64 if x.dtype == torch.float64 else torch.float32       # fp32 math, except that double inputs stay double
    c = cos[pos_offset:pos_offset + T].to(wide)[None, :, None, :]
    s = sin[pos_offset:pos_offset + T].to(wide)[None, :, None, :]
    xf = x.to(wide)
    if neox:
        h = x.shape[-1] // 2
        a, b = xf[..., :h], xf[..., h:]
        return torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)
    a, b = xf[..., 0::2], xf[..., 1::2]
    return torch.stack([a * c - b * s, b * c + a * s], -1).flatten(-2).to(x.dtype)


class _QkvRopeSplit(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, H, Hk, D, neox, pos_offset):
        B, T = qkv.shape[0], qkv.shape[1]
        p = qkv.contiguous().view(B * T, (H + 2 * Hk) * D)
        q = torch.empty(B, T, H, D, dtype=qkv.dtype, device=qkv.device)
        k = torch.empty(B, T, Hk, D, dtype=qkv.dtype, device=qkv.device)
        v = torch.empty(B, T, Hk, D, dtype=qkv.dtype, device=qkv.device)
        N.check(N.lib().ptb_qkv_rope_split(p.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * T, T, H,
                                           Hk, D, int(neox), pos_offset, 0, _is_bf16(p), _stream(p)), "qkv_rope_split")
        ctx.save_for_backward(cos, sin)
        ctx.meta = (B, T, H, Hk, D, neox, pos_offset, qkv.shape)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin = ctx.saved_tensors
        B, T, H, Hk, D, neox, pos_offset, shape = ctx.meta
        dq, dk, dv = dq.contiguous(), dk.contiguous(), dv.contiguous()
        dqkv = torch.empty(B * T, (H + 2 * Hk) * D, dtype=dq.dtype, device=dq.device)
        N.check(N.lib().ptb_qkv_rope_split(dqkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), cos.data_ptr(), sin.data_ptr(), B * T, T,
                                           H, Hk, D, int(neox), pos_offset, 1, _is_bf16(dq), _stream(dq)), "qkv_rope_split_bwd")
        return dqkv.view(shape), None, None, None, None, None, None, None


def qkv_rope_split(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, cos: torch.Tensor, sin: torch.Tensor,
                   neox: bool = True, pos_offset: int = 0):
    """``qkv [B, T, (H + 2 Hk) D]`` (q heads, k heads, v heads) -> rotated ``q [B, T, H, D]``, rotated ``k`` and ``v``
    ``[B, T, Hk, D]``, contiguous, in one pass (the split, both rotary embeddings and the copies of the three slices)."""
    H, Hk, D = num_heads, num_kv_heads, head_dim
    if qkv.is_cuda and D % 16 == 0:
        return _QkvRopeSplit.apply(qkv, cos.float().contiguous(), sin.float().contiguous(), H, Hk, D, neox, pos_offset)
    B, T = qkv.shape[0], qkv.shape[1]
    x = qkv.view(B, T, H + 2 * Hk, D)
    return rope(x[:, :, :H], cos, sin, neox, pos_offset), rope(x[:, :, H:H + Hk], cos, sin, neox, pos_offset), x[:, :, H + Hk:]


# ----------------------------------------------------------------------------- gated activation
class _GatedAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, gelu):
        I = gu.shape[-1] // 2
        g2 = gu.contiguous().view(-1, 2 * I)
        out = torch.empty(g2.shape[0], I, dtype=gu.dtype, device=gu.device)
        N.check(N.lib().ptb_gated_act_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], I, int(gelu), _is_bf16(g2), _stream(gu)), "gated_act")
        ctx.save_for_backward(g2)
        ctx.gelu, ctx.shape = gelu, gu.shape
        return out.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        I = g2.shape[-1] // 2
        d = dout.contiguous().view(-1, I)
        dgu = torch.empty_like(g2)
        N.check(N.lib().ptb_gated_act_bwd(g2.data_ptr(), d.data_ptr(), dgu.data_ptr(), g2.shape[0], I, int(ctx.gelu), _is_bf16(g2), _stream(g2)), "gated_act_bwd")
        return dgu.view(ctx.shape), None


def swiglu(gate_up: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """``act(gate) * up`` for a packed tensor ``[..., 2*I]`` (gate first); SiLU, or tanh-GELU with ``gelu``."""
    if gate_up.is_cuda:
        return _GatedAct.apply(gate_up, gelu)
    g, u = gate_up.chunk(2, dim=-1)
    return (F.gelu(g, approximate="tanh") if gelu else F.silu(g)) * u


# ----------------------------------------------------------------------------- cross entropy
class _Xent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, ignore_index, inplace):
        V = logits.shape[-1]
        l2 = logits.view(-1, V) if logits.is_contiguous() else logits.contiguous().view(-1, V)
        rows = l2.shape[0]
        if l2.stride(0) % 8:          # the kernel reads 8 elements per access: give odd vocabularies a padded pitch
            pad = torch.empty(rows, (V + 7) // 8 * 8, dtype=l2.dtype, device=l2.device)
            pad[:, :V] = l2
            l2, inplace = pad[:, :V], True
        tgt = target.reshape(-1).to(torch.int64).contiguous()
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        need_grad = logits.requires_grad
        n_valid = (tgt != ignore_index).sum().clamp_min(1)
        dl = None
        if need_grad:
            dl = l2 if inplace else torch.empty_like(l2)
        # gradient of the MEAN loss is written in the same pass; 1/n_valid is applied in backward
        N.check(N.lib().ptb_xent(l2.data_ptr(), tgt.data_ptr(), loss.data_ptr(), 0, N.ptr(dl), rows, V, l2.stride(0), 1.0,
                                 ignore_index, _is_bf16(l2), _stream(logits)), "cross_entropy")
        if need_grad:
            ctx.save_for_backward(dl, n_valid)
        ctx.shape = logits.shape
        return loss.sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        dl, n_valid = ctx.saved_tensors
        dl.mul_((g / n_valid).to(dl.dtype))
        return dl.reshape(ctx.shape), None, None, None


def cross_entropy(logits: torch.Tensor, target: torch.Tensor, ignore_index: int = -100, inplace_grad: bool = False) -> torch.Tensor:
    """Mean softmax cross-entropy over rows of ``logits [..., V]`` with int64 ``target``.  The kernel
    computes loss and gradient in one sweep; ``inplace_grad`` lets the gradient overwrite ``logits``
    (saves a ``rows x V`` buffer when the caller no longer needs the logits)."""
    if not logits.is_cuda:
        return F.cross_entropy(logits.float().view(-1, logits.shape[-1]), target.reshape(-1), ignore_index=ignore_index)
    return _Xent.apply(logits, target, ignore_index, inplace_grad)
