"""Python entry points for the dequant-GEMV and decode-attention kernels.

These wrap the C ABI for tests, micro-benchmarks and eager use; the decode
engine calls the same kernels from C++ inside its CUDA graph.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _native as N
from ..io.gguf_model import PackedWeight

EPI_STORE, EPI_RESID, EPI_GATED, EPI_ARGMAX = 0, 1, 2, 3


def _require_cuda(t: torch.Tensor):
    if not t.is_cuda:
        raise RuntimeError("this operator runs on CUDA tensors only")


def _status(dev) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=dev)


def quant_gemv(w: PackedWeight, x: torch.Tensor, *, w2: Optional[PackedWeight] = None,
               norm_weight: Optional[torch.Tensor] = None, eps: float = 1e-6, resid: Optional[torch.Tensor] = None,
               gelu: bool = False, argmax: bool = False, n_ctas: Optional[int] = None):
    """``y = W x`` for a packed Q4_K/Q6_K matrix and an fp32 vector.

    ``norm_weight``: RMS-normalise ``x`` first.  ``w2``: gated pair, returns
    ``act(W x) * (W2 x)``.  ``resid``: returns ``resid + W x``.  ``argmax``:
    additionally returns the index of the largest output.
    """
    _require_cuda(x)
    lib = N.lib()
    dev = x.device
    x = x.float().contiguous()
    assert x.numel() == w.cols, (x.shape, w.cols)
    out = torch.empty(w.rows, dtype=torch.float32, device=dev)
    if n_ctas is None:
        n_ctas = torch.cuda.get_device_properties(dev).multi_processor_count
    n_ctas = min(n_ctas, w.rows)
    epi = EPI_ARGMAX if argmax else EPI_GATED if w2 is not None else EPI_RESID if resid is not None else EPI_STORE
    scratch = torch.zeros(64 + 8 * n_ctas + 64, dtype=torch.uint8, device=dev)
    status = _status(dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    N.check(lib.ptb_gemv(w.data.data_ptr(), N.ptr(w2.data) if w2 is not None else 0, w.qtype, w.rows, w.cols, w.rowbytes, w.layout,
                         x.data_ptr(), N.ptr(norm_weight), eps, N.ptr(w.bias), N.ptr(resid), out.data_ptr(), epi,
                         int(gelu), n_ctas, scratch.data_ptr(), status.data_ptr(), st), "quant_gemv")
    if argmax:
        idx = scratch[8:12].view(torch.int32)
        return out, idx
    return out


def attn_decode(q, k, v, k_cache, v_cache, pos: int, cos, sin, *, q_norm=None, k_norm=None, neox=True, eps=1e-6,
                window: int = 0):
    """One-token attention: writes the new K/V (after optional per-head RMSNorm and RoPE) at
    ``pos`` into the fp16 caches ``[kv_heads, max_seq, d]`` (d = 64, 128 or 256) and returns ``[heads*d]``."""
    _require_cuda(q)
    lib = N.lib()
    dev = q.device
    kvh, max_seq, d = k_cache.shape
    heads = q.numel() // d
    group = heads // kvh
    splits = (max_seq + 127) // 128
    out = torch.empty(heads * d, dtype=torch.float32, device=dev)
    part_o = torch.empty(kvh * splits * group * d, dtype=torch.float32, device=dev)
    part_ml = torch.empty(kvh * splits * group * 2, dtype=torch.float32, device=dev)
    ticket = torch.zeros(kvh, dtype=torch.int32, device=dev)
    ctrl = torch.zeros(8, dtype=torch.int32, device=dev)
    ctrl[1] = pos
    st = torch.cuda.current_stream(dev).cuda_stream
    N.check(lib.ptb_attn_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), N.ptr(q_norm), N.ptr(k_norm), cos.data_ptr(),
                                sin.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
                                part_o.data_ptr(), part_ml.data_ptr(), ticket.data_ptr(), ctrl.data_ptr(), kvh, group, d,
                                max_seq, int(neox), eps, window, st), "attn_decode")
    return out
