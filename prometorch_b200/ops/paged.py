"""Paged KV cache ops: rotary + page write, and one-token attention over a page table.

CUDA tensors go through ``paged_rope_write_kernel`` / ``paged_attn_decode_kernel`` (csrc/paged_attn.cu); CPU tensors
take the plain torch path below, which is also the oracle of the GPU tests.  The page layout is the reference's
(64-token pages from one pool, torch/serve/llm.h:299-334), kept as one tensor ``[page, kv_head, 64, D]`` per layer.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from .. import _native as N

PAGE = 64


@N.register_decls
def _decls(L):
    vp, ci, cf, cll = C.c_void_p, C.c_int, C.c_float, C.c_longlong
    if hasattr(L, "ptb_paged_rope_write"):
        L.ptb_paged_rope_write.argtypes = [vp, ci, ci, ci, ci, vp, vp, vp, ci, ci, vp, vp, ci, vp, vp, vp, vp, vp]
        L.ptb_paged_rope_write.restype = ci
        L.ptb_paged_attn_decode.argtypes = [vp, cll, vp, ci, ci, ci, ci, vp, vp, ci, ci, vp, vp, cf, vp, ci, vp, vp]
        L.ptb_paged_attn_decode.restype = ci
        L.ptb_paged_attn_work_floats.argtypes = [ci, ci, ci, ci]
        L.ptb_paged_attn_work_floats.restype = cll
    if hasattr(L, "ptb_paged_rope_write_partials"):
        L.ptb_paged_rope_write_partials.argtypes = [vp, ci, vp, ci, ci, ci, ci, vp, vp, vp, ci, ci, vp, vp, ci, vp, vp, vp, vp]
        L.ptb_paged_rope_write_partials.restype = ci
        L.ptb_gemm_bf16_splitk_partials.argtypes = [vp, cll, vp, cll, ci, ci, ci, ci, vp, vp, ci, vp]
        L.ptb_gemm_bf16_splitk_partials.restype = ci


_STATUS = {}


def _status(dev) -> torch.Tensor:
    d = torch.device(dev)
    k = d.index if d.index is not None else torch.cuda.current_device()
    if k not in _STATUS:
        _STATUS[k] = torch.zeros(1, dtype=torch.int32, device=torch.device('cuda', k))
    return _STATUS[k]


def check_status(dev):
    """Raise if a paged kernel met a page id or position outside its extent (it skipped the access)."""
    s = int(_status(dev).item())
    if s:
        _status(dev).zero_()
        raise IndexError(f"paged KV kernel reported status {s} (index outside the page pool)")


def rope_tables(max_pos: int, head_dim: int, theta: float, device) -> tuple:
    """cos / sin ``[max_pos, D/2]`` in fp32 for pairs (j, j + D/2)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def _cuda_ok(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and hasattr(N.lib(), "ptb_paged_rope_write")


def paged_rope_write(qkv: torch.Tensor, H: int, Hk: int, D: int, pos: torch.Tensor, req: torch.Tensor, page_table: torch.Tensor,
                     cos: torch.Tensor, sin: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                     want_k: bool = False) -> Optional[torch.Tensor]:
    """Rotate q (in place) and k of the ``n`` tokens in ``qkv [n, (H + 2 Hk) D]`` and store k, v at
    ``page_table[req[i], pos[i] // 64]``, slot ``pos[i] % 64``.  Returns the rotated keys ``[n, Hk, D]`` if asked."""
    n = qkv.shape[0]
    k_out = torch.empty(n, Hk, D, dtype=qkv.dtype, device=qkv.device) if want_k else None
    if _cuda_ok(qkv):
        assert qkv.is_contiguous() and pos.dtype == torch.int32 and req.dtype == torch.int32 and page_table.dtype == torch.int32
        st = torch.cuda.current_stream(qkv.device).cuda_stream
        N.check(N.lib().ptb_paged_rope_write(qkv.data_ptr(), n, H, Hk, D, pos.data_ptr(), req.data_ptr(), page_table.data_ptr(),
                                             page_table.stride(0), k_pages.shape[0], cos.data_ptr(), sin.data_ptr(), cos.shape[0],
                                             k_pages.data_ptr(), v_pages.data_ptr(), N.ptr(k_out), _status(qkv.device).data_ptr(), st),
                "paged_rope_write")
        return k_out
    half = D // 2
    x = qkv.view(n, H + 2 * Hk, D)
    p = pos.long()
    c, s = cos[p][:, None, :], sin[p][:, None, :]
    qk = x[:, :H + Hk].float()
    a, b = qk[..., :half], qk[..., half:]
    rot = torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(qkv.dtype)
    x[:, :H + Hk] = rot
    pages = page_table[req.long(), p // PAGE].long()
    k_pages[pages, :, p % PAGE] = rot[:, H:]
    v_pages[pages, :, p % PAGE] = x[:, H + Hk:]
    if want_k:
        k_out.copy_(rot[:, H:])
    return k_out


def qkv_rope_write(h: torch.Tensor, wqkv: torch.Tensor, H: int, Hk: int, D: int, pos, req, page_table, cos, sin, k_pages, v_pages,
                   fuse_sum: bool = False):
    """``qkv = h Wqkv^T`` followed by :func:`paged_rope_write`; returns a tensor whose first ``H D`` columns are the rotated q.  For
    decode-sized CUDA batches the projection stays as split-K partials and the rotary kernel sums them while it
    reads (no reduce launch, no bf16 round trip of k and v) when ``fuse_sum`` is set.  That is off by default: the
    rotary kernel is one CTA per token and sums the partials with scalar loads, and the decode pass of the 16-layer
    2048-wide model measured 1.24 ms with it against 1.15 ms with the separate, vectorised reduce launch."""
    from .gemm import _skinny_splits, _status as gemm_status, linear
    splits = _skinny_splits(h, wqkv) if h.is_cuda else 0
    if fuse_sum and splits and hasattr(N.lib(), "ptb_paged_rope_write_partials") and not torch.is_grad_enabled():
        n, K, width = h.shape[0], h.shape[1], wqkv.shape[0]
        work = torch.empty(splits * n * width, dtype=torch.float32, device=h.device)
        q = torch.empty(n, H * D, dtype=torch.bfloat16, device=h.device)
        st = torch.cuda.current_stream(h.device).cuda_stream
        real = N.lib().ptb_gemm_bf16_splitk_partials(h.data_ptr(), h.stride(0), wqkv.data_ptr(), wqkv.stride(0), n, width, K, splits,
                                                     work.data_ptr(), gemm_status(h.device).data_ptr(), 0, st)
        N.check(min(real, 0), "gemm_bf16_splitk_partials")
        N.check(N.lib().ptb_paged_rope_write_partials(work.data_ptr(), real, q.data_ptr(), n, H, Hk, D, pos.data_ptr(), req.data_ptr(),
                                                      page_table.data_ptr(), page_table.stride(0), k_pages.shape[0], cos.data_ptr(),
                                                      sin.data_ptr(), cos.shape[0], k_pages.data_ptr(), v_pages.data_ptr(),
                                                      _status(h.device).data_ptr(), st), "paged_rope_write_partials")
        return q
    qkv = linear(h, wqkv) if h.is_cuda else torch.nn.functional.linear(h, wqkv)
    paged_rope_write(qkv, H, Hk, D, pos, req, page_table, cos, sin, k_pages, v_pages)
    return qkv


def pick_splits(B: int, Hk: int, max_len: int, sms: int = 148) -> int:
    """Splits of the page walk.  A CTA is four warps with a few KB of loads in flight each, so the kernel wants about
    eight CTAs per SM to saturate HBM; a split should still own two pages or more.  The page count is rounded up to a
    power of two so that the choice (a key of the engine's graph cache) changes rarely as a context grows."""
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    bucket = 1
    while bucket < pages:
        bucket *= 2
    return int(max(1, min(16, bucket // 2, (8 * sms) // max(1, B * Hk))))


def paged_attention_decode(q: torch.Tensor, H: int, Hk: int, D: int, lens: torch.Tensor, page_table: torch.Tensor,
                           k_pages: torch.Tensor, v_pages: torch.Tensor, scale: Optional[float] = None, nsplit: int = 1,
                           max_len: Optional[int] = None) -> torch.Tensor:
    """``q [B, >= H D]`` (one new token per request, heads packed along the row) against each request's pages.
    ``lens[b]`` counts the cached tokens including the new one.  Returns ``[B, H D]``."""
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if _cuda_ok(q) and D in (64, 128) and H // Hk in (1, 2, 4, 8):
        out = torch.empty(B, H * D, dtype=q.dtype, device=q.device)
        work = torch.empty(int(N.lib().ptb_paged_attn_work_floats(B, H, D, nsplit)), dtype=torch.float32, device=q.device) \
            if nsplit > 1 else None
        st = torch.cuda.current_stream(q.device).cuda_stream
        N.check(N.lib().ptb_paged_attn_decode(q.data_ptr(), q.stride(0), out.data_ptr(), B, H, Hk, D, lens.data_ptr(),
                                              page_table.data_ptr(), page_table.stride(0), k_pages.shape[0], k_pages.data_ptr(),
                                              v_pages.data_ptr(), float(scale), N.ptr(work), nsplit, _status(q.device).data_ptr(), st),
                "paged_attn_decode")
        return out
    return paged_attention_reference(q, H, Hk, D, lens, page_table, k_pages, v_pages, scale)


def paged_attention_reference(q, H, Hk, D, lens, page_table, k_pages, v_pages, scale=None) -> torch.Tensor:
    """fp32 softmax attention over the gathered pages (oracle and CPU path)."""
    B = q.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    G = H // Hk
    out = torch.zeros(B, H * D, dtype=q.dtype, device=q.device)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        pages = page_table[b, :(n + PAGE - 1) // PAGE].long()
        k = k_pages[pages].float().permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :n]          # [Hk, n, D]
        v = v_pages[pages].float().permute(1, 0, 2, 3).reshape(Hk, -1, D)[:, :n]
        qb = q[b, :H * D].float().view(Hk, G, D)
        s = torch.einsum("kgd,knd->kgn", qb, k) * scale
        o = torch.einsum("kgn,knd->kgd", torch.softmax(s, dim=-1), v)
        out[b] = o.reshape(H * D).to(q.dtype)
    return out
