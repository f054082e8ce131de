"""Sequence-parallel column/row linear layers as autograd functions.

Two implementations with the same numerics:

* process-group path — all-gather / reduce-scatter collectives around a local GEMM (CPU ranks,
  and the NCCL baseline on GPUs);
* fused path (``tp.symm`` set, CUDA bf16) — the collective is folded into the tcgen05 GEMM:
  all-gather -> GEMM reads each A (or B) tile straight from the peer that owns those tokens through
  a per-peer TMA tensor map or staged once per launch by a few CTAs; GEMM -> reduce-scatter stores each
  bf16 output tile into this rank's slot of its owner's buffer over NVLink from the epilogue (16-byte
  stores; the owner sums the slots).  Activations to be read by peers are staged in symmetric
  memory (one local copy), and flag barriers order "written" before "read".
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Tuple

import torch

from ... import _native as N
from ...distributed.ddp import PeerChannel, _ptr_array
from ...ops.gemm import EPI_OUT_F32, EPI_SCATTER_ADD, EPI_SCATTER_STORE, _status, gemm_bf16, linear as fused_linear


@N.register_decls
def _decls(L):
    vp, ci, ll = C.c_void_p, C.c_int, C.c_longlong
    pp = C.POINTER(C.c_void_p)
    L.ptb_gemm_bf16_ex.argtypes = [pp, ci, ci, ll, ci, pp, ci, ci, ll, ci, vp, ll, pp, ci, ci, ci, ci, ci, vp, ci, vp, ci, vp, vp, vp]
    L.ptb_gemm_bf16_ex.restype = ci
    L.ptb_slot_sum.argtypes = [vp, ci, ll, vp, vp, vp]
    L.ptb_slot_sum.restype = ci


class Staging(C.Structure):
    """Request to stage a row-sharded operand from the peers inside the GEMM launch (mirrors ``PtbStaging``)."""
    _fields_ = [("peer", C.c_void_p * 8), ("local", C.c_void_p), ("flags", C.c_void_p), ("rank", C.c_int), ("world", C.c_int),
                ("shard_rows", C.c_int), ("stored_rows", C.c_int), ("row_bytes", C.c_longlong), ("seq", C.c_uint), ("external", C.c_int)]


def make_staging(buf, flags: torch.Tensor, rank: int, world: int, shard_rows: int, stored_rows: int, row_bytes: int, seq: int,
                 external: bool = False) -> Staging:
    s = Staging()
    for r in range(world):
        s.peer[r] = buf.peer_ptr(r)
    s.local, s.flags = buf.peer_ptr(rank), flags.data_ptr()
    s.rank, s.world, s.shard_rows, s.stored_rows, s.row_bytes, s.seq = rank, world, shard_rows, stored_rows, row_bytes, seq
    s.external = int(external)
    return s


_COPY_STREAMS: Dict[int, "torch.cuda.Stream"] = {}


def copy_stream(device) -> "torch.cuda.Stream":
    """The side stream the peer copies run on (one per device)."""
    idx = torch.device(device).index
    if idx not in _COPY_STREAMS:
        _COPY_STREAMS[idx] = torch.cuda.Stream(device=device)
    return _COPY_STREAMS[idx]


def peer_shard_views(buf, elem_cols: int, rank: int, world: int, shard_rows: int):
    """(local full-size [shard_rows*world, cols] view, {peer: view of that peer's own shard in its buffer})."""
    n = shard_rows
    local = buf.tensor(torch.bfloat16)[:n * world * elem_cols].view(n * world, elem_cols)
    peers = {}
    for p in range(world):
        if p != rank:
            peers[p] = buf.tensor(torch.bfloat16, rank=p)[:n * world * elem_cols].view(n * world, elem_cols)[p * n:(p + 1) * n]
    return local, peers


def stage_with_copy_engines(local: torch.Tensor, peers, flags: torch.Tensor, rank: int, world: int, shard_rows: int, seq: int,
                            device):
    """Bring every peer's shard of a row-sharded bf16 matrix into the local full-size buffer with device-to-device
    copies on the side stream (copy engines, no SM), raising the 128-row block flags of each shard as it lands.
    A GEMM launched with an ``external`` staging request of the same ``seq`` waits on those flags tile by tile, so the
    copies overlap its math and it keeps the whole grid for tiles.  The side stream first waits for what the
    current stream has queued (the barrier that says every rank's rows are in place)."""
    side = copy_stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    n = shard_rows
    with torch.cuda.stream(side):
        for d in range(1, world):
            p = (rank + d) % world
            local[p * n:(p + 1) * n].copy_(peers[p], non_blocking=True)
            flags[p * n // 128:((p + 1) * n + 127) // 128].fill_(seq)
    return side


def gemm_ex(a_ptrs, a_shard_rows, lda, a_mn, b_ptrs, b_shard_rows, ldb, b_mn, M, Nn, K, device, out=None, c_peers=None,
            out_shard_rows=0, ldc=None, out_dtype=torch.bfloat16, accumulate=False, stage_a=None, stage_b=None, scatter_slot=None):
    """Raw access to the sharded-operand GEMM.  ``a_ptrs`` / ``b_ptrs``: lists of device addresses.
    ``c_peers``: the output is scattered to its owners, added with fp32 atomics, or (``scatter_slot`` = this rank)
    stored as bf16 into slot ``scatter_slot`` of the owner's ``[world][out_shard_rows][ldc]`` buffer."""
    flags = 0
    if c_peers is not None:
        flags |= EPI_SCATTER_ADD if scatter_slot is None else (EPI_SCATTER_STORE | (int(scatter_slot) << 8))
        cp, nc, cptr = _ptr_array(c_peers), len(c_peers), 0
    else:
        if out is None:
            out = torch.empty(M, Nn, dtype=out_dtype, device=device)
        if out.dtype == torch.float32:
            flags |= EPI_OUT_F32
        if accumulate:
            flags |= 2
        cp, nc, cptr = _ptr_array([0]), 0, out.data_ptr()
        ldc = out.stride(0)
    st = torch.cuda.current_stream(device).cuda_stream
    N.check(N.lib().ptb_gemm_bf16_ex(_ptr_array(a_ptrs), len(a_ptrs), a_shard_rows, lda, int(a_mn), _ptr_array(b_ptrs), len(b_ptrs),
                                     b_shard_rows, ldb, int(b_mn), cptr, ldc, cp, nc, out_shard_rows, M, Nn, K, 0, flags,
                                     _status(device).data_ptr(), 0, st, C.addressof(stage_a) if stage_a is not None else None,
                                     C.addressof(stage_b) if stage_b is not None else None), "gemm_bf16_ex")
    return out


class _Site:
    """Symmetric staging for one layer call site: a bf16 activation buffer peers read, an fp32
    accumulation buffer peers add into, and the flag channel for the barriers."""

    def __init__(self, symm, rows: int, cols_act: int, cols_acc: int):
        self.symm = symm
        self.rows = rows
        W = symm.world
        # full-size activation buffer [rows*W, cols]: this rank's tokens are rows [rank*rows, ...), the peers'
        # rows are staged in by the GEMM that consumes them
        self.act = PeerChannel(symm, rows * W * cols_act * 2) if cols_act else None
        self.acc = PeerChannel(symm, max(rows * cols_acc * 4, rows * W * cols_acc * 2)) if cols_acc else None
        self.chan = self.act or self.acc
        self.cols_act = cols_act
        self.stage_flags = torch.zeros((rows * W + 127) // 128, dtype=torch.int32, device=symm.device)
        self.stage_seq = 0
        self._views = None

    def publish(self, x: torch.Tensor):
        """Put this rank's rows in place, wait until every rank has done so, and return (full view, staging)."""
        W, r, n = self.symm.world, self.symm.rank, self.rows
        if self._views is None:
            self._views = peer_shard_views(self.act.buf, self.cols_act, r, W, n)
        full, peers = self._views
        full[r * n:(r + 1) * n].copy_(x)
        self.barrier()
        self.stage_seq += 1
        ext = _external_staging()
        if ext:
            stage_with_copy_engines(full, peers, self.stage_flags, r, W, n, self.stage_seq, self.symm.device)
        st = make_staging(self.act.buf, self.stage_flags, r, W, n, n * W, self.cols_act * 2, self.stage_seq, external=ext)
        return full, st

    def barrier(self):
        ch = self.chan
        st = torch.cuda.current_stream(self.symm.device).cuda_stream
        N.check(N.lib().ptb_peer_barrier(ch.flag_ptrs, self.symm.rank, self.symm.world, ch.next_seq(), ch.ticket.data_ptr(),
                                         ch.status.data_ptr(), st), "peer_barrier")


def _external_staging() -> bool:
    """Peer rows are staged by copy engines on a side stream (default) or, with PTB_STAGE_IN_KERNEL=1, by stager CTAs
    of the consuming GEMM launch."""
    import os
    return os.environ.get("PTB_STAGE_IN_KERNEL", "0") != "1"


_SITES: Dict[Tuple, _Site] = {}


def _site(tp, key, rows, cols_act, cols_acc) -> _Site:
    k = (id(tp.symm), key, rows, cols_act, cols_acc)
    if k not in _SITES:
        _SITES[k] = _Site(tp.symm, rows, cols_act, cols_acc)
    return _SITES[k]


def _fused_ok(x, tp):
    return tp.symm is not None and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] % 128 == 0


class _ColumnSP(torch.autograd.Function):
    """y[tokens_full, out/W] = gather_tokens(x) @ Wc^T (+ b)."""

    @staticmethod
    def forward(ctx, x, w, bias, tp, key):
        n, K = x.shape
        W = tp.world_size
        site = _site(tp, ("col", key), n, K, K)
        full, st = site.publish(x)                       # every rank's tokens are in place; peers' rows get staged by the GEMM
        y = gemm_ex([full.data_ptr()], 0, K, False, [w.data_ptr()], 0, w.stride(0), False, n * W, w.shape[0], K, x.device, stage_a=st)
        if bias is not None:
            y = y + bias
        # the site's buffer is overwritten by the next call at this site (another micro-batch of a pipeline, a
        # recomputation): the gathered activations that dW needs are kept in a tensor of their own
        ctx.save_for_backward(w, full.clone())
        ctx.site, ctx.tp, ctx.n, ctx.has_bias = site, tp, n, bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        w, full = ctx.saved_tensors
        site, tp, n = ctx.site, ctx.tp, ctx.n
        W, K, dev = tp.world_size, w.shape[1], dy.device
        dy = dy.contiguous()
        # dW[out/W, in] = dY^T gather(X): X was gathered into the local buffer by the forward GEMM, read MN-major
        dw = gemm_ex([dy.data_ptr()], 0, dy.stride(0), True, [full.data_ptr()], 0, K, True, w.shape[0], K, n * W, dev)
        # dX = reduce_scatter_tokens(dY Wc): the epilogue stores each bf16 tile into this rank's slot of the owner's
        # buffer over NVLink; the owner then sums the slots (no atomics, nothing to zero)
        parts = site.acc.buf.tensor(torch.bfloat16)[:W * n * K].view(W, n, K)
        site.barrier()                                   # the owners are done reading the previous contents
        c_peers = [site.acc.buf.peer_ptr(r) for r in range(W)]
        gemm_ex([dy.data_ptr()], 0, dy.stride(0), False, [w.data_ptr()], 0, w.stride(0), True, n * W, K, w.shape[0], dev,
                c_peers=c_peers, out_shard_rows=n, ldc=K, scatter_slot=tp.rank)
        site.barrier()                                   # every peer's contribution has landed
        db = dy.float().sum(0).to(dy.dtype) if ctx.has_bias else None
        return parts.sum(0, dtype=torch.float32).to(torch.bfloat16), dw, db, None, None


class _RowSP(torch.autograd.Function):
    """y[tokens_local, out] = reduce_scatter_tokens(z @ Wr^T)."""

    @staticmethod
    def forward(ctx, z, w, tp, key, resid=None):
        nfull, Kl = z.shape
        W = tp.world_size
        n, out = nfull // W, w.shape[0]
        site = _site(tp, ("row", key), n, out, out)
        parts = site.acc.buf.tensor(torch.bfloat16)[:W * n * out].view(W, n, out)
        site.barrier()                                   # the owners are done reading the previous contents
        c_peers = [site.acc.buf.peer_ptr(r) for r in range(W)]
        z = z.contiguous()
        gemm_ex([z.data_ptr()], 0, z.stride(0), False, [w.data_ptr()], 0, w.stride(0), False, nfull, out, Kl, z.device,
                c_peers=c_peers, out_shard_rows=n, ldc=out, scatter_slot=tp.rank)
        site.barrier()                                   # every rank's partial tiles have landed
        ctx.save_for_backward(z, w)
        ctx.site, ctx.tp, ctx.n = site, tp, n
        ctx.has_resid = resid is not None
        # the owner's sum over the ranks' slots (fp32 accumulation, one pass, the residual folded in when given)
        y = torch.empty(n, out, dtype=torch.bfloat16, device=z.device)
        if resid is not None:
            resid = resid.reshape(n, out).contiguous()
        N.check(N.lib().ptb_slot_sum(parts.data_ptr(), W, n * out, N.ptr(resid), y.data_ptr(),
                                     torch.cuda.current_stream(z.device).cuda_stream), "slot_sum")
        return y

    @staticmethod
    def backward(ctx, dy):
        z, w = ctx.saved_tensors
        site, tp, n = ctx.site, ctx.tp, ctx.n
        W, out, dev = tp.world_size, w.shape[0], dy.device
        full, st = site.publish(dy)
        # dZ[tokens_full, in/W] = gather(dY) Wr : A staged from the peers by this launch, B = Wr read MN-major
        dz = gemm_ex([full.data_ptr()], 0, out, False, [w.data_ptr()], 0, w.stride(0), True, n * W, w.shape[1], out, dev, stage_a=st)
        # dWr[out, in/W] = gather(dY)^T Z : A = gathered dY (now local) read MN-major, B = Z MN-major
        dw = gemm_ex([full.data_ptr()], 0, out, True, [z.data_ptr()], 0, z.stride(0), True, out, w.shape[1], n * W, dev)
        site.barrier()                                   # peers are done reading my dY before it is reused
        return dz, dw, None, None, (dy if ctx.has_resid else None)


_counter = [0]


def column_sp_forward(x, w, bias, tp, key=None):
    if _fused_ok(x, tp):
        return _ColumnSP.apply(x, w, bias, tp, key if key is not None else id(w))
    from .tensor_parallel import _GatherTokens
    return fused_linear(_GatherTokens.apply(x, tp), w, bias)


def row_sp_forward(z, w, tp, key=None, resid=None):
    """``resid`` (optional, ``[tokens_local, out]`` bf16): returned value is ``resid + reduce_scatter(z @ w^T)``, the
    addition done by the kernel that sums the ranks' partial tiles."""
    if _fused_ok(z, tp) and (z.shape[0] // tp.world_size) % 128 == 0 and (z.shape[0] // tp.world_size * w.shape[0]) % 8 == 0:
        return _RowSP.apply(z, w, tp, key if key is not None else id(w), resid)
    from .tensor_parallel import _ScatterTokens
    y = _ScatterTokens.apply(fused_linear(z, w, None), tp)
    return y if resid is None else y + resid
