"""ZeRO-3 / FSDP with the collectives fused into the compute kernels.

Every ``nn.Linear`` weight ``W[out, in]`` is sharded by rows over the ranks (shard height rounded up to
128 rows so GEMM tiles never straddle shards).  Each rank keeps, per weight:

* a full-size bf16 weight buffer in symmetric memory: this rank's shard is its own rows of it (what the peers read),
  the other rows are a staged copy of the peers' shards, refreshed after every optimizer step;
* the fp32 master shard and AdamW moments (sharded: 1/world of the model per rank);
* a full-size bf16 gradient buffer in symmetric memory.

Forward  ``y = x W^T``: one tcgen05 GEMM over the full-size buffer.  The peers' rows arrive block by block
(128 rows) while the GEMM runs: copy engines on a side stream (the default) or stager CTAs of the same launch
(``PTB_STAGE_IN_KERNEL=1``) copy them exactly once and raise a per-block flag; the GEMM's TMA producer waits for the
flags of the rows it is about to read, so the all-gather overlaps the math tile by tile.  The price is the full-size
bf16 copy per weight on every rank (masters and moments stay sharded).
Backward ``dX = dY W``: the same, with ``W`` read as an N-major operand sharded along K.
``dW = dY^T X`` accumulates into the local full-size gradient buffer.
Step: one kernel per weight reads slice *r* of every peer's gradient buffer, sums in fp32 and applies
AdamW to the master shard, writing the new bf16 shard in the same pass (reduce-scatter fused with the
sharded optimizer).  Small replicated parameters (norm weights, embeddings) ride in one bucket that is
all-reduced by the DDP kernel and stepped by the fused multi-tensor AdamW.

``FusedFSDP(window=K)`` trades the per-layer full-size copies for a window of K gathered weights and a few gradient
slots shared by all layers (:class:`WindowPool`): ZeRO-3 memory, two gathers per step.

Compare the reference: all parameters gathered before forward, never resharded, reduce-scatter by
reading every rank's full gradient file (torch/distributed/fsdp.h:227-322).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from .. import _native as N
from ..distributed.ddp import PeerChannel
from ..nn.parallel.fused_tp import Staging, _external_staging, gemm_ex, make_staging, peer_shard_views, stage_with_copy_engines
from ..optim import AdamW


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, holder):
        sh = holder
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) != x2.shape[1]:
            x2 = x2.contiguous()
        # B = the local full-size buffer; rows owned by peers cross NVLink once per optimizer step: copy engines
        # start bringing them in as soon as the owner's optimizer kernel is done (or stager CTAs of this launch
        # do), and the tile producers of this launch wait on the 128-row block flags, so transfer and math overlap
        wptr, stg = sh.weight_operand(forward=True)
        y = gemm_ex([x2.data_ptr()], 0, x2.stride(0), False, [wptr], 0, sh.inf, False, x2.shape[0], sh.out, sh.inf, x.device,
                    stage_b=stg)
        sh.weight_used()
        ctx.save_for_backward(x2)
        ctx.sh, ctx.xshape = sh, x.shape
        return y.view(*x.shape[:-1], sh.out)

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        sh = ctx.sh
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        dev = dy.device
        # dX[M, in] = dY[M, out] W[out, in]: W stored [K=out (row-sharded over ranks), N=in], read N-major
        wptr, stg = sh.weight_operand(forward=False)
        dx = gemm_ex([dy2.data_ptr()], 0, dy2.stride(0), False, [wptr], 0, sh.inf, True, dy2.shape[0], sh.inf, sh.out, dev,
                     stage_b=stg)
        sh.weight_used()
        # dW[out, in] (+)= dY^T X into the local full-size gradient buffer, or into a slot of the gradient window, whose
        # reduce-scatter into this rank's fp32 gradient shard starts right behind it on the reduce stream
        target, accumulate = sh.grad_target()
        gemm_ex([dy2.data_ptr()], 0, dy2.stride(0), True, [x2.data_ptr()], 0, x2.stride(0), True, sh.out, sh.inf, dy2.shape[0], dev,
                out=target[:sh.out], accumulate=accumulate)
        sh.grad_written()
        return dx.view(ctx.xshape), None


class WindowPool:
    """Staging shared by all sharded layers of a ``FusedFSDP(window=K)``: ZeRO-3 memory.

    * ``K`` weight slots (plain device memory, each as large as the largest gathered weight).  A layer's weight is
      gathered into a slot right before the GEMM that reads it (own rows by a local copy, the peers' rows by the copy
      engines on the side stream, 128-row block flags raised as they land, the GEMM's producer waiting on those
      flags), the next layer's gather is queued before this layer's GEMM is launched, and a slot is taken over by
      another layer once the GEMMs that read it are done.  Backward gathers again.
    * ``G`` gradient slots (symmetric memory, same size).  A layer's dW goes into a slot, and a reduce-scatter kernel
      on the reduce stream adds slice *r* of every rank's slot into rank *r*'s fp32 gradient shard; the slot is free
      again when that kernel is over (its closing barrier says every rank has read).

    Per rank this leaves the bf16 shard, the fp32 master / moments / gradient shard (all 1/world of the model) and
    ``K + G`` layer-sized buffers, instead of a full-size bf16 weight and gradient copy of every layer."""

    def __init__(self, symm, n_weight: int, n_grad: int, status: torch.Tensor):
        self.symm, self.n_weight, self.n_grad, self.status = symm, max(int(n_weight), 1), max(int(n_grad), 1), status
        self.layers: List["ShardedLinear"] = []
        self.wslots: List[dict] = []
        self.gslots: List[PeerChannel] = []
        self.g_events: List[Optional[torch.cuda.Event]] = []
        self._w_next = self._g_next = 0
        self.reduce_stream = None
        self.gathers = 0                      # how many times a weight was brought in (tests, metrics)

    def register(self, sl: "ShardedLinear"):
        sl.index = len(self.layers)
        self.layers.append(sl)

    def allocate(self):
        """Called once every layer is registered: the slots take the size of the largest layer."""
        dev, W = self.symm.device, self.symm.world
        self.max_numel = max(sl.S * W * sl.inf for sl in self.layers)
        max_rows = max(sl.S * W for sl in self.layers)
        for _ in range(self.n_weight):
            self.wslots.append(dict(buf=torch.empty(self.max_numel, dtype=torch.bfloat16, device=dev),
                                    flags=torch.zeros((max_rows + 127) // 128, dtype=torch.int32, device=dev), seq=0, owner=None,
                                    owner_seq=-1, event=None))
        for _ in range(self.n_grad):
            self.gslots.append(PeerChannel(self.symm, self.max_numel * 2, status=self.status))
            self.g_events.append(None)
        self.reduce_stream = torch.cuda.Stream(device=dev)
        self.symm.barrier()

    @property
    def window_bytes(self) -> int:
        return (self.n_weight + self.n_grad) * self.max_numel * 2

    # ---- weights
    def _resident(self, sl):
        for s in self.wslots:
            if s["owner"] is sl and s["owner_seq"] == sl.stage_seq:
                return s
        return None

    def _gather(self, sl) -> dict:
        dev, W, r, n = self.symm.device, self.symm.world, self.symm.rank, sl.S
        s = self.wslots[self._w_next]
        self._w_next = (self._w_next + 1) % len(self.wslots)
        cur = torch.cuda.current_stream(dev)
        if s["event"] is not None:
            cur.wait_event(s["event"])        # the GEMMs that read the slot's previous tenant
        s["seq"] += 1
        s["owner"], s["owner_seq"] = sl, sl.stage_seq
        view = s["buf"][:n * W * sl.inf].view(n * W, sl.inf)
        view[r * n:(r + 1) * n].copy_(sl.shard)      # own rows: the GEMM does not look at flags for them
        if W > 1:
            stage_with_copy_engines(view, sl.peer_views, s["flags"], r, W, n, s["seq"], dev)
        s["view"] = view
        self.gathers += 1
        return s

    def weight(self, sl, forward: bool) -> dict:
        s = self._resident(sl) or self._gather(sl)
        # queue the neighbour's gather before this layer's GEMM goes onto the compute stream
        j = sl.index + (1 if forward else -1)
        if len(self.wslots) > 1 and 0 <= j < len(self.layers) and self._resident(self.layers[j]) is None:
            nxt = self.wslots[self._w_next]
            if nxt is not s:
                self._gather(self.layers[j])
        return s

    def used(self, s: dict):
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.symm.device))
        s["event"] = ev

    # ---- gradients
    def grad_slot(self, sl):
        i = self._g_next
        self._g_next = (i + 1) % len(self.gslots)
        if self.g_events[i] is not None:
            torch.cuda.current_stream(self.symm.device).wait_event(self.g_events[i])
        ch = self.gslots[i]
        W = self.symm.world
        view = ch.buf.tensor(torch.bfloat16)[:sl.S * W * sl.inf].view(sl.S * W, sl.inf)
        if sl.out < sl.S * W:
            view[sl.out:].zero_()             # padding rows take part in the sum
        return i, view

    def reduce(self, sl, i: int, n_ctas: int = 64):
        dev = self.symm.device
        ch = self.gslots[i]
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
        rs = self.reduce_stream
        rs.wait_event(ev)
        N.check(N.lib().ptb_fsdp_rs_accum(ch.bufs, ch.flag_ptrs, self.symm.rank, self.symm.world, sl.S * self.symm.world * sl.inf,
                                          sl.gacc.data_ptr(), 1.0, ch.next_seq(), ch.ticket.data_ptr(), ch.status.data_ptr(), n_ctas,
                                          rs.cuda_stream), "fsdp_rs_accum")
        done = torch.cuda.Event()
        done.record(rs)
        self.g_events[i] = done


class ShardedLinear(nn.Module):
    """Drop-in for a bias-free ``nn.Linear`` whose weight lives row-sharded across the ranks."""

    def __init__(self, lin: nn.Linear, symm, pg, status: Optional[torch.Tensor] = None, pool: Optional[WindowPool] = None):
        super().__init__()
        self.pool = pool
        if lin.bias is not None:
            raise NotImplementedError("ShardedLinear: bias-free layers only")
        W, r = symm.world, symm.rank
        self.out, self.inf = lin.out_features, lin.in_features
        self.S = (math.ceil(self.out / W) + 127) // 128 * 128
        dev = symm.device
        full = lin.weight.detach().to(dev, torch.float32)
        pg.broadcast(full, 0)
        padded = torch.zeros(self.S * W, self.inf, device=dev)
        padded[:self.out] = full
        self.master = padded[r * self.S:(r + 1) * self.S].clone().contiguous()
        self.m, self.v = torch.zeros_like(self.master), torch.zeros_like(self.master)
        self.symm = symm
        self.stage_seq = 1
        self.step_count = 0
        if pool is not None:
            # window mode: only this rank's shard lives here (in symmetric memory, the peers gather from it) plus the fp32
            # gradient shard the reduce-scatter kernels add into
            self.shard_ch = PeerChannel(symm, self.S * self.inf * 2)
            self.shard = self.shard_ch.buf.tensor(torch.bfloat16)[:self.S * self.inf].view(self.S, self.inf)
            self.shard.copy_(self.master)
            self.peer_views = {q: self.shard_ch.buf.tensor(torch.bfloat16, rank=q)[:self.S * self.inf].view(self.S, self.inf)
                               for q in range(W) if q != r}
            self.gacc = torch.zeros_like(self.master)
            self._slot = self._gslot = None
            pool.register(self)
            symm.barrier()
            return
        # full-size symmetric buffer; this rank's shard is rows [r*S, (r+1)*S) of it (what peers read)
        self.shard_ch = PeerChannel(symm, self.S * W * self.inf * 2)
        self.w_full = self.shard_ch.buf.tensor(torch.bfloat16)[:self.S * W * self.inf].view(self.S * W, self.inf)
        self.w_full.zero_()
        self.shard = self.w_full[r * self.S:(r + 1) * self.S]
        self.shard.copy_(self.master)
        self.full_ptr = self.shard_ch.buf.peer_ptr(r)
        self.stage_flags = torch.zeros((self.S * W + 127) // 128, dtype=torch.int32, device=dev)
        self.grad_ch = PeerChannel(symm, self.S * W * self.inf * 2, status=status)
        self.grad_full = self.grad_ch.buf.tensor(torch.bfloat16)[:self.S * W * self.inf].view(self.S * W, self.inf)
        self.grad_full.zero_()
        self._staged_seq = 0
        self._views = None
        symm.barrier()
        self.prefetch()

    def prefetch(self):
        """Start copying the peers' current shards into the local full-size buffer on the copy stream (the owners'
        shards are final: the optimizer kernel ends with a barrier across the ranks).  The block flags rise as
        the shards land; the first GEMM that reads the weight checks them."""
        if self.pool is not None or not _external_staging() or self.symm.world == 1:
            return
        if self._views is None:
            self._views = peer_shard_views(self.shard_ch.buf, self.inf, self.symm.rank, self.symm.world, self.S)
        stage_with_copy_engines(self._views[0], self._views[1], self.stage_flags, self.symm.rank, self.symm.world, self.S,
                                self.stage_seq, self.symm.device)

    def staging(self):
        """Staging request for the first GEMM that touches the weight after an optimizer step; ``None`` afterwards:
        by the end of that launch every peer block is local (it waited for, or copied, the whole matrix), so later
        launches on the same stream read the local copy without looking at the flags."""
        if self._staged_seq == self.stage_seq:
            return None
        self._staged_seq = self.stage_seq
        return make_staging(self.shard_ch.buf, self.stage_flags, self.symm.rank, self.symm.world, self.S,
                            self.S * self.symm.world, self.inf * 2, self.stage_seq, external=_external_staging())

    # ---- what the GEMMs of the autograd function read and write
    def weight_operand(self, forward: bool):
        """(address of the gathered ``[S * world, in]`` bf16 weight, staging request or None)."""
        if self.pool is None:
            return self.full_ptr, self.staging()
        s = self._slot = self.pool.weight(self, forward)
        W = self.symm.world
        if W == 1:
            return s["view"].data_ptr(), None
        stg = Staging()
        for q in range(W):
            stg.peer[q] = s["view"].data_ptr()        # unused: the copy engines bring the rows in (external staging)
        stg.local, stg.flags = s["view"].data_ptr(), s["flags"].data_ptr()
        stg.rank, stg.world, stg.shard_rows, stg.stored_rows = self.symm.rank, W, self.S, self.S * W
        stg.row_bytes, stg.seq, stg.external = self.inf * 2, s["seq"], 1
        return s["view"].data_ptr(), stg

    def weight_used(self):
        if self.pool is not None:
            self.pool.used(self._slot)

    def grad_target(self):
        """(``[S * world, in]`` bf16 buffer the dW GEMM writes, whether it accumulates)."""
        if self.pool is None:
            return self.grad_full, True
        self._gslot, view = self.pool.grad_slot(self)
        return view, False

    def grad_written(self):
        if self.pool is not None:
            self.pool.reduce(self, self._gslot)

    def forward(self, x):
        return _ShardedLinearFn.apply(x, self)

    @torch.no_grad()
    def step(self, lr, betas, eps, wd, grad_scale=1.0, n_ctas=64):
        """Reduce-scatter the gradient and apply AdamW to the local shard (one kernel)."""
        self.step_count += 1
        ch = self.grad_ch
        st = torch.cuda.current_stream(self.symm.device).cuda_stream
        N.check(N.lib().ptb_fsdp_rs_adamw(ch.bufs, ch.flag_ptrs, self.symm.rank, self.symm.world, self.grad_full.numel(),
                                          self.master.data_ptr(), self.m.data_ptr(), self.v.data_ptr(), self.shard.data_ptr(), lr,
                                          betas[0], betas[1], eps, wd, self.step_count, grad_scale, ch.next_seq(),
                                          ch.ticket.data_ptr(), ch.status.data_ptr(), n_ctas, st), "fsdp_rs_adamw")
        self.grad_full.zero_()
        self.stage_seq += 1             # the peers' rows of w_full are stale now
        self.prefetch()

    def full_weight(self) -> torch.Tensor:
        """Gather the bf16 weight (checkpointing / tests)."""
        if self.pool is not None:
            parts = [self.shard.clone() if k == self.symm.rank else self.peer_views[k].clone() for k in range(self.symm.world)]
            return torch.cat(parts)[:self.out]
        parts = [self.shard_ch.buf.tensor(torch.bfloat16, rank=k)[:self.S * self.symm.world * self.inf]
                 .view(self.S * self.symm.world, self.inf)[k * self.S:(k + 1) * self.S].clone() for k in range(self.symm.world)]
        return torch.cat(parts)[:self.out]


class FusedFSDP(nn.Module):
    """Wraps a model: linear layers become :class:`ShardedLinear`; everything else is replicated and
    kept in sync by the fused bucket all-reduce.  ``step()`` runs the sharded AdamW kernels and the
    replicated-parameter AdamW; hyper-parameters follow an optional LR scheduler through ``param_groups``."""

    def __init__(self, model: nn.Module, symm, pg, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 min_shard_numel: int = 1 << 16, check_every: int = 1, window: int = 0, grad_window: int = 2):
        """``check_every``: every that many ``step()`` calls the host reads the one status word all the fused kernels of
        this wrapper share and raises ``CollectiveTimeout`` if one of them gave up waiting for a peer (a kernel that
        gives up applies no update).  0 leaves the check to ``check()``.

        ``window`` = K > 0 selects ZeRO-3 memory (:class:`WindowPool`): gathered weights live in K slots shared by all
        layers and are re-gathered in backward (the reference's ``reshard_params`` / ``drop_full_param``,
        torch/distributed/fsdp.h:200-213,255-262), gradients pass through ``grad_window`` slots and are reduce-scattered
        layer by layer during backward.  ``window`` = 0 keeps a gathered bf16 copy and a full gradient buffer per layer
        (ZeRO-3 traffic with ZeRO-2 memory; one gather per step instead of two)."""
        super().__init__()
        self.symm, self.pg = symm, pg
        self.check_every, self._steps = int(check_every), 0
        self.status = torch.zeros(1, dtype=torch.int32, device=symm.device)
        self.sharded: List[ShardedLinear] = []
        self.pool = WindowPool(symm, window, grad_window, self.status) if window > 0 else None
        self._replace(model, min_shard_numel)
        if self.pool is not None and self.sharded:
            self.pool.allocate()
            self.bar_ch = PeerChannel(symm, 256, status=self.status)
            self._win_table = None
            self._win_scale = torch.ones(1, device=symm.device)
        self.model = model
        self.param_groups = [dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, params=[])]
        rest = [p for p in model.parameters() if p.requires_grad]
        self.rest = rest
        with torch.no_grad():
            for p in rest:
                pg.broadcast(p.data, 0)
        # fp32 masters for the replicated bf16 parameters; their gradients share one symmetric bucket
        self.rest_master = [p.detach().float().clone().requires_grad_(False) for p in rest]
        n = sum(p.numel() for p in rest)
        self.bucket_numel = (n + 63) // 64 * 64
        self.rest_opt = None
        if rest:
            self.bucket = PeerChannel(symm, self.bucket_numel * 2, status=self.status)
            flat = self.bucket.buf.tensor(torch.bfloat16)[:self.bucket_numel]
            flat.zero_()
            self.rest_grads, off = [], 0
            for p in rest:
                self.rest_grads.append(flat[off:off + p.numel()].view_as(p))
                off += p.numel()
            masters = [nn.Parameter(m, requires_grad=False) for m in self.rest_master]
            self.rest_master_params = masters
            self.rest_opt = AdamW(masters, lr=lr, betas=betas, eps=eps, weight_decay=0.0, fused=True)
            for mp, g, p in zip(masters, self.rest_grads, rest):
                self.rest_opt.set_grad_source(mp, g)
                if p.dtype == torch.bfloat16:
                    self.rest_opt.attach_lowp(mp, p.data)
            self._copy_back = [(mp, p) for mp, p in zip(masters, rest) if p.dtype != torch.bfloat16]
            self.flat = flat

    def _replace(self, mod: nn.Module, min_numel: int):
        for name, child in list(mod.named_children()):
            if isinstance(child, nn.Linear) and child.bias is None and child.weight.numel() >= min_numel \
                    and child.in_features % 64 == 0:
                sl = ShardedLinear(child, self.symm, self.pg, self.status, self.pool)
                setattr(mod, name, sl)
                self.sharded.append(sl)
            else:
                self._replace(child, min_numel)

    def forward(self, *a, **kw):
        return self.model(*a, **kw)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        g = self.param_groups[0]
        if self.pool is not None and self.sharded:
            self._window_step(g, grad_scale)
        else:
            for sl in self.sharded:
                sl.step(g["lr"], g["betas"], g["eps"], g["weight_decay"], grad_scale / self.symm.world)
        if self.rest_opt is not None:
            # fold .grad of the replicated parameters into the symmetric bucket, all-reduce it in one kernel
            for p, gv in zip(self.rest, self.rest_grads):
                if p.grad is not None:
                    gv.copy_(p.grad)
                    p.grad = None
            ch = self.bucket
            st = torch.cuda.current_stream(self.symm.device).cuda_stream
            N.check(N.lib().ptb_ddp_allreduce(ch.bufs, ch.flag_ptrs, self.symm.rank, self.symm.world, self.bucket_numel, 1,
                                              grad_scale / self.symm.world, ch.next_seq(), ch.ticket.data_ptr(), ch.status.data_ptr(),
                                              32, st), "ddp_allreduce")
            self.rest_opt.param_groups[0]["lr"] = g["lr"]
            self.rest_opt.step()
            for mp, p in self._copy_back:
                p.data.copy_(mp.data)
            self.flat.zero_()
        self._steps += 1
        if self.check_every > 0 and self._steps % self.check_every == 0 and self.sharded:
            ch = self.pool.gslots[0] if self.pool is not None else self.sharded[0].grad_ch
            ch.raise_if_failed(ch.stage_status())

    @torch.no_grad()
    def _window_step(self, g, grad_scale: float):
        """Window mode: the reduce-scatters have run during backward; one fused multi-tensor AdamW steps every fp32
        master shard from its fp32 gradient shard and writes the bf16 shards, then a barrier across the ranks keeps
        anyone from gathering a shard its owner has not written yet."""
        import ctypes as C
        from ..optim.optimizers import OPT_ADAMW, TensorTable
        dev = self.symm.device
        cur = torch.cuda.current_stream(dev)
        cur.wait_stream(self.pool.reduce_stream)
        if self._win_table is None:
            self._win_table = TensorTable()
        ps = [sl.master for sl in self.sharded]
        self._win_table.build(ps, [sl.gacc for sl in self.sharded], [(sl.m, sl.v, None) for sl in self.sharded],
                              [sl.shard for sl in self.sharded], dev)
        for sl in self.sharded:
            sl.step_count += 1
        t = self.sharded[0].step_count
        b1, b2 = g["betas"]
        self._win_scale.fill_(grad_scale / self.symm.world)
        h = [g["lr"], b1, b2, g["eps"], g["weight_decay"], 1 - b1 ** t, 1 - b2 ** t, 0.0]
        harr = (C.c_float * 16)(*(h + [0.0] * (16 - len(h))))
        tab = self._win_table
        N.check(N.lib().ptb_multi_tensor_opt(tab.rows.data_ptr(), tab.chunks.data_ptr(), tab.n_chunks, OPT_ADAMW, 0, harr,
                                             self._win_scale.data_ptr(), None, cur.cuda_stream), "multi_tensor_opt")
        for sl in self.sharded:
            sl.gacc.zero_()
            sl.stage_seq += 1                 # what the window slots hold of this layer is stale now
        ch = self.bar_ch
        N.check(N.lib().ptb_peer_barrier(ch.flag_ptrs, self.symm.rank, self.symm.world, ch.next_seq(), ch.ticket.data_ptr(),
                                         ch.status.data_ptr(), cur.cuda_stream), "peer_barrier")

    def memory_report(self) -> Dict[str, int]:
        """Bytes this rank holds for the sharded layers: what scales with 1/world, and the fixed window (or, without a
        window, the full-size copies)."""
        shard = sum(sl.master.numel() * (4 * 3 + 2) for sl in self.sharded)            # master, m, v, bf16 shard
        if self.pool is not None:
            shard += sum(sl.gacc.numel() * 4 for sl in self.sharded)
            return {"sharded_state": shard, "window": self.pool.window_bytes, "full_copies": 0}
        full = sum(sl.w_full.numel() * 2 + sl.grad_full.numel() * 2 for sl in self.sharded)
        return {"sharded_state": shard - sum(sl.master.numel() * 2 for sl in self.sharded), "window": 0, "full_copies": full}

    def zero_grad(self):
        for p in self.rest:
            p.grad = None

    # ------------------------------------------------------------------ sharded checkpoints
    def save_sharded(self, directory: str, extra: Optional[dict] = None):
        """One ``.safetensors`` file per rank (fp32 master shard and AdamW moments of every sharded weight) plus, from rank 0,
        the replicated parameters with their optimizer state and ``manifest.json``.  Every rank calls this."""
        import json
        import os
        from ..distributed.checkpoint import _opt_state_tensors, _rank_file
        from ..io.safetensors import save_file
        os.makedirs(directory, exist_ok=True)
        r, W = self.symm.rank, self.symm.world
        torch.cuda.synchronize(self.symm.device)
        t: Dict[str, torch.Tensor] = {}
        for i, sl in enumerate(self.sharded):
            t[f"layer.{i}.master"], t[f"layer.{i}.m"], t[f"layer.{i}.v"] = sl.master.cpu(), sl.m.cpu(), sl.v.cpu()
        if r == 0 and self.rest_opt is not None:
            for j, mp in enumerate(self.rest_master_params):
                t[f"rest.{j}.master"] = mp.data.cpu()
            t.update({"rest." + k: v for k, v in _opt_state_tensors(self.rest_opt, self.rest_master_params).items()})
        save_file(t, _rank_file(directory, r) + ".tmp", metadata={"rank": str(r), "world": str(W)})
        os.replace(_rank_file(directory, r) + ".tmp", _rank_file(directory, r))
        if r == 0:
            groups = [{k: v for k, v in g.items() if k != "params" and isinstance(v, (int, float, bool, str, list, tuple))}
                      for g in (self.rest_opt.param_groups if self.rest_opt is not None else [])]
            manifest = {"format": "ptb-fused-fsdp-1", "world_size": W,
                        "layers": [{"out": sl.out, "in": sl.inf, "shard_rows": sl.S, "step_count": sl.step_count} for sl in self.sharded],
                        "rest": [list(p.shape) for p in self.rest], "rest_param_groups": groups,
                        "param_groups": [{k: (list(v) if isinstance(v, tuple) else v) for k, v in g.items() if k != "params"}
                                         for g in self.param_groups], "extra": extra or {}}
            with open(os.path.join(directory, "manifest.json.tmp"), "w") as f:
                json.dump(manifest, f, indent=1)
            os.replace(os.path.join(directory, "manifest.json.tmp"), os.path.join(directory, "manifest.json"))
        self.symm.barrier()

    @torch.no_grad()
    def load_sharded(self, directory: str) -> dict:
        """Restore what :meth:`save_sharded` wrote, also when this run has a different number of ranks (each rank re-cuts
        its rows from the writers' files).  Returns the manifest's ``extra``."""
        import json
        import os
        from ..distributed.checkpoint import _rank_file
        from ..io.safetensors import SafeTensorsFile
        with open(os.path.join(directory, "manifest.json")) as f:
            man = json.load(f)
        if man.get("format") != "ptb-fused-fsdp-1":
            raise ValueError(f"{directory}: not a fused-FSDP checkpoint")
        if len(man["layers"]) != len(self.sharded) or any(m["out"] != sl.out or m["in"] != sl.inf for m, sl in zip(man["layers"], self.sharded)):
            raise ValueError(f"{directory}: the sharded layers of the checkpoint do not match this model")
        r, oldW = self.symm.rank, int(man["world_size"])
        files = [SafeTensorsFile(_rank_file(directory, q)) for q in range(oldW)]
        try:
            for i, (sl, meta) in enumerate(zip(self.sharded, man["layers"])):
                So = int(meta["shard_rows"])
                lo, hi = r * sl.S, (r + 1) * sl.S
                for key, dst in (("master", sl.master), ("m", sl.m), ("v", sl.v)):
                    buf = torch.zeros(sl.S, sl.inf)
                    for q in range(lo // So, min(oldW, (hi - 1) // So + 1)):
                        a, b = max(lo, q * So), min(hi, (q + 1) * So)
                        buf[a - lo:b - lo] = files[q].get_tensor(f"layer.{i}.{key}")[a - q * So:b - q * So]
                    buf[max(0, min(hi, sl.out) - lo):] = 0                     # rows past the weight are padding
                    dst.copy_(buf)
                sl.shard.copy_(sl.master)
                sl.step_count = int(meta["step_count"])
            if self.rest_opt is not None:
                for j, (mp, p) in enumerate(zip(self.rest_master_params, self.rest)):
                    mp.data.copy_(files[0].get_tensor(f"rest.{j}.master"))
                    p.data.copy_(mp.data)
                    st = self.rest_opt.state[mp]
                    for k in [k for k in files[0].keys() if k.startswith(f"rest.opt.{j}.")]:
                        v = files[0].get_tensor(k)
                        name = k[len(f"rest.opt.{j}."):]
                        st[name] = v.to(mp.device).view_as(mp) if v.dim() else (st[name].new_tensor(float(v)) if torch.is_tensor(st.get(name)) else torch.tensor(float(v)))
                for g, saved in zip(self.rest_opt.param_groups, man.get("rest_param_groups", [])):
                    for k, v in saved.items():
                        g[k] = tuple(v) if isinstance(g.get(k), tuple) and isinstance(v, list) else v
        finally:
            for f in files:
                f.close()
        for g, saved in zip(self.param_groups, man.get("param_groups", [])):
            for k, v in saved.items():
                g[k] = tuple(v) if k == "betas" else v
        torch.cuda.synchronize(self.symm.device)
        self.symm.barrier()                                   # every owner's bf16 shard is in place
        for sl in self.sharded:
            sl.stage_seq += 1                                 # the peers' rows held locally are stale
            sl.prefetch()
        return man.get("extra", {})

    def check(self):
        if self.sharded and self.pool is not None:
            self.pool.gslots[0].check()
        elif self.sharded:
            self.sharded[0].grad_ch.check()        # one status word serves every channel of this wrapper
        elif self.rest_opt is not None:
            self.bucket.check()
