"""DistributedDataParallel: bucketed gradient all-reduce overlapped with backward.

The reference's DDP all-reduces parameter by parameter after backward has
finished and scales on the host (torch/distributed/ddp.cpp:1067-1091); its
``no_sync()`` is a flag that turns that call into a no-op (ddp.h:168-186).
This one keeps the same surface — ``no_sync()``, ``require_grad_sync``,
``finish_gradient_synchronization()``, ``sync_gradients()`` / ``allreduce_grads()``
— and changes the mechanics:

* gradients live in flat buckets (≈25 MB, filled in reverse parameter order);
  ``param.grad`` is a view into its bucket, so accumulation under ``no_sync()``
  happens in place and nothing is copied at reduce time;
* a post-accumulate-grad hook on every parameter counts the bucket down; the
  bucket that completes is reduced at once on a communication stream while
  backward keeps running;
* with a symmetric-memory group on CUDA the reduction is ONE kernel per bucket
  that reads every peer's bucket over NVLink, sums in fp32, folds in the 1/world
  scale and writes the result into every peer's bucket (csrc/collectives.cu);
  without one it is the process group's all-reduce (NCCL or Gloo) and a scale.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import List, Optional

import torch
import torch.nn as nn

from .. import _native as N
from .process_group import ProcessGroup, ReduceOp, SingleProcessGroup, TorchProcessGroup


@N.register_decls
def _decls(L):
    vp, ci, cf, ll, cu = C.c_void_p, C.c_int, C.c_float, C.c_longlong, C.c_uint
    pp = C.POINTER(C.c_void_p)
    L.ptb_ddp_allreduce.argtypes = [pp, pp, ci, ci, ll, ci, cf, cu, vp, vp, ci, vp]
    L.ptb_ddp_allreduce.restype = ci
    L.ptb_fsdp_rs_adamw.argtypes = [pp, pp, ci, ci, ll, vp, vp, vp, vp, cf, cf, cf, cf, cf, ci, cf, cu, vp, vp, ci, vp]
    L.ptb_fsdp_rs_adamw.restype = ci
    L.ptb_fsdp_rs_accum.argtypes = [pp, pp, ci, ci, ll, vp, cf, cu, vp, vp, ci, vp]
    L.ptb_fsdp_rs_accum.restype = ci
    L.ptb_allgather.argtypes = [pp, pp, ci, ci, vp, ll, cu, vp, vp, ci, vp]
    L.ptb_allgather.restype = ci
    L.ptb_peer_barrier.argtypes = [pp, ci, ci, cu, vp, vp, vp]
    L.ptb_peer_barrier.restype = ci
    L.ptb_ddp_allreduce_master.argtypes = [pp, pp, pp, ci, ci, ll, cf, cu, vp, vp, ci, vp]
    L.ptb_ddp_allreduce_master.restype = ci
    L.ptb_set_collective_timeout_ms.argtypes = [ci]
    L.ptb_set_collective_timeout_ms.restype = None
    L.ptb_get_collective_timeout_ms.argtypes = []
    L.ptb_get_collective_timeout_ms.restype = ci


def set_collective_timeout(seconds: float):
    """Wall-clock budget of every wait inside the fused collective kernels (default 10 s, or the environment variable
    PTB_COLLECTIVE_TIMEOUT_MS).  A peer that is further behind than this makes the kernel give up: it records a status
    code, leaves the data untouched and the next status check raises ``CollectiveTimeout``."""
    N.lib().ptb_set_collective_timeout_ms(int(seconds * 1000))


def _ptr_array(ptrs):
    return (C.c_void_p * len(ptrs))(*ptrs)


class PeerChannel:
    """A symmetric buffer plus its flag block and launch bookkeeping for the fused collectives."""

    def __init__(self, symm, nbytes: int, status: Optional[torch.Tensor] = None):
        """``status``: share one status word between several channels (one host read then covers all of them)."""
        self.symm = symm
        self.buf = symm.alloc(nbytes)
        self.flags = symm.alloc(2 * 8 * 4)
        self.bufs = _ptr_array([self.buf.peer_ptr(r) for r in range(symm.world)])
        self.flag_ptrs = _ptr_array([self.flags.peer_ptr(r) for r in range(symm.world)])
        self.ticket = torch.zeros(1, dtype=torch.int32, device=symm.device)
        self.status = status if status is not None else torch.zeros(1, dtype=torch.int32, device=symm.device)
        self._host_status = torch.zeros(1, dtype=torch.int32).pin_memory() if symm.device.type == "cuda" else None
        self.seq = 0

    def next_seq(self) -> int:
        self.seq += 1
        return self.seq

    def stage_status(self, stream=None):
        """Queue a copy of the status word to pinned host memory behind the kernels already on ``stream``; returns the
        event that marks its arrival.  ``raise_if_failed(event)`` then costs no more than waiting for that event."""
        st = stream if stream is not None else torch.cuda.current_stream(self.status.device)
        with torch.cuda.stream(st):
            self._host_status.copy_(self.status, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(st)
        return ev

    def raise_if_failed(self, event=None):
        if event is not None:
            event.synchronize()
            s = int(self._host_status[0])
        else:
            s = int(self.status)
        if s:
            self.status.zero_()
            from .process_group import CollectiveTimeout
            raise CollectiveTimeout(f"fused collective: a peer GPU did not arrive within the wait budget (status {s})")

    def check(self):
        self.raise_if_failed()


class _Bucket:
    def __init__(self, params: List[nn.Parameter], dtype, device, symm, fp32_master: bool = False):
        self.params = params
        n = sum(p.numel() for p in params)
        self.numel = (n + 63) // 64 * 64
        self.channel = None
        self.master = None             # fp32 copy of the reduced gradients (bf16 buckets with fp32_master_grads)
        self.master_views = None
        if symm is not None and device.type == "cuda":
            self.channel = PeerChannel(symm, self.numel * torch.empty(0, dtype=dtype).element_size())
            self.flat = self.channel.buf.tensor(dtype)[:self.numel]
            if fp32_master and dtype == torch.bfloat16:
                self.master_buf = symm.alloc(self.numel * 4)
                self.master_ptrs = _ptr_array([self.master_buf.peer_ptr(r) for r in range(symm.world)])
                self.master = self.master_buf.tensor(torch.float32)[:self.numel]
                self.master.zero_()
        else:
            self.flat = torch.zeros(self.numel, dtype=dtype, device=device)
        self.flat.zero_()
        off = 0
        self.views = []
        if self.master is not None:
            self.master_views = []
        for p in params:
            v = self.flat[off:off + p.numel()].view_as(p)
            self.views.append(v)
            if self.master is not None:
                self.master_views.append(self.master[off:off + p.numel()].view_as(p))
            off += p.numel()
        self.pending = len(params)
        self.work = None
        self.event = None
        self.launched = False


class DistributedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, process_group: Optional[ProcessGroup] = None, broadcast_parameters: bool = True,
                 bucket_mb: float = 25.0, symm=None, comm_ctas: int = 32, check_every: int = 1,
                 fp32_master_grads: bool = False, metrics=None):
        """``check_every``: with the fused (symmetric-memory) reduction, every that many calls
        ``finish_gradient_synchronization()`` waits for the reductions and raises ``CollectiveTimeout`` if a kernel
        gave up waiting for a peer, so the optimizer never steps on gradients that were not reduced (0 = only
        ``check()`` looks).  ``fp32_master_grads``: bf16 buckets are reduced into fp32 copies
        (``master_grad(param)``) by the same kernel, for optimizers that keep fp32 master weights.
        ``metrics``: a ``utils.metrics.MetricsWriter``; every bucket reduction is then timed (CUDA events on the
        communication stream, the host clock on CPU) and logged with its bytes on the wire, GB/s and fraction of the
        NVLink roofline when ``finish_gradient_synchronization()`` collects it (this waits for the reductions)."""
        super().__init__()
        self.metrics = metrics
        self.check_every, self._finish_calls = int(check_every), 0
        self.fp32_master_grads = bool(fp32_master_grads)
        self.module = module
        if process_group is None:
            import torch.distributed as dist
            process_group = TorchProcessGroup() if dist.is_available() and dist.is_initialized() else SingleProcessGroup()
        self.process_group = process_group
        self.rank, self.world_size = process_group.rank, process_group.world_size
        self.require_grad_sync = True
        self.symm, self.comm_ctas = symm, comm_ctas
        self._params = [p for p in module.parameters() if p.requires_grad]
        self._comm_stream = None
        if self._params and self._params[0].is_cuda:
            self._comm_stream = torch.cuda.Stream(device=self._params[0].device)
        if broadcast_parameters and self.world_size > 1:
            self._broadcast_state()
        self._build_buckets(bucket_mb)
        self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(p)) for p in self._params]

    # ------------------------------------------------------------------ construction
    def _broadcast_state(self):
        with torch.no_grad():
            for t in list(self.module.parameters()) + list(self.module.buffers()):
                self.process_group.broadcast(t.data, 0)

    def _build_buckets(self, bucket_mb: float):
        self.buckets: List[_Bucket] = []
        self._bucket_of = {}
        self._view_of = {}
        cap = int(bucket_mb * 1024 * 1024)
        groups, cur, cur_bytes, key = [], [], 0, None
        for p in reversed(self._params):            # gradients arrive roughly in reverse order
            k = (p.dtype, p.device)
            nbytes = p.numel() * p.element_size()
            if cur and (k != key or cur_bytes + nbytes > cap):
                groups.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            key = k
        if cur:
            groups.append(cur)
        for g in groups:
            b = _Bucket(g, g[0].dtype, g[0].device, self.symm, self.fp32_master_grads)
            for p, v in zip(g, b.views):
                p.grad = v                          # the gradient IS the bucket slice
                self._bucket_of[id(p)] = b
                self._view_of[id(p)] = v
            self.buckets.append(b)

    def _make_hook(self, p):
        def hook(param):
            b = self._bucket_of[id(param)]
            v = self._view_of[id(param)]
            if param.grad is not None and param.grad.data_ptr() != v.data_ptr():
                # someone replaced .grad (e.g. zero_grad(set_to_none=True)): fold it back into the bucket
                v.copy_(param.grad)
                param.grad = v
            b.pending -= 1
            if b.pending == 0 and self.require_grad_sync and self.world_size > 1:
                self._launch(b)
        return hook

    # ------------------------------------------------------------------ reduction
    def _launch(self, b: _Bucket):
        b.launched = True
        scale = 1.0 / self.world_size
        timed = self.metrics is not None
        b.t0 = b.seconds = None

        def start_event():
            if timed:
                b.t0 = torch.cuda.Event(enable_timing=True)
                b.t0.record(self._comm_stream)
        if b.channel is not None:
            cur = torch.cuda.current_stream(b.flat.device)
            self._comm_stream.wait_stream(cur)
            with torch.cuda.stream(self._comm_stream):
                start_event()
                ch = b.channel
                if b.master is not None:
                    N.check(N.lib().ptb_ddp_allreduce_master(ch.bufs, b.master_ptrs, ch.flag_ptrs, self.rank, self.world_size,
                                                             b.numel, scale, ch.next_seq(), ch.ticket.data_ptr(),
                                                             ch.status.data_ptr(), self.comm_ctas,
                                                             self._comm_stream.cuda_stream), "ddp_allreduce_master")
                else:
                    N.check(N.lib().ptb_ddp_allreduce(ch.bufs, ch.flag_ptrs, self.rank, self.world_size, b.numel,
                                                      int(b.flat.dtype == torch.bfloat16), scale, ch.next_seq(), ch.ticket.data_ptr(),
                                                      ch.status.data_ptr(), self.comm_ctas, self._comm_stream.cuda_stream), "ddp_allreduce")
                b.event = torch.cuda.Event(enable_timing=timed)
                b.event.record(self._comm_stream)
        elif isinstance(self.process_group, TorchProcessGroup) and b.flat.is_cuda:
            cur = torch.cuda.current_stream(b.flat.device)
            self._comm_stream.wait_stream(cur)
            with torch.cuda.stream(self._comm_stream):
                start_event()
                self.process_group.all_reduce(b.flat, ReduceOp.AVG)
                b.event = torch.cuda.Event(enable_timing=timed)
                b.event.record(self._comm_stream)
        else:
            import time
            t0 = time.perf_counter()
            self.process_group.all_reduce(b.flat, ReduceOp.SUM)
            b.flat.mul_(scale)
            b.seconds = time.perf_counter() - t0

    def finish_gradient_synchronization(self):
        """Wait for the in-flight bucket reductions (and reduce buckets whose hooks never completed,
        e.g. parameters unused in this step).  Call after ``backward()`` and before ``optimizer.step()``."""
        if self.world_size > 1 and self.require_grad_sync:
            for b in self.buckets:
                if not b.launched:
                    self._launch(b)
        self._finish_calls += 1
        look = self.check_every > 0 and self._finish_calls % self.check_every == 0
        staged = []
        for i, b in enumerate(self.buckets):
            if b.event is not None:
                torch.cuda.current_stream(b.flat.device).wait_event(b.event)
                if self.metrics is not None and getattr(b, "t0", None) is not None:
                    b.event.synchronize()
                    b.seconds = b.t0.elapsed_time(b.event) / 1e3
                b.event = None
                if look and b.channel is not None:
                    staged.append((b.channel, b.channel.stage_status(self._comm_stream)))
            if self.metrics is not None and getattr(b, "seconds", None) is not None:
                self.metrics.collective(f"ddp bucket {i}", b.seconds, b.numel * b.flat.element_size(), self.world_size,
                                        kind="all_reduce", fused=b.channel is not None)
                b.seconds = None
            b.launched = False
            b.pending = len(b.params)
        # a reduction kernel that ran out of time left its bucket unreduced: say so before anybody steps on it
        for ch, ev in staged:
            ch.raise_if_failed(ev)

    def master_grad(self, param):
        """The fp32 reduced gradient of ``param`` (``fp32_master_grads=True`` and a bf16 parameter), else None."""
        b = self._bucket_of.get(id(param))
        if b is None or b.master_views is None:
            return None
        return b.master_views[[id(q) for q in b.params].index(id(param))]

    def sync_gradients(self):
        """Reduce every bucket now, regardless of hooks (the reference's explicit entry point)."""
        if self.world_size > 1:
            for b in self.buckets:
                self._launch(b)
        self.finish_gradient_synchronization()

    allreduce_grads = sync_gradients

    def check(self):
        for b in self.buckets:
            if b.channel is not None:
                b.channel.check()

    @contextlib.contextmanager
    def no_sync(self):
        """Skip gradient reduction inside the block; gradients keep accumulating in the buckets and the
        next synchronised backward reduces the accumulated sum.  Nests and restores the prior value."""
        prev = self.require_grad_sync
        self.require_grad_sync = False
        try:
            yield
        finally:
            self.require_grad_sync = prev
            for b in self.buckets:
                b.pending = len(b.params)

    def set_require_grad_sync(self, v: bool):
        self.require_grad_sync = bool(v)

    def zero_grad(self, set_to_none: bool = False):
        """Zero the buckets (gradients stay views of them)."""
        for b in self.buckets:
            b.flat.zero_()
            for p, v in zip(b.params, b.views):
                p.grad = v

    def forward(self, *a, **kw):
        if torch.is_grad_enabled():
            for b in self.buckets:
                b.pending = len(b.params)
        return self.module(*a, **kw)


class DDPNoSyncGuard:
    """RAII-style spelling of ``no_sync()`` (torch/distributed/ddp.h:168-186)."""

    def __init__(self, ddp: DistributedDataParallel):
        self.ddp, self.prev = ddp, None

    def __enter__(self):
        self.prev = self.ddp.require_grad_sync
        self.ddp.require_grad_sync = False
        return self

    def __exit__(self, *a):
        self.ddp.require_grad_sync = self.prev
