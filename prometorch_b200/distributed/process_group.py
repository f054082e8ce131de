"""Process groups: the collective interface and its backends.

The reference has five transports (TCP star, /dev/shm, files, in-process
threads, a dormant NCCL wrapper; torch/distributed/ddp.cpp and
distributed.h:72-388).  Here there is one interface, ``ProcessGroup``
{``all_reduce, broadcast, barrier, all_gather, reduce_scatter``}, and:

* ``TorchProcessGroup``  — ``torch.distributed`` (``nccl`` on GPUs, ``gloo`` on
  CPU ranks); the plumbing under the fused kernels and the baseline path.
* ``SharedMemoryBackend`` — several ranks as threads of one process sharing a
  condition-variable barrier (unit tests; same role as distributed.h:99-215).
* ``CountingPG``          — counts calls and moves no data: the fake the
  ``no_sync()`` tests use (tests/test_ddp_no_sync.cpp:61-77 in the reference).

Timeouts raise ``CollectiveTimeout``; nothing waits forever.
"""
from __future__ import annotations

import datetime
import os
import threading
import time
from typing import List, Optional, Sequence

import torch


class ReduceOp:
    SUM, AVG, MAX, MIN = 0, 1, 2, 3


class BackendType:
    SHARED_MEMORY, NCCL, GLOO = 0, 1, 2


class CollectiveTimeout(RuntimeError):
    """A collective did not complete within its budget (a rank died, stalled or never joined)."""


class ProcessGroup:
    rank: int = 0
    world_size: int = 1

    def all_reduce(self, tensor: torch.Tensor, op: int = ReduceOp.SUM):
        raise NotImplementedError

    def broadcast(self, tensor: torch.Tensor, src: int = 0):
        raise NotImplementedError

    def barrier(self):
        raise NotImplementedError

    def all_gather(self, out: List[torch.Tensor], tensor: torch.Tensor):
        raise NotImplementedError

    def reduce_scatter(self, out: torch.Tensor, inputs: Sequence[torch.Tensor], op: int = ReduceOp.SUM):
        raise NotImplementedError

    def get_rank(self):
        return self.rank

    def get_world_size(self):
        return self.world_size


class SingleProcessGroup(ProcessGroup):
    """world_size 1: every collective is the identity."""

    def all_reduce(self, tensor, op=ReduceOp.SUM):
        return tensor

    def broadcast(self, tensor, src=0):
        return tensor

    def barrier(self):
        pass

    def all_gather(self, out, tensor):
        out[0].copy_(tensor)

    def reduce_scatter(self, out, inputs, op=ReduceOp.SUM):
        out.copy_(inputs[0])


class CountingPG(ProcessGroup):
    """Counts collectives and does nothing else."""

    def __init__(self, rank: int = 0, world_size: int = 2):
        self.rank, self.world_size = rank, world_size
        self.all_reduce_calls = self.broadcast_calls = self.barrier_calls = 0
        self.all_reduce_elems = 0

    def all_reduce(self, tensor, op=ReduceOp.SUM):
        self.all_reduce_calls += 1
        self.all_reduce_elems += tensor.numel()
        return tensor

    def broadcast(self, tensor, src=0):
        self.broadcast_calls += 1
        return tensor

    def barrier(self):
        self.barrier_calls += 1

    def all_gather(self, out, tensor):
        for o in out:
            o.copy_(tensor)

    def reduce_scatter(self, out, inputs, op=ReduceOp.SUM):
        out.copy_(inputs[self.rank])


class _SharedState:
    def __init__(self, world_size: int, timeout: float):
        self.world_size, self.timeout = world_size, timeout
        self.cv = threading.Condition()
        self.count = 0
        self.generation = 0
        self.slots: List[Optional[torch.Tensor]] = [None] * world_size
        self.result = None


class SharedMemoryBackend(ProcessGroup):
    """Ranks are threads of one process.  Create all ranks with :func:`make_shared_memory_groups`."""

    def __init__(self, state: _SharedState, rank: int):
        self.state, self.rank, self.world_size = state, rank, state.world_size

    def _rendezvous(self, value, combine):
        st = self.state
        with st.cv:
            gen = st.generation
            st.slots[self.rank] = value
            st.count += 1
            if st.count == st.world_size:
                st.result = combine(st.slots)
                st.count = 0
                st.generation += 1
                st.cv.notify_all()
            else:
                if not st.cv.wait_for(lambda: st.generation != gen, timeout=st.timeout):
                    raise CollectiveTimeout(f"rank {self.rank}: peers did not arrive within {st.timeout}s")
            return st.result

    def all_reduce(self, tensor, op=ReduceOp.SUM):
        def comb(slots):
            s = torch.stack([t.detach().clone() for t in slots])
            if op == ReduceOp.SUM:
                return s.sum(0)
            if op == ReduceOp.AVG:
                return s.mean(0)
            if op == ReduceOp.MAX:
                return s.amax(0)
            return s.amin(0)
        r = self._rendezvous(tensor, comb)
        self.barrier()                      # nobody overwrites its slot before everyone has read the result
        tensor.copy_(r)
        return tensor

    def broadcast(self, tensor, src=0):
        r = self._rendezvous(tensor, lambda slots: slots[src].detach().clone())
        self.barrier()
        tensor.copy_(r)
        return tensor

    def barrier(self):
        self._rendezvous(None, lambda slots: None)

    def all_gather(self, out, tensor):
        r = self._rendezvous(tensor, lambda slots: [t.detach().clone() for t in slots])
        self.barrier()
        for o, t in zip(out, r):
            o.copy_(t)

    def reduce_scatter(self, out, inputs, op=ReduceOp.SUM):
        r = self._rendezvous(list(inputs), lambda slots: [torch.stack([s[k] for s in slots]).sum(0) for k in range(len(slots))])
        self.barrier()
        out.copy_(r[self.rank] / (self.world_size if op == ReduceOp.AVG else 1))


def make_shared_memory_groups(world_size: int, timeout: float = 30.0) -> List[SharedMemoryBackend]:
    st = _SharedState(world_size, timeout)
    return [SharedMemoryBackend(st, r) for r in range(world_size)]


class FileBackend(ProcessGroup):
    """Ranks are separate processes that meet through a shared directory, no sockets and no daemon: every rank
    publishes its contribution as ``{dir}/{tag}_g{gen}_r{rank}.bin`` (written to a temporary name and renamed, so a
    reader never sees a partial file) followed by an empty ``.ready`` marker, then polls for the others' markers
    every millisecond and raises :class:`CollectiveTimeout` when they do not show up in time.  This is the reference's
    third transport (torch/nn/parallel/tensor_parallel.h:85-189, torch/distributed/fsdp.h:101-158); here it serves
    CPU jobs and tests, the GPU paths use peer memory."""

    def __init__(self, directory: str, rank: int, world_size: int, tag: str = "pg", timeout: float = 30.0, poll: float = 1e-3):
        self.dir, self.rank, self.world_size, self.tag, self.timeout, self.poll = directory, rank, world_size, tag, timeout, poll
        self.gen = 0
        os.makedirs(directory, exist_ok=True)

    def _path(self, gen: int, rank: int, kind: str = "bin") -> str:
        return os.path.join(self.dir, f"{self.tag}_g{gen}_r{rank}.{kind}")

    def _publish(self, gen: int, tensor: Optional[torch.Tensor]):
        path = self._path(gen, self.rank)
        tmp = path + f".tmp{os.getpid()}"
        with open(tmp, "wb") as f:
            if tensor is not None:
                t = tensor.detach().cpu().contiguous()
                f.write((t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes())
        os.replace(tmp, path)
        open(self._path(gen, self.rank, "ready"), "wb").close()

    def _fetch(self, gen: int, rank: int, like: torch.Tensor) -> torch.Tensor:
        deadline = time.monotonic() + self.timeout
        ready = self._path(gen, rank, "ready")
        while not os.path.exists(ready):
            if time.monotonic() > deadline:
                raise CollectiveTimeout(f"rank {self.rank}: rank {rank} did not publish generation {gen} within {self.timeout}s")
            time.sleep(self.poll)
        with open(self._path(gen, rank), "rb") as f:
            raw = f.read()
        if like is None:
            return None
        src = torch.frombuffer(bytearray(raw), dtype=torch.uint16 if like.dtype == torch.bfloat16 else like.dtype)
        src = src.view(torch.bfloat16) if like.dtype == torch.bfloat16 else src
        return src.view(like.shape).clone()

    def _exchange(self, tensor: Optional[torch.Tensor], like: Optional[torch.Tensor] = None, only: Optional[int] = None):
        """Publish ``tensor`` (or nothing), read what rank ``only`` (or every rank) published; clean up two generations back."""
        gen = self.gen
        self.gen += 1
        self._publish(gen, tensor)
        like = like if like is not None else tensor
        ranks = range(self.world_size) if only is None else [only]
        got = {r: (tensor.detach().cpu().clone() if r == self.rank and tensor is not None else self._fetch(gen, r, like)) for r in ranks}
        if only is not None:                                  # everyone must have read before anyone races ahead by two
            for r in range(self.world_size):
                self._fetch(gen, r, None)
        for kind in ("bin", "ready"):                         # all ranks are past generation gen - 2 once they published gen
            old = self._path(gen - 2, self.rank, kind)
            if gen >= 2 and os.path.exists(old):
                os.remove(old)
        return got

    def all_reduce(self, tensor, op=ReduceOp.SUM):
        got = self._exchange(tensor)
        s = torch.stack([got[r].to(torch.float32) if tensor.dtype == torch.bfloat16 else got[r] for r in range(self.world_size)])
        r = s.sum(0) if op == ReduceOp.SUM else s.mean(0) if op == ReduceOp.AVG else s.amax(0) if op == ReduceOp.MAX else s.amin(0)
        tensor.copy_(r.to(tensor.dtype))
        return tensor

    def broadcast(self, tensor, src=0):
        got = self._exchange(tensor if self.rank == src else None, like=tensor, only=src)
        tensor.copy_(got[src])
        return tensor

    def barrier(self):
        self._exchange(None, like=None)

    def all_gather(self, out, tensor):
        got = self._exchange(tensor)
        for r, o in enumerate(out):
            o.copy_(got[r])

    def reduce_scatter(self, out, inputs, op=ReduceOp.SUM):
        got = self._exchange(torch.stack([t.detach() for t in inputs]))
        r = torch.stack([got[k][self.rank] for k in range(self.world_size)]).sum(0)
        out.copy_(r / (self.world_size if op == ReduceOp.AVG else 1))


_TORCH_OPS = None


def _torch_op(op):
    import torch.distributed as dist
    return {ReduceOp.SUM: dist.ReduceOp.SUM, ReduceOp.AVG: dist.ReduceOp.AVG, ReduceOp.MAX: dist.ReduceOp.MAX,
            ReduceOp.MIN: dist.ReduceOp.MIN}[op]


class TorchProcessGroup(ProcessGroup):
    """``torch.distributed`` group (``nccl`` / ``gloo``).  Gloo has no AVG: it is SUM then a divide."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world_size = dist.get_world_size(self.group)
        self.backend = dist.get_backend(self.group)

    def _wrap(self, fn):
        try:
            return fn()
        except RuntimeError as e:                      # gloo / nccl timeouts surface as RuntimeError
            msg = str(e).lower()
            if "timeout" in msg or "timed out" in msg or "connection" in msg:
                raise CollectiveTimeout(str(e)) from e
            raise

    def all_reduce(self, tensor, op=ReduceOp.SUM, async_op: bool = False):
        if op == ReduceOp.AVG and self.backend != "nccl":
            w = self._wrap(lambda: self.dist.all_reduce(tensor, self.dist.ReduceOp.SUM, group=self.group))
            tensor.div_(self.world_size)
            return w
        return self._wrap(lambda: self.dist.all_reduce(tensor, _torch_op(op), group=self.group, async_op=async_op))

    def broadcast(self, tensor, src=0):
        return self._wrap(lambda: self.dist.broadcast(tensor, self.dist.get_global_rank(self.group, src), group=self.group))

    def barrier(self):
        return self._wrap(lambda: self.dist.barrier(group=self.group))

    def all_gather(self, out, tensor):
        return self._wrap(lambda: self.dist.all_gather(list(out), tensor, group=self.group))

    def all_gather_into(self, out: torch.Tensor, tensor: torch.Tensor, async_op=False):
        return self._wrap(lambda: self.dist.all_gather_into_tensor(out, tensor, group=self.group, async_op=async_op))

    def reduce_scatter(self, out, inputs, op=ReduceOp.SUM):
        if self.backend == "nccl":
            return self._wrap(lambda: self.dist.reduce_scatter(out, list(inputs), _torch_op(op), group=self.group))
        # gloo has no reduce_scatter: all-reduce each piece, keep ours
        for k, t in enumerate(inputs):
            buf = t.clone()
            self.all_reduce(buf, op)
            if k == self.rank:
                out.copy_(buf)

    def send(self, tensor, dst):
        return self._wrap(lambda: self.dist.send(tensor, self.dist.get_global_rank(self.group, dst), group=self.group))

    def isend(self, tensor, dst):
        """Non-blocking send; returns a work handle with ``wait()``."""
        return self._wrap(lambda: self.dist.isend(tensor, self.dist.get_global_rank(self.group, dst), group=self.group))

    def recv(self, tensor, src):
        return self._wrap(lambda: self.dist.recv(tensor, self.dist.get_global_rank(self.group, src), group=self.group))
