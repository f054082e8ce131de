"""Multi-rank training: process groups, DDP (+``no_sync``), FSDP / ZeRO, launcher, failure detection.

Module-level functions mirror the reference's Python surface
(python/promethorch/distributed/__init__.py:218-232): ``init_process_group(backend, rank, world_size,
master_addr, master_port)``, ``all_reduce``, ``broadcast``, ``barrier``, ``get_rank``,
``get_world_size``, ``is_initialized``.  Backends: ``shared_memory`` (single process), ``gloo`` /
``tcp`` (CPU ranks over TCP), ``nccl`` (one process per GPU)."""
from __future__ import annotations

import datetime
import os
from typing import Optional

import torch

from .process_group import (BackendType, CollectiveTimeout, CountingPG, FileBackend, ProcessGroup, ReduceOp, SharedMemoryBackend,
                            SingleProcessGroup, TorchProcessGroup, make_shared_memory_groups)
from .ddp import DDPNoSyncGuard, DistributedDataParallel, PeerChannel
from .checkpoint import load_sharded, save_sharded  # noqa: F401
from .fsdp import (FSDPConfig, FullyShardedDataParallel, OffloadOptimizer, OffloadStateBag, ShardingStrategy, ZeROOptimizer, ZeROStage3,
                   ZeROStage3Config)
from .launcher import DistArgs, launch, parse_dist_args
from .watchdog import DictStore, Heartbeat, RankFailure
from .local_sgd import LocalSGD  # noqa: F401
from .process_group import TorchProcessGroup as NCCLBackend  # noqa: F401  (the reference's name for the NCCL-backed group)

_current_pg: Optional[ProcessGroup] = None


def init_process_group(backend: str = "shared_memory", rank: Optional[int] = None, world_size: Optional[int] = None,
                       master_addr: str = "127.0.0.1", master_port: int = 29500, timeout_sec: float = 300.0,
                       device_id=None) -> ProcessGroup:
    """Bind this process to a group.  ``rank`` / ``world_size`` default to the ``RANK`` / ``WORLD_SIZE``
    environment (torchrun and :func:`launch` set them)."""
    global _current_pg
    rank = int(os.environ.get("RANK", 0)) if rank is None else rank
    world_size = int(os.environ.get("WORLD_SIZE", 1)) if world_size is None else world_size
    b = backend.lower()
    if b in ("shared_memory", "single") or world_size == 1 and b not in ("nccl", "gloo", "tcp"):
        _current_pg = SingleProcessGroup()
        return _current_pg
    import torch.distributed as dist
    if b == "tcp":
        b = "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", master_addr)
        os.environ.setdefault("MASTER_PORT", str(master_port))
        kw = dict(backend=b, rank=rank, world_size=world_size, timeout=datetime.timedelta(seconds=timeout_sec),
                  init_method=f"tcp://{os.environ['MASTER_ADDR']}:{os.environ['MASTER_PORT']}")
        if device_id is not None:
            kw["device_id"] = device_id
        dist.init_process_group(**kw)
    _current_pg = TorchProcessGroup()
    return _current_pg


def destroy_process_group():
    global _current_pg
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
    _current_pg = None


def is_initialized() -> bool:
    return _current_pg is not None


def _pg() -> ProcessGroup:
    if _current_pg is None:
        raise RuntimeError("init_process_group() was not called")
    return _current_pg


def get_rank() -> int:
    return _pg().rank


def get_world_size() -> int:
    return _pg().world_size


def all_reduce(tensor: torch.Tensor, op: int = ReduceOp.SUM):
    return _pg().all_reduce(tensor, op)


def all_reduce_inplace(tensor: torch.Tensor):
    return _pg().all_reduce(tensor, ReduceOp.SUM)


def broadcast(tensor: torch.Tensor, src: int = 0):
    return _pg().broadcast(tensor, src)


def barrier():
    return _pg().barrier()


def all_gather(out, tensor):
    return _pg().all_gather(out, tensor)


def reduce_scatter(out, inputs, op: int = ReduceOp.SUM):
    return _pg().reduce_scatter(out, inputs, op)


def finish_gradient_synchronization(ddp: DistributedDataParallel):
    ddp.finish_gradient_synchronization()


def sync_gradients(ddp: DistributedDataParallel):
    ddp.sync_gradients()


class SyncBatchNorm(torch.nn.SyncBatchNorm):
    """Batch norm with statistics reduced over ranks (the reference's three small all-reduces,
    torch/distributed/distributed.h:765-966, are one fused reduction here)."""

    @classmethod
    def convert_sync_batchnorm(cls, module, process_group=None):
        g = process_group.group if isinstance(process_group, TorchProcessGroup) else None
        return torch.nn.SyncBatchNorm.convert_sync_batchnorm(module, g)


# ----------------------------------------------------------------------------- remaining names of the reference's C++ surface
from dataclasses import dataclass as _dataclass


@_dataclass
class DDPConfig:
    """Connection settings of the reference's process-group singleton (torch/distributed/ddp.h:37-52)."""
    rank: int = 0
    world_size: int = 1
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    timeout_sec: float = 300.0
    backend: str = "gloo"

    def init(self) -> ProcessGroup:
        return init_process_group(self.backend, self.rank, self.world_size, self.master_addr, self.master_port, self.timeout_sec)


def init_process_group_single_rank() -> ProcessGroup:
    """A world of one (every collective is the identity)."""
    return init_process_group("shared_memory", 0, 1)


def all_gather_inplace(buffer: torch.Tensor):
    """``buffer`` holds ``world_size`` equal slots; this rank's slot is filled in, the others arrive from their owners
    (the in-place form of ddp.h's ``all_gather_inplace``)."""
    pg = _pg()
    w, r = pg.world_size, pg.rank
    slots = list(buffer.view(w, -1).unbind(0))
    mine = slots[r].clone()
    pg.all_gather(slots, mine)
    return buffer


class _GatherHandle:
    def __init__(self, work, buffer):
        self.work, self.buffer = work, buffer


def all_gather_post(buffer: torch.Tensor) -> _GatherHandle:
    """Start an in-place all-gather; finish it with :func:`all_gather_wait` (overlaps with compute on NCCL)."""
    pg = _pg()
    if isinstance(pg, TorchProcessGroup) and pg.backend == "nccl":
        mine = buffer.view(pg.world_size, -1)[pg.rank].clone()
        return _GatherHandle(pg.all_gather_into(buffer.view(-1), mine, async_op=True), buffer)
    all_gather_inplace(buffer)
    return _GatherHandle(None, buffer)


def all_gather_wait(handle: _GatherHandle) -> torch.Tensor:
    if handle.work is not None:
        handle.work.wait()
    return handle.buffer


def scatter(tensor: torch.Tensor, rank: int, world_size: int) -> torch.Tensor:
    """Rank ``rank``'s contiguous share of dim 0 (the last rank takes the remainder)."""
    per = tensor.shape[0] // world_size
    lo = rank * per
    hi = tensor.shape[0] if rank == world_size - 1 else lo + per
    return tensor[lo:hi]


def data_parallel_step(fn, data: torch.Tensor, labels: torch.Tensor, params, world_size: int) -> float:
    """One data-parallel step inside a single process (torch/distributed/distributed.h:1159-1215): the batch is cut into
    ``world_size`` shards, ``fn(rank, data_shard, label_shard)`` runs forward + backward for each and returns its loss,
    and the parameters end up with the AVERAGE of the shard gradients.  The shards share the parameters, so their
    backward passes accumulate into the same ``.grad``; the ranks run one after another because autograd accumulation
    into a shared tensor is not safe across threads."""
    losses = []
    for rank in range(world_size):
        losses.append(float(fn(rank, scatter(data, rank, world_size), scatter(labels, rank, world_size))))
    with torch.no_grad():
        for p in params:
            if p.requires_grad and p.grad is not None:
                p.grad.div_(world_size)
    return sum(losses) / max(len(losses), 1)


def __getattr__(name):
    # the pipeline schedule classes live with the other nn.parallel modules (which import this package): resolved lazily
    if name in ("Pipeline1F1BStage", "PipelineScheduleConfig", "Pipeline"):
        from ..nn.parallel import pipeline as _p
        return getattr(_p, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


@_dataclass
class DistributedContext:
    """Rank, world size and process group in one object (what the reference threads through its distributed helpers)."""
    rank: int = 0
    world_size: int = 1
    process_group: object = None

    @classmethod
    def current(cls) -> "DistributedContext":
        return cls(get_rank(), get_world_size(), _pg()) if is_initialized() else cls()

    @property
    def is_main(self) -> bool:
        return self.rank == 0
