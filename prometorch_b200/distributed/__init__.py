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

from .process_group import (BackendType, CollectiveTimeout, CountingPG, ProcessGroup, ReduceOp, SharedMemoryBackend,
                            SingleProcessGroup, TorchProcessGroup, make_shared_memory_groups)
from .ddp import DDPNoSyncGuard, DistributedDataParallel, PeerChannel
from .fsdp import (FSDPConfig, FullyShardedDataParallel, OffloadOptimizer, ShardingStrategy, ZeROOptimizer, ZeROStage3,
                   ZeROStage3Config)
from .launcher import DistArgs, launch, parse_dist_args
from .watchdog import DictStore, Heartbeat, RankFailure

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
