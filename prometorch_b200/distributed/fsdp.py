"""FullyShardedDataParallel / ZeRO with the reference's surface
(torch/distributed/fsdp.h:87-96, 161-176, 248-332, 458-492; zero3.h; deepspeed_offload.h).

Sharding rule: every parameter is flattened and cut into ``ceil(N / world)`` elements per rank (the
last shard zero-padded), exactly the reference's (fsdp.h:161-176).  Strategies: ``FULL_SHARD`` (params,
grads and optimizer state sharded; full params are dropped between steps), ``SHARD_GRAD_OP`` (params
stay whole, grads and state sharded), ``NO_SHARD`` (plain data parallel).  Collectives go through the
process group (NCCL on GPUs, Gloo on CPU ranks, threads in tests) instead of files in /dev/shm.

Manual protocol, as in the reference's self-test (fsdp.h:566-616)::

    fsdp.all_gather_params(); loss = f(fsdp(x)); loss.backward()
    fsdp.reduce_scatter_grads(); opt.step()          # opt built over fsdp.local_shards()
    fsdp.all_gather_params()                         # or let forward() do it (auto mode)

The fused B200 path (shards read straight from peer memory by the GEMM, reduce-scatter fused with
AdamW) lives in :mod:`prometorch_b200.parallel.fsdp_fused`."""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from .process_group import ProcessGroup, ReduceOp, SingleProcessGroup, TorchProcessGroup


class ShardingStrategy(enum.IntEnum):
    FULL_SHARD = 0
    SHARD_GRAD_OP = 1
    NO_SHARD = 2


@dataclass
class FSDPConfig:
    rank: int = 0
    world_size: int = 1
    sync_dir: str = "/dev/shm/pt_fsdp"       # kept for source compatibility; unused (no file transport)
    timeout_ms: int = 120000
    poll_us: int = 1000
    strategy: ShardingStrategy = ShardingStrategy.FULL_SHARD
    ShardingStrategy = ShardingStrategy


class FullyShardedDataParallel(nn.Module):
    def __init__(self, module: nn.Module, config: Optional[FSDPConfig] = None, process_group: Optional[ProcessGroup] = None,
                 auto: bool = True):
        super().__init__()
        self.module = module
        if process_group is None:
            import torch.distributed as dist
            process_group = TorchProcessGroup() if dist.is_available() and dist.is_initialized() else SingleProcessGroup()
        self.pg = process_group
        self.config = config or FSDPConfig(rank=process_group.rank, world_size=process_group.world_size)
        self.rank, self.world = process_group.rank, process_group.world_size
        self.strategy = ShardingStrategy(self.config.strategy)
        self.auto = auto
        self._params: List[nn.Parameter] = [p for p in module.parameters()]
        self._shapes = [p.shape for p in self._params]
        self._numels = [p.numel() for p in self._params]
        self._shard_len = [(n + self.world - 1) // self.world for n in self._numels]
        self._gathered = True
        # everyone starts from rank 0's values
        with torch.no_grad():
            for t in list(module.parameters()) + list(module.buffers()):
                self.pg.broadcast(t.data, 0)
        self._shards: List[nn.Parameter] = []
        for p, n, s in zip(self._params, self._numels, self._shard_len):
            flat = torch.zeros(s * self.world, dtype=p.dtype, device=p.device)
            flat[:n] = p.data.reshape(-1)
            sh = nn.Parameter(flat[self.rank * s:(self.rank + 1) * s].clone(), requires_grad=p.requires_grad)
            self._shards.append(sh)
        if self.strategy == ShardingStrategy.FULL_SHARD:
            self.reshard_params()

    # ------------------------------------------------------------------ reference API
    def local_shards(self) -> List[nn.Parameter]:
        """This rank's flat shards (optimise these)."""
        return self._shards

    def flat_params(self) -> List[torch.Tensor]:
        return [p.data.reshape(-1) for p in self._params]

    @torch.no_grad()
    def all_gather_params(self):
        """Rebuild every full parameter from the ranks' shards."""
        if self.strategy == ShardingStrategy.NO_SHARD:
            return
        for p, sh, n, s, shape in zip(self._params, self._shards, self._numels, self._shard_len, self._shapes):
            parts = [torch.empty(s, dtype=sh.dtype, device=sh.device) for _ in range(self.world)]
            self.pg.all_gather(parts, sh.data)
            p.data = torch.cat(parts)[:n].view(shape)
        self._gathered = True

    @torch.no_grad()
    def reshard_params(self):
        """Drop the full parameters (keeps only the local shards)."""
        if self.strategy != ShardingStrategy.FULL_SHARD:
            return
        for p in self._params:
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        self._gathered = False

    @torch.no_grad()
    def reduce_scatter_grads(self, average: bool = True):
        """Sum (average) full gradients over ranks; each rank keeps its slice as ``shard.grad``."""
        for p, sh, n, s in zip(self._params, self._shards, self._numels, self._shard_len):
            if p.grad is None:
                continue
            if self.strategy == ShardingStrategy.NO_SHARD:
                self.pg.all_reduce(p.grad, ReduceOp.AVG if average else ReduceOp.SUM)
                continue
            flat = torch.zeros(s * self.world, dtype=p.grad.dtype, device=p.grad.device)
            flat[:n] = p.grad.reshape(-1)
            out = torch.empty(s, dtype=flat.dtype, device=flat.device)
            self.pg.reduce_scatter(out, list(flat.view(self.world, s).unbind(0)), ReduceOp.AVG if average else ReduceOp.SUM)
            sh.grad = out
            p.grad = None

    @torch.no_grad()
    def sync_shards_to_params(self):
        """SHARD_GRAD_OP / after a step: write updated shards back into the (kept) full parameters."""
        self.all_gather_params()

    def forward(self, *a, **kw):
        if self.auto and not self._gathered:
            self.all_gather_params()
        return self.module(*a, **kw)

    def step_done(self):
        """Call after ``optimizer.step()`` in auto mode: republish parameters, then drop them if fully sharded."""
        self.all_gather_params()

    # ------------------------------------------------------------------ sharded checkpoints
    def shard_state_dict(self):
        return {f"shard.{i}": s.data.clone() for i, s in enumerate(self._shards)} | {"world": torch.tensor(self.world), "rank": torch.tensor(self.rank)}

    def load_shard_state_dict(self, sd):
        if int(sd["world"]) != self.world:
            raise ValueError(f"checkpoint was written with world size {int(sd['world'])}, this run has {self.world}")
        with torch.no_grad():
            for i, s in enumerate(self._shards):
                s.data.copy_(sd[f"shard.{i}"])
        self._gathered = False

    def full_state_dict(self):
        if not self._gathered:
            self.all_gather_params()
        return self.module.state_dict()


class ZeROOptimizer:
    """ZeRO stage 1-3 wrapper: the inner optimizer sees only this rank's shards
    (torch/distributed/fsdp.h:458-492).  ``stage`` is recorded; with FSDP doing the gradient and
    parameter sharding, stages differ only in what the FSDP strategy keeps whole."""

    def __init__(self, shard_params, inner, stage: int = 3):
        if stage not in (1, 2, 3):
            raise ValueError("ZeRO stage must be 1, 2 or 3")
        self.shard_params, self.inner, self.stage = list(shard_params), inner, stage

    def step(self, *a, **kw):
        return self.inner.step(*a, **kw)

    def zero_grad(self, set_to_none: bool = True):
        for p in self.shard_params:
            p.grad = None if set_to_none else (p.grad.zero_() if p.grad is not None else None)

    def state_dict(self):
        return {"stage": self.stage, "inner": self.inner.state_dict()}

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd["inner"])

    @property
    def param_groups(self):
        return self.inner.param_groups


@dataclass
class ZeROStage3Config:
    prefetch: bool = True
    inner_world: int = 1          # ranks inside a node (hierarchical sharding); 1 node here, so equal to world


class ZeROStage3:
    """Stage-3 driver with parameter prefetch: the gather of the next unit is issued on a side stream
    while the current unit computes (the reference prefetches everything with std::async, zero3.h:96-106)."""

    def __init__(self, fsdp: FullyShardedDataParallel, config: Optional[ZeROStage3Config] = None):
        self.fsdp, self.config = fsdp, config or ZeROStage3Config()
        self._stream = torch.cuda.Stream() if torch.cuda.is_available() and fsdp._shards and fsdp._shards[0].is_cuda else None

    def prefetch_params(self):
        if self._stream is None:
            self.fsdp.all_gather_params()
            return
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            self.fsdp.all_gather_params()

    def wait(self):
        if self._stream is not None:
            torch.cuda.current_stream().wait_stream(self._stream)


class OffloadStateBag(dict):
    """The host-side state of one offloaded parameter: fp32 master copy plus whatever the inner optimizer keeps for it."""


class OffloadOptimizer:
    """Keeps optimizer state (and fp32 master copies) in pinned host memory; each step moves gradients to
    the host, steps there and copies parameters back (torch/distributed/deepspeed_offload.h:53-176)."""

    def __init__(self, params, inner_cls, **inner_kw):
        self.dev_params = [p for p in params]
        self.host_params = [nn.Parameter(p.detach().to("cpu", copy=True).float().pin_memory() if torch.cuda.is_available()
                                         else p.detach().to("cpu", copy=True).float()) for p in self.dev_params]
        self.inner = inner_cls(self.host_params, **inner_kw)

    @torch.no_grad()
    def step(self):
        for d, h in zip(self.dev_params, self.host_params):
            if d.grad is not None:
                h.grad = d.grad.detach().to("cpu", non_blocking=False).float()
        self.inner.step()
        for d, h in zip(self.dev_params, self.host_params):
            d.copy_(h.detach().to(d.dtype), non_blocking=True)

    def zero_grad(self, set_to_none: bool = True):
        for d in self.dev_params:
            d.grad = None
        for h in self.host_params:
            h.grad = None

    def state_bags(self):
        """One :class:`OffloadStateBag` per parameter: ``master`` (the fp32 host copy) plus the inner optimizer's state tensors."""
        return [OffloadStateBag(master=h.detach(), **{k: v for k, v in self.inner.state.get(h, {}).items()}) for h in self.host_params]

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd)
