"""Local SGD: every rank takes ``sync_every`` optimizer steps on its own data, then the replicas are averaged.

One all-reduce of the parameters per ``sync_every`` steps instead of one all-reduce of the gradients per step, which is
the regime for ranks joined by slow links.  ``outer_momentum`` > 0 applies the "slow momentum" outer step to the averaged
displacement (the average moves on by ``outer_lr * (momentum * v + displacement)`` instead of by the displacement).  The
reference lists the strategy without an implementation (its distributed README); this one works over any
``torch.distributed`` backend.

    model = LocalSGD(net, sync_every=8)
    for x, y in loader:
        loss(model(x), y).backward(); opt.step(); opt.zero_grad()
        model.step_done()                  # averages on every 8th call; returns True when it did
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn


class LocalSGD(nn.Module):
    def __init__(self, module: nn.Module, sync_every: int = 8, process_group=None, broadcast_parameters: bool = True,
                 outer_momentum: float = 0.0, outer_lr: float = 1.0, warmup_steps: int = 0):
        super().__init__()
        import torch.distributed as dist
        self.module, self.sync_every, self.group, self.dist = module, int(sync_every), process_group, dist
        self.outer_momentum, self.outer_lr, self.warmup_steps = float(outer_momentum), float(outer_lr), int(warmup_steps)
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.local_steps = 0
        self.total_steps = 0
        self.syncs = 0
        self._anchor: Optional[torch.Tensor] = None          # the last averaged parameters (outer momentum only)
        self._velocity: Optional[torch.Tensor] = None
        if broadcast_parameters and self.world > 1:
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t.data, dist.get_global_rank(process_group, 0) if process_group is not None else 0, group=process_group)
        if self.outer_momentum > 0:
            self._anchor = self._flat().clone()
            self._velocity = torch.zeros_like(self._anchor)

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def _params(self):
        return [p for p in self.module.parameters() if p.requires_grad]

    def _flat(self) -> torch.Tensor:
        return torch.cat([p.data.reshape(-1).float() for p in self._params()])

    @torch.no_grad()
    def _write(self, flat: torch.Tensor):
        o = 0
        for p in self._params():
            n = p.numel()
            p.data.copy_(flat[o:o + n].view_as(p))
            o += n

    @torch.no_grad()
    def average(self):
        """Average the replicas now (one all-reduce of all parameters as one flat buffer)."""
        flat = self._flat()
        if self.world > 1:
            self.dist.all_reduce(flat, group=self.group)
            flat /= self.world
        if self.outer_momentum > 0:
            step = flat - self._anchor
            self._velocity.mul_(self.outer_momentum).add_(step)
            flat = self._anchor + self.outer_lr * self._velocity
            self._anchor = flat.clone()
        self._write(flat)
        for b in self.module.buffers():                       # running statistics: averaged too
            if b.dtype.is_floating_point and self.world > 1:
                self.dist.all_reduce(b.data, group=self.group)
                b.data /= self.world
        self.local_steps = 0
        self.syncs += 1

    def step_done(self) -> bool:
        """Call after every optimizer step.  During ``warmup_steps`` the replicas are averaged every step."""
        self.local_steps += 1
        self.total_steps += 1
        if self.total_steps <= self.warmup_steps or self.local_steps >= self.sync_every:
            self.average()
            return True
        return False
