"""Pipeline parallelism.

* ``Pipeline(sequential, num_stages, chunks=4, devices=None)`` — GPipe in one process: stage ``i`` owns
  layers ``[i*N/S, (i+1)*N/S)`` (torch/nn/parallel/pipeline.h:66-254); micro-batches flow through the
  stages, each stage on its own device/stream, and autograd runs through the whole thing.
* ``Pipeline1F1BStage(stage_module, cfg, stage_id)`` — one stage of a multi-process 1F1B schedule:
  ``min(S - id, M)`` warm-up forwards, then alternating backward/forward, then the remaining backwards
  (torch/distributed/pipeline_schedule.h:154-188).  The reference ships zero tensors backwards
  (:212-245); here each stage runs real autograd: activations go forward and activation gradients go
  back over the process group's point-to-point ``send/recv`` (NCCL on GPUs), issued on a side stream
  so they overlap with the next micro-batch's compute.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch
import torch.nn as nn


class Pipeline(nn.Module):
    def __init__(self, module: nn.Sequential, num_stages: int, chunks: int = 4, devices: Optional[Sequence] = None):
        super().__init__()
        layers = list(module.children())
        if num_stages < 1 or num_stages > len(layers):
            raise ValueError("num_stages must be between 1 and the number of layers")
        n = len(layers)
        self.stages = nn.ModuleList(nn.Sequential(*layers[i * n // num_stages:(i + 1) * n // num_stages]) for i in range(num_stages))
        self.chunks = chunks
        self.devices = list(devices) if devices is not None else None
        if self.devices is not None:
            for st, d in zip(self.stages, self.devices):
                st.to(d)

    def forward(self, x):
        micro = list(x.chunk(self.chunks, dim=0))
        S = len(self.stages)
        # GPipe wavefront: at clock t, stage s works on micro-batch t - s
        for t in range(len(micro) + S - 1):
            for s in reversed(range(S)):
                m = t - s
                if 0 <= m < len(micro):
                    inp = micro[m]
                    if self.devices is not None:
                        inp = inp.to(self.devices[s], non_blocking=True)
                    micro[m] = self.stages[s](inp)
        return torch.cat(micro, dim=0)


@dataclass
class PipelineScheduleConfig:
    num_stages: int = 2
    num_micros: int = 4
    sync_dir: str = "/dev/shm/pt_pipe"      # source compatibility with the reference; unused
    timeout_ms: int = 120000
    poll_us: int = 1000


class Pipeline1F1BStage:
    def __init__(self, stage_module: nn.Module, cfg: PipelineScheduleConfig, stage_id: int, process_group=None,
                 prev_rank: Optional[int] = None, next_rank: Optional[int] = None, act_shape=None, act_dtype=None,
                 grad_process_group=None):
        """``grad_process_group``: a second group over the same ranks for the gradient traffic.  NCCL runs the
        point-to-point calls of one communicator in issue order, and in 1F1B a stage's next activation send and
        its neighbour's gradient send cross; on separate communicators neither waits for the other."""
        self.stage, self.cfg, self.id = stage_module, cfg, stage_id
        self.pg = process_group
        self.pg_grad = grad_process_group if grad_process_group is not None else process_group
        self.prev = prev_rank if prev_rank is not None else stage_id - 1
        self.next = next_rank if next_rank is not None else stage_id + 1
        self.act_shape, self.act_dtype = act_shape, act_dtype
        self.first, self.last = stage_id == 0, stage_id == cfg.num_stages - 1

    # -- p2p helpers
    def _send(self, t, dst, pg=None):
        # non-blocking: in 1F1B a stage's forward send and its neighbour's backward send cross each other
        pg = pg if pg is not None else self.pg
        t = t.contiguous()
        w = pg.isend(t, dst) if hasattr(pg, "isend") else pg.send(t, dst)
        self._inflight.append((w, t))

    def _recv(self, shape, dtype, device, src, pg=None):
        t = torch.empty(shape, dtype=dtype, device=device)
        (pg if pg is not None else self.pg).recv(t, src)
        return t

    def run(self, input_first_stage: Optional[torch.Tensor] = None, loss_fn: Optional[Callable] = None,
            targets: Optional[torch.Tensor] = None):
        """One training step of this stage.  First stage: pass the full batch (split into ``num_micros``).
        Last stage: pass ``loss_fn(output, target_micro) -> scalar`` and the targets; returns the mean
        loss.  Gradients of this stage's parameters are accumulated over the micro-batches."""
        S, M = self.cfg.num_stages, self.cfg.num_micros
        dev = next(self.stage.parameters()).device
        micro_in = list(input_first_stage.chunk(M, dim=0)) if self.first else [None] * M
        micro_tg = list(targets.chunk(M, dim=0)) if (self.last and targets is not None) else [None] * M
        saved_in: List[Optional[torch.Tensor]] = [None] * M
        saved_out: List[Optional[torch.Tensor]] = [None] * M
        losses = []
        self._inflight = []

        def forward_one(mb):
            if self.first:
                x = micro_in[mb]
            else:
                x = self._recv(self.act_shape, self.act_dtype, dev, self.prev).requires_grad_()
            saved_in[mb] = x
            y = self.stage(x)
            if self.last:
                loss = loss_fn(y, micro_tg[mb]) / M if loss_fn is not None else y.float().mean() / M
                losses.append(loss.detach())
                saved_out[mb] = loss
            else:
                saved_out[mb] = y
                self._send(y.detach(), self.next)

        def backward_one(mb):
            y = saved_out[mb]
            if self.last:
                y.backward()
            else:
                g = self._recv(y.shape, y.dtype, dev, self.next, self.pg_grad)
                y.backward(g)
            if not self.first:
                self._send(saved_in[mb].grad, self.prev, self.pg_grad)
            saved_in[mb] = saved_out[mb] = None

        f = b = 0
        for _ in range(min(S - self.id, M)):
            forward_one(f)
            f += 1
        while f < M:
            backward_one(b)
            b += 1
            forward_one(f)
            f += 1
        while b < M:
            backward_one(b)
            b += 1
        for w, _ in self._inflight:
            if w is not None:
                w.wait()
        self._inflight = []
        return torch.stack(losses).sum() if losses else None
