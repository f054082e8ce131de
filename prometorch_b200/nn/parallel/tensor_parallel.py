"""Tensor-parallel linear layers.

``ColumnParallelLinear(in, out, tp, gather_output=True, bias, init_seed)`` shards the rows of
``W[out, in]``; ``RowParallelLinear(in, out, tp, input_is_parallel=True, bias, init_seed)`` shards its
columns and sums partial outputs.  Constructor arguments, divisibility rules and the
"sharded == unsharded" initialisation (one seeded stream generates the full matrix, each rank keeps
its slice) follow torch/nn/parallel/tensor_parallel.h:294-554.  Unlike the reference, whose
collectives are forward-only, these are differentiable: the backward of the column layer
all-reduces dX, the backward of the row layer is local.

``sequence_parallel=True`` switches to the Megatron sequence-parallel form used by the 7B
TP x PP config: activations outside the pair are sharded by tokens; the column layer is
all-gather(X) -> GEMM and the row layer GEMM -> reduce-scatter.  With a symmetric-memory group on
CUDA both are ONE tcgen05 GEMM launch: the column GEMM's TMA producer pulls each A tile from the
peer that owns those tokens, and the row GEMM's epilogue adds each output tile into its owner's
buffer over NVLink (csrc/gemm_sm100.cuh).  Otherwise they run as process-group collectives around
a local GEMM — that path is the baseline the fused one is measured against.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...distributed.process_group import ProcessGroup, ReduceOp, SingleProcessGroup, TorchProcessGroup
from ...ops.gemm import linear as fused_linear


@dataclass
class TPConfig:
    rank: int = 0
    world_size: int = 1
    sync_dir: str = "/dev/shm/pt_tp"          # source compatibility with the reference; unused
    timeout_us: int = 120_000_000
    process_group: Optional[ProcessGroup] = None
    symm: object = None                       # parallel.symm.SymmGroup for the fused peer-memory path

    def pg(self) -> ProcessGroup:
        if self.process_group is None:
            import torch.distributed as dist
            self.process_group = TorchProcessGroup() if (dist.is_available() and dist.is_initialized() and self.world_size > 1) \
                else SingleProcessGroup()
        return self.process_group


# ----------------------------------------------------------------------------- plain collectives (reference names)
def tp_all_gather(x: torch.Tensor, tp: TPConfig, dim: int = -1) -> torch.Tensor:
    if tp.world_size == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(tp.world_size)]
    tp.pg().all_gather(parts, x.contiguous())
    return torch.cat(parts, dim=dim)


def tp_all_reduce_sum(x: torch.Tensor, tp: TPConfig) -> torch.Tensor:
    if tp.world_size > 1:
        tp.pg().all_reduce(x, ReduceOp.SUM)
    return x


def tp_barrier(tp: TPConfig):
    if tp.world_size > 1:
        tp.pg().barrier()


# ----------------------------------------------------------------------------- differentiable collectives
class _CopyToRegion(torch.autograd.Function):        # identity forward, all-reduce backward
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        return tp_all_reduce_sum(g, ctx.tp), None


class _ReduceFromRegion(torch.autograd.Function):    # all-reduce forward, identity backward
    @staticmethod
    def forward(ctx, x, tp):
        return tp_all_reduce_sum(x.contiguous().clone(), tp)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherLastDim(torch.autograd.Function):       # all-gather forward, slice backward
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp, ctx.n = tp, x.shape[-1]
        return tp_all_gather(x, tp, -1)

    @staticmethod
    def backward(ctx, g):
        r = ctx.tp.rank
        return g[..., r * ctx.n:(r + 1) * ctx.n].contiguous(), None


class _GatherTokens(torch.autograd.Function):        # sequence parallel: all-gather dim 0 fwd, reduce-scatter bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp, ctx.n = tp, x.shape[0]
        return tp_all_gather(x, tp, 0)

    @staticmethod
    def backward(ctx, g):
        tp = ctx.tp
        out = torch.empty(ctx.n, *g.shape[1:], dtype=g.dtype, device=g.device)
        tp.pg().reduce_scatter(out, list(g.contiguous().view(tp.world_size, ctx.n, *g.shape[1:]).unbind(0)), ReduceOp.SUM)
        return out, None


class _ScatterTokens(torch.autograd.Function):       # sequence parallel: reduce-scatter dim 0 fwd, all-gather bwd
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        n = x.shape[0] // tp.world_size
        out = torch.empty(n, *x.shape[1:], dtype=x.dtype, device=x.device)
        tp.pg().reduce_scatter(out, list(x.contiguous().view(tp.world_size, n, *x.shape[1:]).unbind(0)), ReduceOp.SUM)
        return out

    @staticmethod
    def backward(ctx, g):
        return tp_all_gather(g, ctx.tp, 0), None


def _seeded_full(out_f: int, in_f: int, seed: int, with_bias: bool):
    """The full ``[out, in]`` weight (and bias) from one seeded stream, U(-1/sqrt(in), 1/sqrt(in))."""
    g = torch.Generator().manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    bound = 1.0 / math.sqrt(in_f)
    w = (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound
    b = (torch.rand(out_f, generator=g) * 2 - 1) * bound if with_bias else None
    return w, b


class ColumnParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, tp: TPConfig, gather_output: bool = True, bias: bool = True,
                 init_seed: Optional[int] = 1234567, sequence_parallel: bool = False, device=None, dtype=None):
        """``init_seed=None`` initialises only the local shard, directly on ``device`` (large models: the full
        matrix is never materialised); with a seed every rank cuts its shard out of the same full matrix."""
        super().__init__()
        if out_features % tp.world_size:
            raise ValueError("ColumnParallelLinear: out_features must be divisible by world_size")
        self.in_features, self.out_features, self.tp = in_features, out_features, tp
        self.gather_output, self.sequence_parallel = gather_output, sequence_parallel
        self.shard = out_features // tp.world_size
        r = tp.rank
        if init_seed is None:
            self.weight = nn.Parameter(torch.empty(self.shard, in_features, device=device, dtype=dtype).normal_(std=0.02))
            self.bias = nn.Parameter(torch.zeros(self.shard, device=device, dtype=dtype)) if bias else None
        else:
            w, b = _seeded_full(out_features, in_features, init_seed, bias)
            self.weight = nn.Parameter(w[r * self.shard:(r + 1) * self.shard].clone().to(device=device, dtype=dtype))
            self.bias = nn.Parameter(b[r * self.shard:(r + 1) * self.shard].clone().to(device=device, dtype=dtype)) if bias else None

    def forward(self, x):
        tp = self.tp
        if self.sequence_parallel and tp.world_size > 1:
            from .fused_tp import column_sp_forward
            shp = x.shape
            y = column_sp_forward(x.reshape(-1, shp[-1]), self.weight, self.bias, tp)     # [tokens_full, shard]
            return y
        if tp.world_size > 1:
            x = _CopyToRegion.apply(x, tp)
        y = fused_linear(x, self.weight, self.bias)
        if self.gather_output and tp.world_size > 1:
            y = _GatherLastDim.apply(y, tp)
        return y

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features} (shard {self.shard}), tp={self.tp.world_size}, sp={self.sequence_parallel}"


class RowParallelLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, tp: TPConfig, input_is_parallel: bool = True, bias: bool = True,
                 init_seed: Optional[int] = 7654321, sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        if in_features % tp.world_size:
            raise ValueError("RowParallelLinear: in_features must be divisible by world_size")
        self.in_features, self.out_features, self.tp = in_features, out_features, tp
        self.input_is_parallel, self.sequence_parallel = input_is_parallel, sequence_parallel
        self.shard = in_features // tp.world_size
        r = tp.rank
        if init_seed is None:
            self.weight = nn.Parameter(torch.empty(out_features, self.shard, device=device, dtype=dtype).normal_(std=0.02))
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype)) if bias else None
        else:
            w, b = _seeded_full(out_features, in_features, init_seed, bias)
            self.weight = nn.Parameter(w[:, r * self.shard:(r + 1) * self.shard].clone().to(device=device, dtype=dtype))
            self.bias = nn.Parameter(b.clone().to(device=device, dtype=dtype)) if bias else None       # added once, after the reduction

    def forward(self, x, residual=None):
        """``residual`` (optional): returns ``residual + layer(x)``; on the fused sequence-parallel path the addition is
        part of the kernel that sums the ranks' partial tiles."""
        tp = self.tp
        if not self.input_is_parallel and tp.world_size > 1:
            x = x[..., tp.rank * self.shard:(tp.rank + 1) * self.shard]
        if self.sequence_parallel and tp.world_size > 1:
            from .fused_tp import row_sp_forward
            y = row_sp_forward(x.reshape(-1, x.shape[-1]), self.weight, tp, resid=residual)      # [tokens_local, out]
            if residual is not None:
                y = y.view(residual.shape)
        else:
            y = fused_linear(x, self.weight, None)
            if tp.world_size > 1:
                y = _ReduceFromRegion.apply(y, tp)
            if residual is not None:
                y = y + residual
        return y + self.bias if self.bias is not None else y

    def extra_repr(self):
        return f"in={self.in_features} (shard {self.shard}), out={self.out_features}, tp={self.tp.world_size}, sp={self.sequence_parallel}"
