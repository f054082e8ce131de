"""Expert parallelism: the experts of a mixture-of-experts layer spread over the ranks, tokens routed by all-to-all.

Forward: router -> top-k experts per token -> token copies sorted by destination rank -> all-to-all (dispatch) -> each rank
runs its local experts over what it received -> all-to-all back (combine) -> gate-weighted sum per token.  Both all-to-alls
are differentiable (their backward is the all-to-all with the split sizes swapped), so router, experts and inputs all get
gradients.  The dense-equivalent check is `ExpertParallelMoE.dense_forward`, the same layer computed by one process that
holds every expert.

The reference runs mixture-of-experts models (deepseek2) on one device only; this is the multi-rank layer the decode
all-to-all ("dispatch / combine") would be fused into.  Works over gloo (CPU ranks) and nccl.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class _AllToAll(torch.autograd.Function):
    """all_to_all_single over rows with explicit split sizes."""

    @staticmethod
    def forward(ctx, x, in_splits: List[int], out_splits: List[int], group):
        import torch.distributed as dist
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits, input_split_sizes=ctx.out_splits, group=ctx.group)
        return out, None, None, None


class Expert(nn.Module):
    """SwiGLU feed-forward block."""

    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.gate, self.up, self.down = nn.Linear(dim, hidden, bias=False), nn.Linear(dim, hidden, bias=False), nn.Linear(hidden, dim, bias=False)

    def forward(self, x):
        return self.down(F.silu(self.gate(x)) * self.up(x))


class ExpertParallelMoE(nn.Module):
    """`num_experts` experts of which this rank holds ``num_experts / world`` (expert e lives on rank ``e // local``).
    The router is replicated.  ``forward(x)`` takes this rank's tokens ``[..., dim]``."""

    def __init__(self, dim: int, hidden: int, num_experts: int, top_k: int = 2, group=None, normalize_gates: bool = True, seed: Optional[int] = None):
        super().__init__()
        import torch.distributed as dist
        self.group, self.dist = group, dist
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert num_experts % self.world == 0, "the number of experts must divide by the number of ranks"
        self.num_experts, self.top_k, self.local, self.normalize_gates = num_experts, top_k, num_experts // self.world, normalize_gates
        gen = torch.Generator().manual_seed(seed) if seed is not None else None
        self.router = nn.Linear(dim, num_experts, bias=False)
        if gen is not None:                       # the same router on every rank, a different stream per expert
            with torch.no_grad():
                self.router.weight.copy_(torch.randn(num_experts, dim, generator=gen) * dim ** -0.5)
        self.experts = nn.ModuleList(Expert(dim, hidden) for _ in range(self.local))
        if seed is not None:
            for j, e in enumerate(self.experts):
                g = torch.Generator().manual_seed(seed + 1 + self.rank * self.local + j)
                with torch.no_grad():
                    for p in e.parameters():
                        p.copy_(torch.randn(p.shape, generator=g) * p.shape[1] ** -0.5)
        self.last_tokens_per_expert: Optional[torch.Tensor] = None

    def route(self, x2):
        logits = self.router(x2)
        gates, idx = torch.topk(F.softmax(logits.float(), dim=-1), self.top_k, dim=-1)
        if self.normalize_gates:
            gates = gates / gates.sum(-1, keepdim=True)
        return gates.to(x2.dtype), idx, logits

    def forward(self, x):
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        n = x2.shape[0]
        gates, idx, logits = self.route(x2)
        flat_e = idx.reshape(-1)                                            # [n * k] expert of every token copy
        order = torch.argsort(flat_e, stable=True)                           # copies sorted by expert, hence by destination rank
        token_of = torch.arange(n, device=x.device).repeat_interleave(self.top_k)[order]
        send = x2[token_of]
        counts = torch.bincount(flat_e, minlength=self.num_experts)          # copies per expert, from this rank
        self.last_tokens_per_expert = counts.detach()
        if self.world > 1:
            all_counts = torch.empty(self.world, self.num_experts, dtype=counts.dtype, device=counts.device)
            self.dist.all_gather_into_tensor(all_counts.view(-1), counts, group=self.group)
            lo, hi = self.rank * self.local, (self.rank + 1) * self.local
            in_splits = counts.view(self.world, self.local).sum(1).tolist()
            recv_counts = all_counts[:, lo:hi]                               # [source rank, local expert]
            out_splits = recv_counts.sum(1).tolist()
            recv = _AllToAll.apply(send, in_splits, out_splits, self.group)
            # what arrived is ordered (source rank, local expert); run each local expert over its rows of every source
            pieces, offset = [None] * (self.world * self.local), 0
            rows = [[] for _ in range(self.local)]
            for src in range(self.world):
                for j in range(self.local):
                    c = int(recv_counts[src, j])
                    rows[j].append((src, offset, c))
                    offset += c
            for j, e in enumerate(self.experts):
                xs = torch.cat([recv[o:o + c] for _, o, c in rows[j]]) if rows[j] else recv[:0]
                ys = e(xs)
                o2 = 0
                for src, _, c in rows[j]:
                    pieces[src * self.local + j] = ys[o2:o2 + c]
                    o2 += c
            back = _AllToAll.apply(torch.cat(pieces), out_splits, in_splits, self.group)
        else:
            outs, offset = [], 0
            for j, e in enumerate(self.experts):
                c = int(counts[j])
                outs.append(e(send[offset:offset + c]))
                offset += c
            back = torch.cat(outs)
        weight = gates.reshape(-1)[order].unsqueeze(-1)
        y = torch.zeros_like(x2).index_add(0, token_of, back * weight)
        return y.reshape(shape)

    def load_balance_loss(self, x) -> torch.Tensor:
        """Switch-style auxiliary loss: num_experts * sum_e (fraction of copies sent to e) * (mean router probability of e)."""
        x2 = x.reshape(-1, x.shape[-1])
        probs = F.softmax(self.router(x2).float(), dim=-1)
        idx = torch.topk(probs, self.top_k, dim=-1).indices
        frac = torch.bincount(idx.reshape(-1), minlength=self.num_experts).float() / idx.numel()
        return self.num_experts * (frac * probs.mean(0)).sum()

    @staticmethod
    def dense_forward(x, router_weight, experts: List[Expert], top_k: int, normalize_gates: bool = True):
        """The same layer with every expert in one process (the oracle of the tests)."""
        x2 = x.reshape(-1, x.shape[-1])
        gates, idx = torch.topk(F.softmax(F.linear(x2, router_weight).float(), dim=-1), top_k, dim=-1)
        if normalize_gates:
            gates = gates / gates.sum(-1, keepdim=True)
        y = torch.zeros_like(x2)
        for e, ex in enumerate(experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel():
                y = y.index_add(0, tok, ex(x2[tok]) * gates[tok, slot].unsqueeze(-1).to(x2.dtype))
        return y.reshape(x.shape)
