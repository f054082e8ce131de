"""Context parallelism: ring attention over a sequence that is cut into contiguous blocks, one per rank.

Every rank keeps the queries of its block and passes key / value blocks around the ring; partial results are merged with
their log-sum-exp, exactly like the split-KV merge of the decode attention kernel (csrc/decode_kernels.cuh), so the result is
the attention over the whole sequence without any rank ever holding more than two KV blocks.  Backward runs the ring again:
the key / value blocks travel with their gradient accumulators and arrive home after ``world`` hops.  Causal masking is by
block: a block from a later rank is skipped, the rank's own block is triangular, earlier ones are full.

The reference has no sequence or context parallelism (its long-context support is RoPE scaling and a sliding window); this
is the ring wrapper its attention API leaves room for.  Block math is plain tensor code in fp32, so the same functions run
on CPU ranks (gloo) and on GPUs (nccl send / recv).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def _block_attention(q, k, v, scale: float, mask: Optional[torch.Tensor]):
    """(out, lse) of softmax(q k^T * scale + mask) v for one KV block; lse is -inf where a row sees nothing."""
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse)).unsqueeze(-1))
    p = torch.where(torch.isfinite(s), p, torch.zeros_like(p))
    return torch.matmul(p, v), lse


def _merge(out, lse, o2, l2):
    """Combine two partial attentions over disjoint key sets."""
    new = torch.logaddexp(lse, l2)
    safe = torch.where(torch.isfinite(new), new, torch.zeros_like(new))
    w1 = torch.where(torch.isfinite(lse), torch.exp(lse - safe), torch.zeros_like(lse)).unsqueeze(-1)
    w2 = torch.where(torch.isfinite(l2), torch.exp(l2 - safe), torch.zeros_like(l2)).unsqueeze(-1)
    return out * w1 + o2 * w2, new


def _exchange(dist, group, rank, world, tensors):
    """Send `tensors` to the next rank of the ring and receive the previous rank's; returns the received ones."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    g = (lambda r: dist.get_global_rank(group, r)) if group is not None else (lambda r: r)
    recv = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, recv):
        ops.append(dist.P2POp(dist.isend, t.contiguous(), g(nxt), group))
        ops.append(dist.P2POp(dist.irecv, r, g(prv), group))
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return recv


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, group):
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        qf, kb, vb = q.float(), k.float().contiguous(), v.float().contiguous()
        T = q.shape[-2]
        tri = torch.ones(T, k.shape[-2], dtype=torch.bool, device=q.device).tril() if causal else None
        out = torch.zeros_like(qf)
        lse = torch.full(q.shape[:-1], float("-inf"), dtype=torch.float32, device=q.device)
        for s in range(world):
            owner = (rank - s) % world
            if not causal or owner <= rank:
                o2, l2 = _block_attention(qf, kb, vb, scale, tri if (causal and owner == rank) else None)
                out, lse = _merge(out, lse, o2, l2)
            if s + 1 < world:
                kb, vb = _exchange(dist, group, rank, world, [kb, vb])
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.causal, ctx.scale, ctx.group = causal, scale, group
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        import torch.distributed as dist
        q, k, v, out, lse = ctx.saved_tensors
        group, causal, scale = ctx.group, ctx.causal, ctx.scale
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        qf, do = q.float(), dout.float()
        kb, vb = k.float().contiguous(), v.float().contiguous()
        dkb, dvb = torch.zeros_like(kb), torch.zeros_like(vb)
        dq = torch.zeros_like(qf)
        delta = (do * out).sum(-1, keepdim=True)
        T = q.shape[-2]
        tri = torch.ones(T, k.shape[-2], dtype=torch.bool, device=q.device).tril() if causal else None
        safe = torch.where(torch.isfinite(lse), lse, torch.zeros_like(lse)).unsqueeze(-1)
        for s in range(world):
            owner = (rank - s) % world
            if not causal or owner <= rank:
                sc = torch.matmul(qf, kb.transpose(-1, -2)) * scale
                p = torch.exp(sc - safe)
                if causal and owner == rank:
                    p = p.masked_fill(~tri, 0.0)
                dvb = dvb + torch.matmul(p.transpose(-1, -2), do)
                ds = p * (torch.matmul(do, vb.transpose(-1, -2)) - delta)
                dq = dq + torch.matmul(ds, kb) * scale
                dkb = dkb + torch.matmul(ds.transpose(-1, -2), qf) * scale
            # the block moves on with its accumulators; after `world` hops it is home again
            if s + 1 < world:
                kb, vb, dkb, dvb = _exchange(dist, group, rank, world, [kb, vb, dkb, dvb])
            else:
                dkb, dvb = _exchange(dist, group, rank, world, [dkb, dvb])
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True, scale: Optional[float] = None, group=None) -> torch.Tensor:
    """Attention of this rank's query block ``[..., T_local, D]`` over the keys / values of every rank's block.
    Blocks are contiguous and ordered by rank; all ranks hold blocks of the same length.  With one rank (or without an
    initialised process group) this is plain attention."""
    import torch.distributed as dist
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        T = q.shape[-2]
        tri = torch.ones(T, k.shape[-2], dtype=torch.bool, device=q.device).tril() if causal else None
        return _block_attention(q.float(), k.float(), v.float(), scale, tri)[0].to(q.dtype)
    return _RingAttention.apply(q, k, v, causal, scale, group)


def shard_sequence(x: torch.Tensor, dim: int = 1, group=None) -> torch.Tensor:
    """This rank's contiguous block of `x` along `dim` (the layout ring_attention expects)."""
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    assert x.shape[dim] % world == 0, "the sequence length must divide by the number of ranks"
    n = x.shape[dim] // world
    return x.narrow(dim, rank * n, n)
