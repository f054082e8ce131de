#!/usr/bin/env python
"""Llama-2-7B-shape training with tensor parallelism x pipeline parallelism (TP=4 x PP=2 on 8 GPUs by default).

    torchrun --nproc-per-node 8 benchmarks/train_llama7b_tp_pp.py [--tp 4] [--pp 2] [--steps K] [--warmup W] [--impl fused|nccl]

Tensor parallel layers are Megatron-style with sequence parallelism: activations between layers are split by
tokens over the TP ranks, the column-parallel projections gather tokens and the row-parallel ones reduce-scatter
them.  ``fused``: those collectives run inside the tcgen05 GEMMs over NVLink peer memory (all-gather -> GEMM
stages the peers' rows in the same launch; GEMM -> reduce-scatter adds tiles into the owner's buffer from the
epilogue).  ``nccl``: the same layers with NCCL collectives around local GEMMs.  Pipeline stages run the 1F1B
schedule with real autograd per stage and NCCL send/recv between them.  8 micro-batches of one 4096-token
sequence per step, bf16 compute, fp32 master weights, fused AdamW.  Smaller shapes for fewer GPUs:
``--layers --hidden --heads --inter --seq --micros``."""
import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=4)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--inter", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--micros", type=int, default=8)
    a = ap.parse_args()
    import torch.distributed as dist
    from prometorch_b200.distributed import TorchProcessGroup
    from prometorch_b200.nn.fused import FusedCrossEntropyLoss, FusedLinear, FusedRMSNorm
    from prometorch_b200.nn.parallel import ColumnParallelLinear, Pipeline1F1BStage, PipelineScheduleConfig, RowParallelLinear, TPConfig
    from prometorch_b200.ops import fused_ops as K
    from prometorch_b200.ops.attention import flash_attention
    from prometorch_b200.optim import AdamW
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    assert world == a.tp * a.pp, f"world size {world} != tp {a.tp} x pp {a.pp}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29514")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    stage, tp_rank = rank // a.tp, rank % a.tp
    tp_group = pp_group = pp_group_grad = None
    for s in range(a.pp):                                    # every rank creates every group, in the same order
        g = dist.new_group(list(range(s * a.tp, (s + 1) * a.tp)))
        if s == stage:
            tp_group = g
    for r in range(a.tp):                                    # two communicators per pipeline: activations, gradients
        g = dist.new_group([r + s * a.tp for s in range(a.pp)])
        g2 = dist.new_group([r + s * a.tp for s in range(a.pp)])
        if r == tp_rank:
            pp_group, pp_group_grad = g, g2
    symm = None
    if a.impl == "fused" and a.tp > 1:
        from prometorch_b200.parallel.symm import SymmGroup
        symm = SymmGroup(tp_group, dev)
    tp = TPConfig(tp_rank, a.tp, process_group=TorchProcessGroup(tp_group), symm=symm)
    H, heads, d, I, T = a.hidden, a.heads, a.hidden // a.heads, a.inter, a.seq
    hl, T_local = heads // a.tp, T // a.tp
    bf = torch.bfloat16
    inv = 10000.0 ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None]
    cos, sin = ang.cos().float().to(dev), ang.sin().float().to(dev)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            kw = dict(bias=False, init_seed=None, sequence_parallel=True, device=dev, dtype=bf)
            self.attn_norm, self.mlp_norm = FusedRMSNorm(H).to(dev, bf), FusedRMSNorm(H).to(dev, bf)
            self.qkv = ColumnParallelLinear(H, 3 * H, tp, gather_output=False, **kw)
            self.o = RowParallelLinear(H, H, tp, **kw)
            self.gate_up = ColumnParallelLinear(H, 2 * I, tp, gather_output=False, **kw)
            self.down = RowParallelLinear(I, H, tp, **kw)

        def forward(self, x):                                # x: [T_local, H], this rank's tokens
            q, k, v = self.qkv(self.attn_norm(x)).view(1, T, 3, hl, d).unbind(2)
            q, k = K.rope(q, cos, sin, True, 0), K.rope(k, cos, sin, True, 0)
            att = flash_attention(q, k, v, causal=True).reshape(T, hl * d)
            h, x = self.mlp_norm(self.o(att), x)             # residual add fused into the norm
            return self.down(K.swiglu(self.gate_up(h), False), residual=x)     # the add rides in the slot-sum kernel

    class Stage(nn.Module):
        def __init__(self, first, last, n_layers):
            super().__init__()
            self.first, self.last = first, last
            if first:
                self.embed = nn.Embedding(a.vocab, H, device=dev, dtype=bf)
                nn.init.normal_(self.embed.weight, std=0.02)
            self.blocks = nn.ModuleList(Block() for _ in range(n_layers))
            if last:
                self.norm = FusedRMSNorm(H).to(dev, bf)
                self.lm_head = FusedLinear(H, a.vocab, bias=False).to(dev, bf)
                nn.init.normal_(self.lm_head.weight, std=0.02)

        def forward(self, x):
            if self.first:                                   # x: token ids [1, T]; keep this rank's slice of the sequence
                x = self.embed(x.view(-1)[tp_rank * T_local:(tp_rank + 1) * T_local])
            for b in self.blocks:
                x = b(x)
            if self.last:
                x = self.lm_head(self.norm(x))               # logits of the local tokens
            return x

    torch.manual_seed(1234 + rank)
    per = a.layers // a.pp
    model = Stage(stage == 0, stage == a.pp - 1, per)
    nparams_local = sum(p.numel() for p in model.parameters())
    replicated = [p for n, p in model.named_parameters() if "norm" in n or "embed" in n or "lm_head" in n]
    with torch.no_grad():
        for p in replicated:                                 # replicated parameters start equal on the TP ranks
            dist.broadcast(p.data, src=stage * a.tp, group=tp_group)
    params = list(model.parameters())
    for p in params:
        p.grad = torch.zeros_like(p)
    masters = [nn.Parameter(p.detach().float().clone(), requires_grad=False) for p in params]
    opt = AdamW(masters, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    for mp, p in zip(masters, params):
        opt.set_grad_source(mp, p.grad)
        opt.attach_lowp(mp, p.data)
    cfg = PipelineScheduleConfig(num_stages=a.pp, num_micros=a.micros)
    pipe = Pipeline1F1BStage(model, cfg, stage, process_group=TorchProcessGroup(pp_group), act_shape=(T_local, H), act_dtype=bf,
                             grad_process_group=TorchProcessGroup(pp_group_grad))
    xent = FusedCrossEntropyLoss()

    def loss_fn(logits, tgt):                                # mean over all tokens = mean over ranks of local means
        return xent(logits, tgt.view(-1)[tp_rank * T_local:(tp_rank + 1) * T_local]) / a.tp

    g = torch.Generator().manual_seed(7)                     # the same tokens on every rank
    host = torch.randint(0, a.vocab, (a.micros, T + 1), generator=g).pin_memory()

    def step():
        tok = host.to(dev, non_blocking=True)
        for p in params:
            p.grad.zero_()
        loss = pipe.run(tok[:, :-1] if stage == 0 else None, loss_fn=loss_fn if stage == a.pp - 1 else None,
                        targets=tok[:, 1:] if stage == a.pp - 1 else None)
        for p in replicated:
            dist.all_reduce(p.grad, group=tp_group)
        opt.step()
        return loss

    for _ in range(a.warmup):
        l = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    lv = 0.0
    for _ in range(a.steps):
        l = step()
        if l is not None:
            lv = float(l)                                    # device -> host read of the loss on the last stage
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    if symm is not None:
        from prometorch_b200.ops.gemm import check_status
        check_status()
    t = torch.tensor([e0.elapsed_time(e1), wall * 1e3, lv * a.tp if stage == a.pp - 1 else 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    npar = torch.tensor([float(nparams_local)], device=dev, dtype=torch.float64)
    dist.all_reduce(npar)
    if rank == 0:
        tokens = a.micros * T * a.steps
        ms = float(t[0])
        total_params = float(npar)                           # replicated parameters counted once per TP rank
        flops = 6.0 * (a.layers * (4 * H * H + 3 * H * I) + a.vocab * H) * tokens + 12.0 * a.layers * H * T * tokens * 0.5
        print(json.dumps({"metric": "Llama-2-7B-shape TPxPP 1F1B train tokens/s", "value": round(tokens / (ms / 1e3), 1), "unit": "tok/s",
                          "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 2), "impl": a.impl,
                          "loss": round(float(t[2]), 4), "params_all_ranks": int(total_params), "dtype": "bf16", "data": "synthetic",
                          "model_tflops_per_gpu": round(flops / (ms / 1e3) / 1e12 / world, 1),
                          "e2e": {"value": round(tokens / (float(t[1]) / 1e3), 1), "unit": "tok/s",
                                  "h2d_bytes_per_step": a.micros * (T + 1) * 8, "d2h_bytes_per_step": 4},
                          "config": {"model": f"llama {a.layers}L/{H}/{heads}h ffn{I} vocab{a.vocab}", "global_batch": a.micros, "seq_len": T,
                                     "parallelism": f"tp{a.tp}xpp{a.pp}", "micro_batches": a.micros}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
