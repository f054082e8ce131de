#!/usr/bin/env python
"""Character-level GPT (6 layers, d_model 384, 6 heads, context 256, vocab 65: 10.7 M parameters) under
DistributedDataParallel, bf16 compute with fp32 master weights, 1..8 GPUs of one node.

    torchrun --nproc-per-node N benchmarks/train_chargpt_ddp.py [--steps K] [--warmup W] [--impl fused|nccl]

``fused``: gradient buckets live in symmetric memory and each bucket is reduced by ONE peer-memory kernel
(sum in fp32, 1/world scale folded in) launched from the backward hooks.  ``nccl``: the same buckets
all-reduced by NCCL.  64 sequences of 256 tokens per GPU per step (weak scaling), synthetic uniform tokens,
AdamW through the fused multi-tensor kernel.  Every step copies its batch host->device from pinned memory and
reads the loss back."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--batch-per-gpu", type=int, default=64)
    a = ap.parse_args()
    import torch.distributed as dist
    from prometorch_b200.distributed import DistributedDataParallel, TorchProcessGroup
    from prometorch_b200.models.gpt import CharGPT, GPTConfig
    from prometorch_b200.optim import AdamW
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29513")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    pg = TorchProcessGroup()
    cfg = GPTConfig()
    torch.manual_seed(0)
    model = CharGPT(cfg).to(dev).to(torch.bfloat16)
    nparams = sum(p.numel() for p in model.parameters())
    symm = None
    if a.impl == "fused" and world > 1:
        from prometorch_b200.parallel.symm import SymmGroup
        symm = SymmGroup(dist.group.WORLD, dev)
    ddp = DistributedDataParallel(model, pg, symm=symm, bucket_mb=8.0)
    # fp32 masters stepped by the fused AdamW; the bf16 gradients in the buckets are their gradient source
    masters = [torch.nn.Parameter(p.detach().float().clone(), requires_grad=False) for p in model.parameters()]
    opt = AdamW(masters, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    for mp, p in zip(masters, model.parameters()):
        opt.set_grad_source(mp, p.grad)
        opt.attach_lowp(mp, p.data)
    g = torch.Generator().manual_seed(rank)
    B, T = a.batch_per_gpu, cfg.block_size
    host = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=g).pin_memory() for _ in range(4)]

    def step(i):
        tok = host[i % 4].to(dev, non_blocking=True)
        ddp.zero_grad()
        loss = ddp(tok[:, :-1], tok[:, 1:])
        loss.backward()
        ddp.finish_gradient_synchronization()
        opt.step()
        return loss.detach()

    for i in range(a.warmup):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for i in range(a.steps):
        lv = float(step(i))
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ddp.check()
    t = torch.tensor([e0.elapsed_time(e1), wall * 1e3], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        tokens = world * B * T * a.steps
        ms = float(t[0])
        print(json.dumps({"metric": "char-GPT (10.7M) DDP train tokens/s", "value": round(tokens / (ms / 1e3), 1), "unit": "tok/s",
                          "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 3), "impl": a.impl,
                          "loss": round(lv, 4), "params": nparams, "dtype": "bf16", "scaling": "weak", "data": "synthetic",
                          "buckets": len(ddp.buckets),
                          "e2e": {"value": round(tokens / (float(t[1]) / 1e3), 1), "unit": "tok/s", "h2d_bytes_per_step": B * (T + 1) * 8,
                                  "d2h_bytes_per_step": 4},
                          "config": {"model": "char-gpt 6L/384/6h ctx256 vocab65", "global_batch": world * B, "seq_len": T,
                                     "parallelism": f"dp{world}"}}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
