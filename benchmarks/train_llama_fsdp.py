#!/usr/bin/env python
"""Llama-1.1B-shape FSDP/ZeRO-3 training throughput (tokens/s), 1..8 GPUs of one node.

    torchrun --nproc-per-node N benchmarks/train_llama_fsdp.py [--steps K] [--warmup W] [--impl fused|nccl]

``fused``: parameter all-gather inside the tcgen05 GEMMs, reduce-scatter fused with AdamW
(prometorch_b200.parallel.fsdp_fused).  ``nccl``: the same model under the process-group FSDP
(all-gather / reduce-scatter through NCCL around local GEMMs) — the baseline the fused path is
compared with.  Global batch 64 sequences of 2048 tokens (weak scaling below 8 GPUs keeps 8 sequences
per GPU), bf16 compute, fp32 master weights, AdamW lr 3e-4 with warm-up + cosine."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(impl="fused", steps=5, warmup=3, seqs_per_gpu=8, micro=2, seq_len=2048, model_name="llama-1b", window=0):
    """One measurement inside an initialised process group; returns the result dict on every rank."""
    import torch.distributed as dist
    from prometorch_b200.distributed import TorchProcessGroup
    from prometorch_b200.models.llama import Llama, LlamaConfig
    from prometorch_b200.optim import WarmupCosineAnnealingLR
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    pg = TorchProcessGroup()
    cfg = LlamaConfig.llama_1b() if model_name == "llama-1b" else LlamaConfig.tiny(hidden_size=512, num_heads=8, num_kv_heads=2,
                                                                                 intermediate_size=1408, vocab_size=4096, max_seq=seq_len)
    cfg.max_seq = max(cfg.max_seq, seq_len)
    torch.manual_seed(0)
    model = Llama(cfg).to(dev).to(torch.bfloat16)
    nparams = model.num_parameters()
    sharded = sum(m.weight.numel() for m in model.modules() if isinstance(m, torch.nn.Linear) and m.bias is None and m.weight.numel() >= (1 << 16))
    symm = None
    if impl == "fused":
        from prometorch_b200.parallel.fsdp_fused import FusedFSDP
        from prometorch_b200.parallel.symm import SymmGroup
        symm = SymmGroup(dist.group.WORLD, dev)
        eng = FusedFSDP(model, symm, pg, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, window=window)
        sched = WarmupCosineAnnealingLR(eng, warmup_epochs=100, total_epochs=10000)
    else:
        # the baseline: the same model, the same kernels and the same fused multi-tensor AdamW, with the
        # all-gather and the reduce-scatter done by NCCL around them
        from prometorch_b200.distributed import FullyShardedDataParallel
        from prometorch_b200.optim import AdamW
        eng = FullyShardedDataParallel(model, process_group=pg)
        opt = AdamW(eng.local_shards(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)      # fused multi-tensor kernel (the default on CUDA)
        sched = WarmupCosineAnnealingLR(opt, warmup_epochs=100, total_epochs=10000)
    g = torch.Generator().manual_seed(rank)
    n_micro = seqs_per_gpu // micro
    host = [torch.randint(0, cfg.vocab_size, (micro, seq_len + 1), generator=g).pin_memory() for _ in range(n_micro)]

    def step():
        total = None
        for mb in host:
            tok = mb.to(dev, non_blocking=True)                 # host -> device every step
            loss = eng(tok[:, :-1], tok[:, 1:]) / n_micro
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if impl == "fused":
            eng.step()
            eng.zero_grad()
        else:
            eng.reduce_scatter_grads()
            opt.step()
            opt.zero_grad()
            eng.all_gather_params()
        sched.step()
        return total

    for _ in range(warmup):
        l = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        l = step()
        lv = float(l)                                           # device -> host read of the loss every step
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    t = torch.tensor([e0.elapsed_time(e1), wall * 1e3], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if impl == "fused":
        eng.check()
    tokens = world * seqs_per_gpu * seq_len * steps
    ms = float(t[0])
    flops = 6.0 * nparams * tokens + 12.0 * cfg.num_layers * cfg.hidden_size * seq_len * tokens * 0.5
    tflops = flops / (ms / 1e3) / 1e12 / world
    # bytes this rank moves over NVLink per step: it gathers the (world-1)/world of every sharded bf16 weight it does
    # not own once per micro-batch pass that needs it (forward + backward re-use the staged copy within a step: once),
    # and reads (world-1) peers' slices of the bf16 gradient for its own shard
    nv_bytes = 2.0 * sharded * (world - 1) / world * 2
    out = {"metric": "Llama-1.1B-shape FSDP train tokens/s", "value": round(tokens / (ms / 1e3), 1), "unit": "tok/s",
           "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms / steps, 2),
           "impl": impl, "loss": round(lv, 4), "params": nparams, "dtype": "bf16",
           "model_tflops_per_gpu": round(tflops, 1),
           "nvlink_bytes_per_gpu_per_step": int(nv_bytes),
           "roofline": {"compute_ms": round(flops / steps / world / 1391.1e12 * 1e3, 2),
                        "nvlink_ms": round(nv_bytes / 770e9 * 1e3, 2),
                        "frac_of_roofline": round(max(flops / steps / world / 1391.1e12, nv_bytes / 770e9) / (ms / steps / 1e3), 3)},
           "e2e": {"value": round(tokens / (float(t[1]) / 1e3), 1), "unit": "tok/s",
                   "h2d_bytes_per_step": seqs_per_gpu * (seq_len + 1) * 8, "d2h_bytes_per_step": 4},
           "config": {"model": model_name, "global_batch": world * seqs_per_gpu, "seq_len": seq_len,
                      "parallelism": f"fsdp{world}", "micro_batch": micro}}
    del eng, model, sched
    if impl != "fused":
        del opt
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--micro", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--model", default="llama-1b", choices=["llama-1b", "tiny"])
    ap.add_argument("--window", type=int, default=0, help="ZeRO-3 memory: gathered weights live in this many shared slots (0 = one resident copy per layer)")
    args = ap.parse_args()
    import torch.distributed as dist
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    out = run(args.impl, args.steps, args.warmup, args.seqs_per_gpu, args.micro, args.seq_len, args.model, args.window)
    out["window"] = args.window
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
