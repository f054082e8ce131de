#!/usr/bin/env python
"""MLP 784-512-256-10 with Adam on CPU, one epoch over an MNIST-shaped synthetic set; optionally as
DistributedDataParallel over two CPU ranks (Gloo on 127.0.0.1).

    python benchmarks/train_mlp_cpu.py [--ddp] [--samples 60000] [--batch 64]

There is no dataset on the box: the inputs are 10 class prototypes plus noise, so the accuracy is a real
training signal (the reference's published figure for this network on MNIST is 97.03 % after two epochs,
BENCH_10MODELS.md:29).  Prints one JSON line with the time of the epoch and the accuracy on held-out samples."""
import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_data(n, seed):
    g = torch.Generator().manual_seed(1234)
    protos = torch.randn(10, 784, generator=g)
    g2 = torch.Generator().manual_seed(seed)
    y = torch.randint(0, 10, (n,), generator=g2)
    x = protos[y] + 7.0 * torch.randn(n, 784, generator=g2)
    return x, y


def worker(rank, world, args=None):
    import prometorch_b200 as pt
    from prometorch_b200 import distributed as D
    from prometorch_b200.models.mlp import MLPClassifier
    from prometorch_b200.optim import Adam
    a = args or _ARGS
    torch.manual_seed(0)
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // max(world, 1)))
    model = MLPClassifier((784, 512, 256, 10))
    if world > 1:
        D.init_process_group("gloo", rank, world, os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), timeout_sec=120)
        model = D.DistributedDataParallel(model)
    opt = Adam(model.parameters(), lr=1e-3)
    x, y = make_data(a["samples"], 1)
    xs, ys = x[rank::world], y[rank::world]
    loss_fn = nn.CrossEntropyLoss()
    bs = a["batch"] // world
    t0 = time.perf_counter()
    for i in range(0, xs.shape[0] - bs + 1, bs):
        model.zero_grad() if world > 1 else opt.zero_grad()
        loss = loss_fn(model(xs[i:i + bs]), ys[i:i + bs])
        loss.backward()
        if world > 1:
            model.finish_gradient_synchronization()
        opt.step()
    dt = time.perf_counter() - t0
    xt, yt = make_data(10000, 2)
    with torch.no_grad():
        acc = float((model(xt).argmax(-1) == yt).float().mean())
    if rank == 0:
        print(json.dumps({"metric": "MLP 784-512-256-10 Adam CPU epoch time", "value": round(dt, 3), "unit": "s", "higher_is_better": False,
                          "accuracy": round(acc, 4), "final_loss": round(float(loss.detach()), 4), "world": world, "samples": a["samples"],
                          "global_batch": a["batch"], "data": "synthetic prototypes + noise (MNIST shape)", "backend": "gloo" if world > 1 else "none"}),
              flush=True)
    if world > 1:
        D.barrier()
        D.destroy_process_group()
    return 0


_ARGS = {"samples": 60000, "batch": 64}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ddp", action="store_true")
    ap.add_argument("--samples", type=int, default=60000)
    ap.add_argument("--batch", type=int, default=64)
    a = ap.parse_args()
    os.environ["PTB_MLP_SAMPLES"], os.environ["PTB_MLP_BATCH"] = str(a.samples), str(a.batch)
    _ARGS.update(samples=a.samples, batch=a.batch)
    if a.ddp:
        from prometorch_b200 import distributed as D
        sys.exit(D.launch(2, _ddp_entry, "127.0.0.1", 29733, timeout=1800))
    worker(0, 1)


def _ddp_entry(rank, world):
    return worker(rank, world, {"samples": int(os.environ.get("PTB_MLP_SAMPLES", 60000)), "batch": int(os.environ.get("PTB_MLP_BATCH", 64))})


if __name__ == "__main__":
    main()
