#!/usr/bin/env python
"""FlashAttention forward/backward timings on one GPU: tcgen05 forward against the mma.sync forward, and backward.

    python benchmarks/attention_bench.py [--iters 10]

Shapes of the training configs: Llama-1.1B (B 2, T 2048, 32 q / 4 kv heads of 64) and Llama-2-7B (B 1, T 4096, 32 heads of
128).  Causal.  FLOP count: 4 * B * H * T^2 * D / 2 for the forward, 2.5x that for the backward."""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--shapes", nargs="*", default=["llama-1b", "llama-7b", "long"])
    ap.add_argument("--tcgen05-fwd-only", action="store_true", help="time only the tcgen05 forward (profiling runs)")
    a = ap.parse_args()
    from prometorch_b200.ops.attention import flash_attention
    from prometorch_b200.ops.gemm import check_status
    all_shapes = {"llama-1b": (2, 2048, 32, 4, 64), "llama-7b": (1, 4096, 32, 32, 128), "long": (1, 16384, 8, 8, 128)}
    for name in a.shapes:
        B, T, H, Hk, D = all_shapes[name]
        q = torch.randn(B, T, H, D, device="cuda").bfloat16().requires_grad_()
        k = torch.randn(B, T, Hk, D, device="cuda").bfloat16().requires_grad_()
        v = torch.randn(B, T, Hk, D, device="cuda").bfloat16().requires_grad_()
        flops = 4.0 * B * H * T * T * D / 2
        res = {"shape": name, "B": B, "T": T, "H": H, "Hk": Hk, "D": D}
        for impl in (("1",) if a.tcgen05_fwd_only else ("1", "0")):
            os.environ["PTB_FA_SM100"] = impl
            with torch.no_grad():
                ms = timeit(lambda: flash_attention(q, k, v, causal=True), a.iters)
            res["fwd_tcgen05" if impl == "1" else "fwd_mma_sync"] = {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1)}
        os.environ["PTB_FA_SM100"] = "1"
        if a.tcgen05_fwd_only:
            check_status()
            print(json.dumps(res), flush=True)
            continue
        o = flash_attention(q, k, v, causal=True)
        do = torch.randn_like(o)
        for impl in ("1", "0"):
            os.environ["PTB_FA_BWD_SM100"] = impl
            ms = timeit(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True), a.iters)
            res["bwd_tcgen05" if impl == "1" else "bwd_mma_sync"] = {"us": round(ms * 1e3, 1), "tflops": round(2.5 * flops / ms / 1e9, 1)}
        os.environ["PTB_FA_BWD_SM100"] = "1"
        check_status()
        print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
