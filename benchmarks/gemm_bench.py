#!/usr/bin/env python
"""tcgen05 bf16 GEMM against cuBLAS (torch.matmul) on one GPU.

    python benchmarks/gemm_bench.py [--shapes MxNxK[:tn|nt|nn|tt] ...] [--iters I] [--no-cublas] [--json PATH]

Each shape runs 3 warm-up and I timed launches between CUDA events; operands are cycled through
enough copies to exceed the 126 MB L2, so every launch reads HBM.  Fractions are of the measured
cuBLAS bf16 peak when ``MEASURED_PEAKS.json`` sits at the repository root."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

DEFAULT = ["8192x8192x8192", "4096x4096x4096", "16384x2048x2048", "16384x11264x2048", "16384x2048x5632", "16384x32000x2048",
           "16384x2048x2560:nt", "2560x2048x16384:tt"]


def _peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops", 0)) or None
    except Exception:
        return None


def bench(M, N, K, a_mn, b_mn, iters, cublas=True):
    from prometorch_b200.ops.gemm import check_status, gemm_bf16
    dev = "cuda"
    per_set = 2 * (M * K + N * K + M * N)
    copies = max(1, min(8, (160 << 20) // per_set + 1))
    As = [torch.randn((K, M) if a_mn else (M, K), device=dev).bfloat16() for _ in range(copies)]
    Bs = [torch.randn((K, N) if b_mn else (N, K), device=dev).bfloat16() for _ in range(copies)]
    outs = [torch.empty(M, N, device=dev, dtype=torch.bfloat16) for _ in range(copies)]

    def run(fn):
        for i in range(3):
            fn(i % copies)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(i % copies)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ms = run(lambda i: gemm_bf16(As[i], Bs[i], a_mn=a_mn, b_mn=b_mn, out=outs[i]))
    check_status()
    res = {"M": M, "N": N, "K": K, "a_mn": a_mn, "b_mn": b_mn, "us": round(ms * 1e3, 1), "tflops": round(2 * M * N * K / ms / 1e9, 1)}
    if cublas:
        ms2 = run(lambda i: torch.matmul(As[i].t() if a_mn else As[i], Bs[i] if b_mn else Bs[i].t(), out=outs[i]))
        res.update(cublas_us=round(ms2 * 1e3, 1), cublas_tflops=round(2 * M * N * K / ms2 / 1e9, 1))
    pk = _peak()
    if pk:
        res["frac_of_measured_peak"] = round(res["tflops"] / pk, 3)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="*", default=DEFAULT)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    out = []
    for s in a.shapes:
        dims, _, maj = s.partition(":")
        M, N, K = (int(v) for v in dims.lower().split("x"))
        maj = maj or "nn"
        r = bench(M, N, K, maj[0] == "t", maj[1] == "t", a.iters, not a.no_cublas)
        out.append(r)
        print(json.dumps(r), flush=True)
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
