"""Multi-tensor optimizer kernels: achieved HBM bandwidth of one fused step over a set of parameters.

    python benchmarks/optim_bench.py [--tensors 64] [--numel 1048576] [--kinds AdamW,SGD,Lion,LAMB] [--grad bf16|fp32]

A step of the fused path is one launch for all tensors (three for LAMB).  Bytes per element are counted from what the rule
must touch: the fp32 parameter read and written, every fp32 state tensor read and written, the gradient read once.  Timed
with CUDA events over `--iters` steps after warm-up, with an L2 flush (a 256 MB fill) between steps; prints one JSON line per
optimizer with the fraction of the measured copy bandwidth (6537 GB/s on this pool's B200s unless MEASURED_PEAKS.json says
otherwise).  The tensor-op form of the same rule (`fused=False`) is timed beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# fp32 state tensors each rule keeps per parameter (read + written every step)
STATE_TENSORS = {"SGD": 1, "Adam": 2, "AdamW": 2, "Lion": 1, "RMSprop": 1, "Adagrad": 1, "NAdam": 2, "RAdam": 2, "Adamax": 2, "LAMB": 2, "SophiaG": 2}
KWARGS = {"SGD": dict(lr=0.1, momentum=0.9), "LAMB": dict(lr=1e-3, weight_decay=0.01)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tensors", type=int, default=64)
    ap.add_argument("--numel", type=int, default=1 << 20)
    ap.add_argument("--kinds", default="AdamW,SGD,Lion,LAMB")
    ap.add_argument("--grad", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-unfused", action="store_true")
    a = ap.parse_args()
    import torch
    from prometorch_b200 import optim as O
    peak = 6537.0
    try:
        peak = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))["hbm_gbs"])
    except Exception:                                      # noqa: BLE001
        pass
    dev = torch.device("cuda")
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    gdt = torch.bfloat16 if a.grad == "bf16" else torch.float32

    def timed(opt, params):
        for p in params:
            g = torch.randn(p.shape, device=dev).to(gdt)
            if gdt == torch.float32:
                p.grad = g
            else:
                opt.set_grad_source(p, g)
        for _ in range(3):
            opt.step()
        ms = []
        for _ in range(a.iters):
            flush.fill_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            opt.step()
            e1.record()
            torch.cuda.synchronize()
            ms.append(e0.elapsed_time(e1))
        ms.sort()
        return ms[len(ms) // 2]

    for kind in a.kinds.split(","):
        cls = getattr(O, kind)
        kw = KWARGS.get(kind, dict(lr=1e-3))
        n_el = a.tensors * a.numel
        bytes_per_el = 8 + 8 * STATE_TENSORS.get(kind, 2) + (2 if gdt == torch.bfloat16 else 4)
        out = {"bench": "optim", "kind": kind, "tensors": a.tensors, "numel_each": a.numel, "grad": a.grad, "bytes_per_element": bytes_per_el}
        params = [torch.nn.Parameter(torch.randn(a.numel, device=dev)) for _ in range(a.tensors)]
        ms = timed(cls(params, fused=True, **kw), params)
        out.update(fused_ms=round(ms, 4), fused_gbs=round(n_el * bytes_per_el / ms / 1e6, 1), frac_of_measured_hbm=round(n_el * bytes_per_el / ms / 1e6 / peak, 3))
        if not a.no_unfused and gdt == torch.float32:
            params2 = [torch.nn.Parameter(torch.randn(a.numel, device=dev)) for _ in range(a.tensors)]
            ms2 = timed(cls(params2, fused=False, **kw), params2)
            out.update(tensor_ops_ms=round(ms2, 4), speedup=round(ms2 / ms, 2))
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
