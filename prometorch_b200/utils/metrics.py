"""Structured metrics: one JSON object per line (step time, tokens/s, bytes moved per collective and the
achieved fraction of a roofline).  The reference only prints tagged lines to stdout."""
from __future__ import annotations

import json
import time
from typing import Optional


class MetricsWriter:
    def __init__(self, path: Optional[str] = None, also_print: bool = False):
        self.f = open(path, "a") if path else None
        self.also_print = also_print

    def log(self, **kv):
        kv.setdefault("ts", time.time())
        line = json.dumps(kv, default=float)
        if self.f:
            self.f.write(line + "\n")
            self.f.flush()
        if self.also_print or not self.f:
            print(line)

    def roofline(self, name: str, seconds: float, flops: float = 0.0, bytes_moved: float = 0.0, peak_flops: float = 1.6263e15,
                 peak_bw: float = 6.537e12, **extra):
        """Log achieved/peak for a kernel: the bound is the slower of compute at peak and bytes at bandwidth."""
        bound = max(flops / peak_flops if flops else 0.0, bytes_moved / peak_bw if bytes_moved else 0.0)
        self.log(kind="roofline", name=name, seconds=seconds, flops=flops, bytes=bytes_moved,
                 fraction=(bound / seconds if seconds > 0 else 0.0), **extra)

    def collective(self, name: str, seconds: float, payload_bytes: float, world: int, kind: str = "all_reduce",
                   flops: float = 0.0, link_bw: float = 770e9, peak_flops: float = 1.391e15, **extra):
        """Log one collective (or a fused compute+collective kernel): bytes each GPU must send over NVLink for a payload of
        ``payload_bytes`` per rank, the achieved per-direction GB/s, NCCL's bus bandwidth convention, and the achieved
        fraction of max(bytes / link bandwidth, FLOPs / peak).  ``link_bw`` defaults to the measured 770 GB/s per
        direction per GPU."""
        wire = wire_bytes(kind, payload_bytes, world)
        bound = max(wire / link_bw if wire else 0.0, flops / peak_flops if flops else 0.0)
        rec = dict(kind="collective", name=name, op=kind, world=world, seconds=seconds, payload_bytes=payload_bytes,
                   wire_bytes_per_gpu=wire, gbps_per_direction=(wire / seconds / 1e9 if seconds > 0 else 0.0),
                   busbw_gbps=(bus_bandwidth(kind, payload_bytes, world, seconds) / 1e9 if seconds > 0 else 0.0),
                   roofline_seconds=bound, fraction=(bound / seconds if seconds > 0 else 0.0), flops=flops, **extra)
        self.log(**rec)
        return rec

    def close(self):
        if self.f:
            self.f.close()


def wire_bytes(kind: str, payload_bytes: float, world: int) -> float:
    """Bytes one GPU sends (= receives) for a collective over ``world`` ranks with all-to-all connectivity.
    ``payload_bytes``: the full vector for all_reduce / reduce_scatter / all_gather (result size for all_gather), the
    local send buffer for all_to_all, the message for broadcast / send."""
    w = max(int(world), 1)
    if w == 1:
        return 0.0
    if kind == "all_reduce":
        return 2.0 * payload_bytes * (w - 1) / w          # reduce-scatter + all-gather
    if kind in ("reduce_scatter", "all_gather", "all_to_all"):
        return payload_bytes * (w - 1) / w
    if kind in ("broadcast", "send", "p2p"):
        return float(payload_bytes)
    raise ValueError(f"unknown collective {kind!r}")


def bus_bandwidth(kind: str, payload_bytes: float, world: int, seconds: float) -> float:
    """NCCL-tests' bus bandwidth: algorithm bandwidth times 2(n-1)/n for all_reduce, (n-1)/n for the one-phase ones."""
    return wire_bytes(kind, payload_bytes, world) / seconds if seconds > 0 else 0.0


def measured_peaks(path: Optional[str] = None) -> dict:
    """``{hbm_bw, flops_burst, flops_sustained}`` from a MEASURED_PEAKS.json written by a calibration run (searched beside
    the package when ``path`` is None); the defaults are an earlier measurement on B200."""
    import os
    out = {"hbm_bw": 6.537e12, "flops_burst": 1.6263e15, "flops_sustained": 1.391e15}
    cand = [path] if path else [os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                             "MEASURED_PEAKS.json")]
    for p in cand:
        if p and os.path.exists(p):
            try:
                d = json.load(open(p))
            except (OSError, ValueError):
                continue
            if "hbm_gbs" in d:
                out["hbm_bw"] = float(d["hbm_gbs"]) * 1e9
            if "bf16_tflops" in d:
                out["flops_burst"] = float(d["bf16_tflops"]) * 1e12
            if "bf16_tflops_sustained" in d:
                out["flops_sustained"] = float(d["bf16_tflops_sustained"]) * 1e12
    return out


class CollectiveTimer:
    """CUDA-event timer around a collective on the current stream; ``stop()`` synchronises and returns seconds."""

    def __init__(self, stream=None):
        import torch
        self.stream = stream if stream is not None else torch.cuda.current_stream()
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def start(self):
        self.e0.record(self.stream)
        return self

    def stop(self) -> float:
        self.e1.record(self.stream)
        self.e1.synchronize()
        return self.e0.elapsed_time(self.e1) / 1e3
