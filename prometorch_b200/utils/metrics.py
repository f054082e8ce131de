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

    def close(self):
        if self.f:
            self.f.close()
