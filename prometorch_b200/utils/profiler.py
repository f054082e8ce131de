"""Section profiler with the reference's interface (``enable, begin/end(name), count_tokens, sample_vram,
print_report``; torch/io/inference_profiler.h:28-230) but without its per-section synchronisation: sections
are bracketed by CUDA events on the caller's stream and resolved once, when the report is requested, so
profiling does not serialise the pipeline it measures.  ``nvtx_range`` marks ranges for external tools."""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch


class Timer:
    def __init__(self):
        self.t0 = time.perf_counter()

    def reset(self):
        self.t0 = time.perf_counter()

    def elapsed_ms(self) -> float:
        return (time.perf_counter() - self.t0) * 1e3


class ScopedTimer:
    def __init__(self, name: str, sink=None):
        self.name, self.sink = name, sink

    def __enter__(self):
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *a):
        ms = (time.perf_counter() - self.t0) * 1e3
        if self.sink is not None:
            self.sink[self.name] = self.sink.get(self.name, 0.0) + ms
        else:
            print(f"[{self.name}] {ms:.3f} ms")


@contextlib.contextmanager
def nvtx_range(name: str):
    use = torch.cuda.is_available()
    if use:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if use:
            torch.cuda.nvtx.range_pop()


class InferenceProfiler:
    def __init__(self):
        self.enabled = False
        self._open: Dict[str, object] = {}
        self._pairs: List[Tuple[str, object, object]] = []
        self._cpu: Dict[str, float] = defaultdict(float)
        self._counts: Dict[str, int] = defaultdict(int)
        self.tokens = 0
        self.vram: List[Tuple[int, int]] = []

    def enable(self, on: bool = True):
        self.enabled = on

    def begin(self, name: str):
        if not self.enabled:
            return
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._open[name] = e
        else:
            self._open[name] = time.perf_counter()

    def end(self, name: str):
        if not self.enabled or name not in self._open:
            return
        s = self._open.pop(name)
        self._counts[name] += 1
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((name, s, e))
        else:
            self._cpu[name] += (time.perf_counter() - s) * 1e3

    def count_tokens(self, n: int = 1):
        self.tokens += n
        if self.enabled and self.tokens % 16 == 0:
            self.sample_vram()

    def sample_vram(self):
        if torch.cuda.is_available():
            self.vram.append((self.tokens, torch.cuda.memory_allocated()))

    def totals(self) -> Dict[str, float]:
        if self._pairs:
            torch.cuda.synchronize()
            for name, s, e in self._pairs:
                self._cpu[name] += s.elapsed_time(e)
            self._pairs = []
        return dict(self._cpu)

    def print_report(self):
        tot = self.totals()
        allms = sum(tot.values()) or 1.0
        print(f"[Profiler] {self.tokens} tokens")
        for k, v in sorted(tot.items(), key=lambda kv: -kv[1]):
            print(f"  {k:28s} {v:10.3f} ms  {100 * v / allms:5.1f}%  x{self._counts[k]}")
