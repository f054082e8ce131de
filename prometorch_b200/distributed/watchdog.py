"""Failure detection on the host: a per-rank heartbeat through the rendezvous store.

Every rank publishes ``hb/<rank> = <counter>`` from a daemon thread; ``check()`` (call it between
steps, before launching collectives) raises :class:`RankFailure` naming ranks whose counter has not
moved for ``timeout`` seconds.  This is the host half of failure detection; the device half is the
bounded flag waits inside the fused kernels, which return a status instead of hanging.  The
reference only has socket/file timeouts that throw (torch/distributed/ddp.cpp:249-261, fsdp.h:149-158)."""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], msg: str):
        super().__init__(msg)
        self.ranks = ranks


class DictStore:
    """In-process stand-in for ``torch.distributed.TCPStore`` (tests)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        with self._lock:
            return self._d[k]

    def check(self, keys):
        with self._lock:
            return all(k in self._d for k in keys)


class Heartbeat:
    def __init__(self, store, rank: int, world_size: int, interval: float = 0.5, timeout: float = 10.0):
        self.store, self.rank, self.world, self.interval, self.timeout = store, rank, world_size, interval, timeout
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}
        self._count = 0

    def start(self):
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def _beat(self):
        self._count += 1
        self.store.set(f"hb/{self.rank}", str(self._count))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._beat()
            except Exception:
                return

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def dead_ranks(self) -> List[int]:
        now = time.time()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                val = self.store.get(f"hb/{r}") if self.store.check([f"hb/{r}"]) else None
            except Exception:
                val = None
            last = self._seen.get(r)
            if val is not None and (last is None or last[0] != val):
                self._seen[r] = (val, now)
            elif last is None:
                self._seen[r] = (None, now)
            if now - self._seen[r][1] > self.timeout:
                dead.append(r)
        return dead

    def check(self):
        dead = self.dead_ranks()
        if dead:
            raise RankFailure(dead, f"rank(s) {dead} sent no heartbeat for {self.timeout}s")
