"""A CPU model of the flag protocol of the fused collectives (csrc/collectives.cu), for tests that need a peer to misbehave.

Every rank is a group of threads ("CTAs") over shared Python lists that stand for the symmetric buffers and flag blocks; the
waits are wall-clock bounded and record a status instead of spinning for ever, exactly as the kernels do.  What the model
keeps from the kernels: the entry barrier (CTA 0 of a rank writes its sequence number into word [0][rank] of every peer's
flag block, every CTA waits for all words of its own block), the slice-wise reduction, the exit barrier taken by the last CTA
of a rank (a ticket counts the CTAs), and the failure path: a rank whose entry barrier ran out of time skips its work, still
signals the exit words and resets its ticket, so that the channel works again with the next sequence number.  Fault
injection happens here, on the host: a rank that never launches, a flag write that is withheld, a rank that is late.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

OK, ERR_FLAG_TIMEOUT = 0, 3


@dataclass
class FakeRankMemory:
    """What one rank exposes to its peers: a data buffer and a flag block ``[2 phases][world]``."""
    data: List[float]
    flags: List[List[int]]
    ticket: int = 0
    status: int = OK
    lock: threading.Lock = field(default_factory=threading.Lock)


class FakeSymmChannel:
    def __init__(self, world: int, numel: int, budget_s: float = 0.3):
        self.world, self.numel, self.budget_s = world, numel, budget_s
        self.mem = [FakeRankMemory([0.0] * numel, [[0] * world for _ in range(2)]) for _ in range(world)]
        self.drop: Optional[Callable[[int, int, int, int], bool]] = None      # (writer, target, phase, seq) -> True to withhold the write

    # ------------------------------------------------------------------ the device-side primitives
    def _store_flag(self, writer: int, target: int, phase: int, seq: int):
        if self.drop is not None and self.drop(writer, target, phase, seq):
            return
        self.mem[target].flags[phase][writer] = seq

    def _wait_flag_ge(self, rank: int, phase: int, src: int, seq: int) -> bool:
        t0 = time.monotonic()
        while self.mem[rank].flags[phase][src] < seq:
            if self.mem[rank].status != OK or time.monotonic() - t0 > self.budget_s:
                self.mem[rank].status = ERR_FLAG_TIMEOUT
                return False
            time.sleep(0.0005)
        return True

    def _barrier_in(self, rank: int, cta: int, seq: int) -> bool:
        if cta == 0:
            for p in range(self.world):
                self._store_flag(rank, p, 0, seq)
        return all([self._wait_flag_ge(rank, 0, src, seq) for src in range(self.world)])

    def _barrier_out(self, rank: int, n_ctas: int, seq: int, ok: bool):
        m = self.mem[rank]
        with m.lock:
            m.ticket += 1
            last = m.ticket == n_ctas
        if not last:
            return
        for p in range(self.world):
            self._store_flag(rank, p, 1, seq)
        if ok:
            for src in range(self.world):
                self._wait_flag_ge(rank, 1, src, seq)
        m.ticket = 0

    # ------------------------------------------------------------------ one "kernel launch" of one rank
    def allreduce_rank(self, rank: int, seq: int, n_ctas: int = 2, scale: float = 1.0, delay_s: float = 0.0) -> int:
        """The bucket all-reduce as rank `rank` runs it: returns the rank's status word after the launch."""
        if delay_s:
            time.sleep(delay_s)
        lo, hi = self.numel * rank // self.world, self.numel * (rank + 1) // self.world

        def cta(c):
            ok = self._barrier_in(rank, c, seq)
            if ok:
                for i in range(lo + c, hi, n_ctas):
                    total = sum(self.mem[p].data[i] for p in range(self.world)) * scale
                    for p in range(self.world):
                        self.mem[p].data[i] = total
            self._barrier_out(rank, n_ctas, seq, ok)
        ts = [threading.Thread(target=cta, args=(c,)) for c in range(n_ctas)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return self.mem[rank].status

    def clear_status(self, rank: int):
        self.mem[rank].status = OK

    def run(self, seq: int, values: Dict[int, List[float]], skip=(), delays: Dict[int, float] = None, n_ctas: int = 2, scale: float = 1.0) -> Dict[int, int]:
        """Launch the all-reduce on every rank but those in `skip` (one thread per rank); returns rank -> status."""
        for r, v in values.items():
            self.mem[r].data[:] = list(v)
        out: Dict[int, int] = {}

        def one(r):
            out[r] = self.allreduce_rank(r, seq, n_ctas, scale, (delays or {}).get(r, 0.0))
        ts = [threading.Thread(target=one, args=(r,)) for r in range(self.world) if r not in skip]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return out
