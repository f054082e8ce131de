"""Process launcher: ``launch(world_size, fn, master_addr, master_port)`` starts ``world_size``
workers with ``MASTER_ADDR / MASTER_PORT / WORLD_SIZE / RANK / LOCAL_RANK`` set, waits for all of
them and returns the worst exit code (128+signal for a killed worker); if one worker fails the
others are terminated.  Same contract as the reference's fork-based launcher
(torch/distributed/launcher.h:101-176); ``parse_dist_args`` reads the same flags (:50-80)."""
from __future__ import annotations

import multiprocessing as mp
import os
import sys
import time
from dataclasses import dataclass
from typing import Callable, List, Optional


@dataclass
class DistArgs:
    rank: int = 0
    world_size: int = 1
    master_addr: str = "127.0.0.1"
    master_port: int = 29500
    nprocs: int = 1


def parse_dist_args(argv: Optional[List[str]] = None) -> DistArgs:
    argv = list(sys.argv[1:] if argv is None else argv)
    a = DistArgs(rank=int(os.environ.get("RANK", 0)), world_size=int(os.environ.get("WORLD_SIZE", 1)),
                 master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"), master_port=int(os.environ.get("MASTER_PORT", 29500)))
    i = 0
    while i < len(argv):
        k = argv[i]
        v = argv[i + 1] if i + 1 < len(argv) else None
        if k == "--rank" and v is not None:
            a.rank = int(v); i += 1
        elif k in ("--world-size", "--world_size") and v is not None:
            a.world_size = int(v); i += 1
        elif k in ("--master-addr", "--master_addr") and v is not None:
            a.master_addr = v; i += 1
        elif k in ("--master-port", "--master_port") and v is not None:
            a.master_port = int(v); i += 1
        elif k == "--nprocs" and v is not None:
            a.nprocs = int(v); i += 1
        i += 1
    return a


def _worker(fn, rank, world, addr, port):
    os.environ.update(MASTER_ADDR=addr, MASTER_PORT=str(port), WORLD_SIZE=str(world), RANK=str(rank), LOCAL_RANK=str(rank))
    rc = fn(rank, world)
    sys.exit(int(rc) if rc else 0)


def launch(world_size: int, worker_fn: Callable[[int, int], Optional[int]], master_addr: str = "127.0.0.1",
           master_port: int = 29500, timeout: Optional[float] = None, start_method: str = "spawn") -> int:
    if world_size <= 1:
        os.environ.update(MASTER_ADDR=master_addr, MASTER_PORT=str(master_port), WORLD_SIZE="1", RANK="0", LOCAL_RANK="0")
        rc = worker_fn(0, 1)
        return int(rc) if rc else 0
    ctx = mp.get_context(start_method)
    procs = [ctx.Process(target=_worker, args=(worker_fn, r, world_size, master_addr, master_port)) for r in range(world_size)]
    for p in procs:
        p.start()
    deadline = None if timeout is None else time.time() + timeout
    worst = 0
    alive = set(range(world_size))
    killed = set()                            # ranks this launcher terminated: their signal codes do not count
    while alive:
        for r in list(alive):
            p = procs[r]
            p.join(timeout=0.05)
            if p.exitcode is None:
                continue
            alive.discard(r)
            code = p.exitcode if p.exitcode >= 0 else 128 - p.exitcode
            if r in killed:
                continue
            worst = max(worst, code)
            if code != 0:                     # a failed rank takes the job down: terminate exactly our children
                for q in alive:
                    procs[q].terminate()
                    killed.add(q)
        if deadline is not None and time.time() > deadline and alive:
            for q in alive:
                procs[q].terminate()
            worst = max(worst, 124)
            for q in alive:
                procs[q].join()
            break
    return worst
