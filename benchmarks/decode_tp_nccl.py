"""Tensor-parallel GGUF decode: the in-kernel exchange against an NCCL-only arm.

Both arms run the same shards, the same GEMV / attention kernels and one CUDA graph per token; they differ only in
how the partial sums of the K-split projections (attention output, FFN down: two per layer) and the arg-max of the
vocabulary shards meet:

* ``fused``: the package's default flow, the exchange inside the GEMV kernels over NVLink peer memory
  (``EPI_ALLREDUCE`` / ``EPI_PARTIAL`` epilogues, csrc/decode_kernels.cuh);
* ``nccl``: the engine's "external" flow: no kernel touches a peer; after each K-split projection the residual vector
  is all-reduced in place by ``ncclAllReduce`` (rank 0 has added the residual to its partial sums), and the
  {id, value} pairs of the lm_head are all-gathered and finished by a one-thread kernel.  73 collectives per token,
  the shape of the reference's tensor-parallel decode (torch/io/gguf_model.h:6225,6442,6512).

Run:  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
          benchmarks/decode_tp_nccl.py --steps 64 --warmup 8
Prints one JSON line (device-timed with CUDA events on the engine stream, max over ranks).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class NcclTokenGraph:
    """One token of the external flow, captured once: engine launch ranges with NCCL collectives between them."""

    def __init__(self, model, dist, world):
        import torch
        self.m, self.dist, self.world = model, dist, world
        lib, eng = model._lib, model._engine
        self.x = model._wrap(lib.ptb_engine_buffer(eng, 0), model.cfg.hidden_size)
        self.pair = model._wrap(lib.ptb_engine_buffer(eng, 1), 2, torch.int32)
        self.pairs = torch.zeros(2 * world, dtype=torch.int32, device=model.device)
        self.graph = None

    def enqueue(self):
        from prometorch_b200 import _native as N
        lib, eng, dist = self.m._lib, self.m._engine, self.dist
        first = 0
        for l in range(self.m.cfg.num_layers):
            o, down = 3 + 5 * l, 5 + 5 * l                 # launch numbers of this layer's K-split projections
            N.check(lib.ptb_engine_enqueue_range(eng, first, o + 1 - first), "enqueue")
            dist.all_reduce(self.x)
            N.check(lib.ptb_engine_enqueue_range(eng, o + 1, down - o), "enqueue")
            dist.all_reduce(self.x)
            first = down + 1
        N.check(lib.ptb_engine_enqueue_range(eng, first, 1), "enqueue")          # lm_head with this shard's arg-max
        dist.all_gather_into_tensor(self.pairs, self.pair)
        N.check(lib.ptb_engine_finish_token(eng, self.pairs.data_ptr(), self.world), "finish_token")

    def capture(self):
        import torch
        s = self.m.stream
        with torch.cuda.stream(s):
            for _ in range(2):                              # NCCL sets its channels up on first use
                self.enqueue()
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s, capture_error_mode="thread_local"):
            self.enqueue()
        self.graph = g

    def run(self, n):
        import torch
        with torch.cuda.stream(self.m.stream):
            for _ in range(n):
                self.graph.replay()

    def release(self):
        """Drop the captured graph.  It holds NCCL kernels: the communicator must not be torn down while it exists
        (destroying the process group first blocks forever)."""
        import gc
        import torch
        self.m.stream.synchronize()
        self.graph = None
        gc.collect()
        torch.cuda.synchronize()


def timed(model, run, dist, dev, prompt, warmup, steps, repeats):
    """tok/s of `steps` decode steps after the prompt and `warmup` more, median of `repeats` regions, max over ranks."""
    import torch
    lib, eng = model._lib, model._engine
    from prometorch_b200 import _native as N
    n = len(prompt)
    arr = (C.c_int * n)(*prompt)
    N.check(lib.ptb_engine_begin_script(eng, arr, n, 0), "begin_script")
    run(n - 1 + warmup)
    s = model.stream
    ms = []
    for _ in range(repeats):
        dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        run(steps)
        e1.record(s)
        s.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms.append(float(t))
    model.check_status()
    ids = model.read_generated(n, warmup + repeats * steps)
    ms.sort()
    return steps / (ms[len(ms) // 2] / 1e3), ids


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--model", default="qwen3-4b", choices=["qwen3-4b", "tiny"])
    ap.add_argument("--impl", default="both", choices=["both", "fused", "nccl"])
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    import bench as B
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.parallel.symm import SymmGroup
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("launch under torch.distributed.run with at least 2 ranks")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    symm = SymmGroup(dist.group.WORLD, dev)
    if rank == 0:
        B.ensure_gguf(args.model, str(dev))
    dist.barrier()
    path, cfg = B.ensure_gguf(args.model, str(dev))
    prompt = B.bench_prompt(cfg.vocab_size, args.prompt_len)
    max_seq = args.prompt_len + args.warmup + args.repeats * args.steps + 16
    out = {"bench": "decode_tp_nccl", "model": args.model, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
           "repeats": args.repeats, "collectives_per_token_nccl": 2 * cfg.num_layers + 1}
    ids = {}
    if args.impl in ("both", "fused"):
        m = GGUFModel(path, device=str(dev), max_seq=max_seq, tp_rank=rank, tp_world=world, symm=symm)
        m.capture()
        lib, eng = m._lib, m._engine

        def run_fused(n):
            from prometorch_b200 import _native as N
            N.check(lib.ptb_engine_run(eng, n), "run")
        out["fused_tok_s"], ids["fused"] = timed(m, run_fused, dist, dev, prompt, args.warmup, args.steps, args.repeats)
        out["fused_tok_s"] = round(out["fused_tok_s"], 1)
        m.close()
    if args.impl in ("both", "nccl"):
        old = os.environ.get("PTB_DECODE_FLOW")
        os.environ["PTB_DECODE_FLOW"] = "external"
        try:
            m = GGUFModel(path, device=str(dev), max_seq=max_seq, tp_rank=rank, tp_world=world, symm=symm)
        finally:
            if old is None:
                del os.environ["PTB_DECODE_FLOW"]
            else:
                os.environ["PTB_DECODE_FLOW"] = old
        tg = NcclTokenGraph(m, dist, world)
        tg.capture()
        out["nccl_tok_s"], ids["nccl"] = timed(m, tg.run, dist, dev, prompt, args.warmup, args.steps, args.repeats)
        out["nccl_tok_s"] = round(out["nccl_tok_s"], 1)
        tg.release()
        m.close()
    if len(ids) == 2:
        a, b = ids["fused"], ids["nccl"]
        same = 0
        while same < min(len(a), len(b)) and a[same] == b[same]:
            same += 1
        # the arms sum the partials in different orders, so near-tied logits of a random-weight model may split later on
        out["ids_equal_prefix"] = same
        out["first_id_equal"] = bool(a[0] == b[0])
        out["fused_over_nccl"] = round(out["fused_tok_s"] / out["nccl_tok_s"], 3)
    if rank == 0:
        print(json.dumps(out), flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    # leave without tearing the communicator down: a process that captured NCCL kernels into a graph has been seen to block
    # in the teardown even after the graph was released
    os._exit(0)


if __name__ == "__main__":
    main()
