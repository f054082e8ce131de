#!/usr/bin/env python
"""Device-timed micro-benchmark of the fused peer-memory collectives against their NCCL counterparts.

    torchrun --nproc-per-node N benchmarks/collectives_bench.py [--mb 256] [--iters 10]
    python benchmarks/collectives_bench.py --world1          # one GPU, the peer is the GPU itself (for ncu captures)

Rows (each: CUDA events on the launching stream, max over ranks, median of --iters, buffers larger than L2):
  ddp_allreduce        one kernel: sum of every rank's bf16 bucket slice, x 1/world, written back to every rank
  ddp_allreduce_master the same with the result cast to fp32 master gradients
  nccl_allreduce       torch.distributed.all_reduce(AVG) on the same bucket
  fsdp_rs_adamw        one kernel: gradient reduce-scatter + AdamW on the fp32 master shard + bf16 shard out
  nccl_rs_adamw        reduce_scatter_tensor + the fused multi-tensor AdamW kernel
The roofline of a row is the slower of (bytes that cross NVLink per GPU / 770 GB/s, the measured peer-copy rate) and
(bytes the GPU's own HBM moves / the measured copy bandwidth); the printed fraction is roofline time / measured time.
"""
import argparse
import ctypes as C
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS, HBM_GBS = 770.0, 6537.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=int, default=256, help="bucket size in MB (bf16)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--world1", action="store_true")
    a = ap.parse_args()
    import torch.distributed as dist
    from prometorch_b200 import _native as N
    from prometorch_b200.distributed.ddp import PeerChannel, _ptr_array
    from prometorch_b200.optim import AdamW
    from prometorch_b200.parallel.symm import SymmGroup
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    symm = SymmGroup(dist.group.WORLD, dev)
    lib = N.lib()
    numel = a.mb * (1 << 20) // 2 // (64 * world) * (64 * world)
    ch = PeerChannel(symm, numel * 2)
    bucket = ch.buf.tensor(torch.bfloat16)[:numel]
    master_buf = symm.alloc(numel * 4)
    master_ptrs = _ptr_array([master_buf.peer_ptr(r) for r in range(world)])
    shard = numel // world
    mst, m, v = (torch.zeros(shard, device=dev) for _ in range(3))
    shard_out = torch.zeros(shard, dtype=torch.bfloat16, device=dev)
    st = torch.cuda.current_stream(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        ts = []
        for i in range(a.iters + 3):
            bucket.normal_()
            flush.zero_()                        # L2 holds none of the bucket when the timed call starts
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(st)
            fn()
            e1.record(st)
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if i >= 3:
                ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]

    def ddp_fused():
        N.check(lib.ptb_ddp_allreduce(ch.bufs, ch.flag_ptrs, rank, world, numel, 1, 1.0 / world, ch.next_seq(), ch.ticket.data_ptr(),
                                      ch.status.data_ptr(), 128, st.cuda_stream), "ddp_allreduce")

    def ddp_master():
        N.check(lib.ptb_ddp_allreduce_master(ch.bufs, master_ptrs, ch.flag_ptrs, rank, world, numel, 1.0 / world, ch.next_seq(),
                                             ch.ticket.data_ptr(), ch.status.data_ptr(), 128, st.cuda_stream), "ddp_allreduce_master")

    def nccl_ar():
        dist.all_reduce(bucket, op=dist.ReduceOp.AVG)

    step = [0]

    def rs_fused():
        step[0] += 1
        N.check(lib.ptb_fsdp_rs_adamw(ch.bufs, ch.flag_ptrs, rank, world, numel, mst.data_ptr(), m.data_ptr(), v.data_ptr(),
                                      shard_out.data_ptr(), 3e-4, 0.9, 0.95, 1e-8, 0.1, step[0], 1.0 / world, ch.next_seq(),
                                      ch.ticket.data_ptr(), ch.status.data_ptr(), 128, st.cuda_stream), "fsdp_rs_adamw")

    p32 = torch.nn.Parameter(torch.zeros(shard, device=dev))
    gshard = torch.zeros(shard, dtype=torch.bfloat16, device=dev)
    opt = AdamW([p32], lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    opt.set_grad_source(p32, gshard)
    opt.attach_lowp(p32, shard_out)

    def rs_nccl():
        dist.reduce_scatter_tensor(gshard, bucket, op=dist.ReduceOp.AVG)
        opt.step()

    S = numel * 2                                          # bucket bytes
    f = (world - 1) / world
    rows = [
        # name, fn, NVLink bytes per GPU (read + written), own-HBM bytes per GPU
        ("ddp_allreduce", ddp_fused, 2 * f * S, (S / world) * (1 + 1) + f * S),                 # own slice r+w, peers' writes land here
        ("ddp_allreduce_master", ddp_master, f * S + f * 2 * S, S / world + 2 * S),
        ("nccl_allreduce", nccl_ar, 2 * f * S, 2 * S),
        ("fsdp_rs_adamw", rs_fused, f * S, S / world + shard * (3 * 8 + 2)),
        ("nccl_rs_adamw", rs_nccl, f * S, S + shard * (2 + 3 * 8 + 2 + 2)),
    ]
    out = {"world": world, "bucket_mb": S / 1e6, "rows": []}
    for name, fn, nv, hbm in rows:
        ms = timed(fn)
        roof_ms = max(nv / (NVLINK_GBS * 1e9), hbm / (HBM_GBS * 1e9)) * 1e3
        out["rows"].append({"name": name, "ms": round(ms, 4), "nvlink_gb_per_gpu": round(nv / 1e9, 4), "hbm_gb_per_gpu": round(hbm / 1e9, 4),
                            "nvlink_gbs": round(nv / 1e9 / (ms / 1e3), 1) if nv else 0.0,
                            "roofline_ms": round(roof_ms, 4), "frac_of_roofline": round(roof_ms / ms, 3)})
    ch.check()
    if rank == 0:
        print(json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
