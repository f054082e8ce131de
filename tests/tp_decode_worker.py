"""Worker for the tensor-parallel decode test: launched by torchrun with one rank per GPU."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])

    def stage(msg):                     # progress on stderr: shows where a run stopped if it has to be killed
        if rank == 0:
            print(f"[tp worker] {msg}", file=sys.stderr, flush=True)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from prometorch_b200.io.config import tiny_qwen3_config
    from prometorch_b200.io.gguf_model import GGUFModel
    from prometorch_b200.io.synthetic import write_synthetic_gguf
    from prometorch_b200.parallel.symm import SymmGroup
    path = sys.argv[1]
    cfg = tiny_qwen3_config(layers=3, hidden=1024, heads=16, kv_heads=8, inter=4096, vocab=2048)
    if rank == 0:
        write_synthetic_gguf(path, cfg, seed=5, device=str(dev), std=0.05)
    dist.barrier()
    symm = SymmGroup(dist.group.WORLD, dev)
    tp = GGUFModel(path, device=str(dev), max_seq=256, tp_rank=rank, tp_world=world, symm=symm)
    ref = GGUFModel(path, device=str(dev), max_seq=256) if rank == 0 else None
    toks = [7, 99, 1500, 3, 2047, 640, 12, 12, 800, 77, 5, 1023]
    ok = True
    stage("models loaded; stepped decode against the 1-GPU engine")
    for pos, t in enumerate(toks):
        nxt = tp.forward_decode(t, pos)
        if rank == 0:
            r = ref.forward_decode(t, pos)
            cos = float(torch.nn.functional.cosine_similarity(tp.hidden_view(), ref.hidden_view(), dim=0))
            if cos < 0.9995:
                ok = False
                print(f"pos {pos}: hidden cosine {cos}", flush=True)
        got = torch.tensor([nxt], device=dev)
        lst = [torch.zeros_like(got) for _ in range(world)]
        dist.all_gather(lst, got)
        if len({int(x) for x in lst}) != 1:
            ok = False
            print(f"pos {pos}: ranks disagree on the token: {[int(x) for x in lst]}", flush=True)
    stage("scripted run")
    # a scripted run must agree across ranks as well
    out = tp.run_script(toks[:4], 16)
    got = torch.tensor(out, device=dev)
    lst = [torch.zeros_like(got) for _ in range(world)]
    dist.all_gather(lst, got)
    if any(not torch.equal(lst[0], x) for x in lst):
        ok = False
        print("scripted tokens differ across ranks", flush=True)
    tp.check_status()
    # batched prompt pass under tensor parallelism (collective): the cache it writes must continue like the stepped one
    stage("batched prefill under tensor parallelism")
    hid_step = None
    for pos, t in enumerate(toks):
        tp.forward_decode(t, pos)
    hid_step = tp.hidden_view().clone()
    if not tp.supports_prefill:
        ok = False
        print("tensor-parallel model reports no batched prefill", flush=True)
    else:
        tp.prefill(toks[:-1])
        tp.forward_decode(toks[-1], len(toks) - 1)
        cos = float(torch.nn.functional.cosine_similarity(tp.hidden_view(), hid_step, dim=0))
        if cos < 0.995:
            ok = False
            print(f"prefill + decode against stepped decode: hidden cosine {cos}", flush=True)
    # the NCCL-only arm (external all-reduce flow) runs the same shards and must land on the same hidden state
    stage("external all-reduce flow (NCCL arm)")
    import ctypes as C
    from benchmarks.decode_tp_nccl import NcclTokenGraph
    from prometorch_b200 import _native as N
    os.environ["PTB_DECODE_FLOW"] = "external"
    ext = GGUFModel(path, device=str(dev), max_seq=256, tp_rank=rank, tp_world=world, symm=symm)
    del os.environ["PTB_DECODE_FLOW"]
    tg = NcclTokenGraph(ext, dist, world)
    tg.capture()
    stage("NCCL token graph captured")
    arr = (C.c_int * len(toks))(*toks)
    N.check(ext._lib.ptb_engine_begin_script(ext._engine, arr, len(toks), 0), "begin_script")
    tg.run(len(toks))
    ext.stream.synchronize()
    ext.check_status()
    cos = float(torch.nn.functional.cosine_similarity(ext.hidden_view(), hid_step, dim=0))
    ids_ext = ext.read_generated(len(toks), 1)
    got = torch.tensor(ids_ext, device=dev)
    lst = [torch.zeros_like(got) for _ in range(world)]
    dist.all_gather(lst, got)
    if cos < 0.9995 or any(not torch.equal(lst[0], x) for x in lst):
        ok = False
        print(f"external all-reduce flow: hidden cosine {cos}, ids {[int(x) for x in lst]}", flush=True)
    stage("NCCL arm checked; teardown")
    tg.release()                                         # the graph holds NCCL kernels: drop it before any teardown
    ext.close()
    dist.barrier()
    symm.check_canaries()                                # the all-reduce slots stayed inside their buffers
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    tp.close()
    if ref is not None:
        ref.close()
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("TP_DECODE_OK" if int(flag) == 1 else "TP_DECODE_FAIL", flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    # no destroy_process_group: this process captured NCCL kernels into a CUDA graph, and tearing the communicator down
    # afterwards has been seen to block
    os._exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
