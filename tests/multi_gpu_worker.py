"""Worker for the fused multi-GPU training tests: launched by torchrun, one rank per GPU.

Each case checks a fused compute+collective path against plain torch math on gathered data."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def case_staged_gemm(rank, world, dev, symm, pg):
    """A row-sharded operand staged from the peers inside the GEMM launch, K-major and MN-major."""
    from prometorch_b200.distributed.ddp import PeerChannel
    from prometorch_b200.nn.parallel.fused_tp import gemm_ex, make_staging
    S, K, Nn = 256, 512, 384
    g = torch.Generator(device="cpu").manual_seed(3)
    A_full = (torch.randn(S * world, K, generator=g) * 0.5).to(dev, torch.bfloat16)
    B = (torch.randn(Nn, K, generator=g) * 0.5).to(dev, torch.bfloat16)
    ch = PeerChannel(symm, S * world * K * 2)
    buf = ch.buf.tensor(torch.bfloat16)[:S * world * K].view(S * world, K)
    flags = torch.zeros((S * world + 127) // 128, dtype=torch.int32, device=dev)
    errs = []
    for seq in (1, 2):                                  # a second round must restage, not reuse stale rows
        buf.fill_(float("nan"))
        scale = float(seq)
        buf[rank * S:(rank + 1) * S] = A_full[rank * S:(rank + 1) * S] * scale
        symm.barrier()
        st = make_staging(ch.buf, flags, rank, world, S, S * world, K * 2, seq)
        y = gemm_ex([buf.data_ptr()], 0, K, False, [B.data_ptr()], 0, K, False, S * world, Nn, K, dev, stage_a=st)
        ref = (A_full.float() * scale) @ B.float().t()
        errs.append(_rel(y, ref))
        # the same stored matrix as an MN-major B operand sharded along K: C[M2, K] = X[M2, S*world] @ buf
        X = (torch.randn(128, S * world, generator=g) * 0.5).to(dev, torch.bfloat16)
        flags2 = torch.zeros_like(flags)
        buf2_ch = PeerChannel(symm, S * world * K * 2)
        buf2 = buf2_ch.buf.tensor(torch.bfloat16)[:S * world * K].view(S * world, K)
        buf2.fill_(float("nan"))
        buf2[rank * S:(rank + 1) * S] = A_full[rank * S:(rank + 1) * S]
        symm.barrier()
        st2 = make_staging(buf2_ch.buf, flags2, rank, world, S, S * world, K * 2, 1)
        y2 = gemm_ex([X.data_ptr()], 0, S * world, False, [buf2.data_ptr()], 0, K, True, 128, K, S * world, dev, stage_b=st2)
        errs.append(_rel(y2, X.float() @ A_full.float()))
        symm.barrier()
    assert max(errs) < 1e-2, errs
    return errs


def case_ddp_fused(rank, world, dev, symm, pg):
    """Bucket all-reduce in one peer-memory kernel == NCCL all-reduce of the same gradients."""
    from prometorch_b200.distributed import DistributedDataParallel
    torch.manual_seed(1)
    model = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 512), nn.GELU(), nn.Linear(512, 64)).to(dev)
    ddp = DistributedDataParallel(model, pg, symm=symm, bucket_mb=0.5)
    assert len(ddp.buckets) > 1 and ddp.buckets[0].channel is not None
    torch.manual_seed(100 + rank)
    x = torch.randn(32, 256, device=dev)
    worst = 0.0
    for it in range(3):
        ddp.zero_grad()
        ddp(x).pow(2).mean().backward()
        ddp.finish_gradient_synchronization()
        torch.cuda.synchronize()
        ddp.check()
        got = [p.grad.clone() for p in model.parameters()]
        # reference: local gradients recomputed without DDP, averaged by NCCL
        ref_model = nn.Sequential(*[m for m in model])
        gs = torch.autograd.grad(ref_model(x).pow(2).mean(), list(ref_model.parameters()))
        for a, g in zip(got, gs):
            g = g.clone()
            dist.all_reduce(g)
            g /= world
            worst = max(worst, _rel(a, g))
    assert worst < 1e-5, worst
    return worst


def case_fsdp_fused(rank, world, dev, symm, pg):
    """FusedFSDP on a small Llama tracks a replicated model trained with all-reduced gradients and torch AdamW."""
    import copy
    from prometorch_b200.models.llama import Llama, LlamaConfig
    from prometorch_b200.parallel.fsdp_fused import FusedFSDP
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, intermediate_size=768, vocab_size=1024, num_layers=2, max_seq=256)
    torch.manual_seed(0)
    base = Llama(cfg).to(dev).to(torch.bfloat16)
    ref = copy.deepcopy(base)                            # bf16 replica stepped through fp32 masters
    eng = FusedFSDP(base, symm, pg, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.0, min_shard_numel=1 << 14)
    assert len(eng.sharded) > 0
    masters = [p.detach().float().clone().requires_grad_() for p in ref.parameters()]
    opt = torch.optim.AdamW(masters, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.0)
    g = torch.Generator().manual_seed(50 + rank)
    losses, ref_losses = [], []
    for step in range(4):
        tok = torch.randint(0, cfg.vocab_size, (2, 257), generator=g).to(dev)
        loss = eng(tok[:, :-1], tok[:, 1:])
        loss.backward()
        eng.step()
        eng.zero_grad()
        rl = ref(tok[:, :-1], tok[:, 1:])
        ref.zero_grad()
        rl.backward()
        for p, m in zip(ref.parameters(), masters):
            gr = p.grad.float() if p.grad is not None else torch.zeros_like(m)
            dist.all_reduce(gr)
            m.grad = gr / world
        opt.step()
        with torch.no_grad():
            for p, m in zip(ref.parameters(), masters):
                p.copy_(m)
        losses.append(float(loss))
        ref_losses.append(float(rl))
    torch.cuda.synchronize()
    eng.check()
    assert all(abs(a - b) < 0.05 * abs(b) for a, b in zip(losses, ref_losses)), (losses, ref_losses)
    assert losses[-1] < losses[0]
    # the sharded weights moved the same way as the replica's
    sl = eng.sharded[0]
    w = sl.full_weight().float()
    name = [n for n, m in base.named_modules() if m is sl][0]
    wref = dict(ref.named_modules())[name].weight.detach()
    cos = float(torch.nn.functional.cosine_similarity(w.flatten(), wref.flatten(), dim=0))
    assert cos > 0.999, cos
    return losses, ref_losses, cos


def case_fsdp_window(rank, world, dev, symm, pg):
    """FusedFSDP(window=2): ZeRO-3 memory.  Same losses as the per-layer full copies on the same data (both sum the same
    gradients in fp32), every weight gathered twice per step, per-rank state = 1/world of the model plus the window."""
    import copy
    from prometorch_b200.models.llama import Llama, LlamaConfig
    from prometorch_b200.parallel.fsdp_fused import FusedFSDP
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, intermediate_size=768, vocab_size=1024, num_layers=3, max_seq=256)
    torch.manual_seed(0)
    base = Llama(cfg).to(dev).to(torch.bfloat16)
    twin = copy.deepcopy(base)
    kw = dict(lr=1e-3, betas=(0.9, 0.95), weight_decay=0.05, min_shard_numel=1 << 14)
    full = FusedFSDP(twin, symm, pg, **kw)
    free0 = torch.cuda.mem_get_info(dev)[0]
    win = FusedFSDP(base, symm, pg, window=2, grad_window=2, **kw)
    torch.cuda.synchronize()
    held = free0 - torch.cuda.mem_get_info(dev)[0]
    rep, rep_full = win.memory_report(), full.memory_report()
    n_sharded = sum(sl.S * world * sl.inf for sl in win.sharded)
    largest = max(sl.S * world * sl.inf for sl in win.sharded)
    # 18 bytes per sharded element / world (bf16 shard, fp32 master, two moments, fp32 gradient shard) + 4 layer-sized bf16 slots
    assert rep["sharded_state"] == 18 * n_sharded // world and rep["window"] == 4 * largest * 2 and rep["full_copies"] == 0
    assert rep_full["full_copies"] == 4 * n_sharded and rep_full["sharded_state"] == 12 * n_sharded // world
    # nothing in the window mode grows with the model at fixed world except the 1/world state: at 8 ranks and this model
    # repeated 8 times over it would hold 18 n / 8 + window against 12 n / 8 + 4 n
    deep = 8 * n_sharded
    assert 18 * deep // 8 + rep["window"] < 12 * deep // 8 + 4 * deep
    g = torch.Generator().manual_seed(70 + rank)
    la, lb = [], []
    for step in range(4):
        for micro in range(2):                             # gradient accumulation: the reduce-scatter runs per micro-batch
            tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)
            a = win(tok[:, :-1], tok[:, 1:]) / 2
            a.backward()
            b = full(tok[:, :-1], tok[:, 1:]) / 2
            b.backward()
            la.append(float(a)); lb.append(float(b))
        win.step(); win.zero_grad()
        full.step(); full.zero_grad()
    torch.cuda.synchronize()
    win.check(); full.check()
    assert all(abs(x - y) < 0.02 * abs(y) + 1e-3 for x, y in zip(la, lb)), (la, lb)
    # 3 layers x 7 sharded matrices, gathered for forward and again for backward in every micro-batch
    assert win.pool.gathers >= (2 * len(win.sharded) - 4) * 8, (win.pool.gathers, len(win.sharded))
    wa, wb = win.sharded[0].full_weight().float(), full.sharded[0].full_weight().float()
    cos = float(torch.nn.functional.cosine_similarity(wa.flatten(), wb.flatten(), dim=0))
    assert cos > 0.9999, cos
    return la[-1], lb[-1], cos, held, rep


def case_tp_sp_fused(rank, world, dev, symm, pg):
    """Sequence-parallel column -> row pair with the collectives inside the GEMMs == unsharded layers."""
    from prometorch_b200.nn.parallel import ColumnParallelLinear, RowParallelLinear, TPConfig
    tp = TPConfig(rank, world, process_group=pg, symm=symm)
    tp1 = TPConfig(0, 1)
    n, H, F = 128, 256, 1024
    torch.manual_seed(7)
    x = (torch.randn(n * world, H, device=dev) * 0.5).to(torch.bfloat16)
    col = ColumnParallelLinear(H, F, tp, gather_output=False, bias=False, init_seed=21, sequence_parallel=True).to(dev).to(torch.bfloat16)
    row = RowParallelLinear(F, H, tp, bias=False, init_seed=22, sequence_parallel=True).to(dev).to(torch.bfloat16)
    colf = ColumnParallelLinear(H, F, tp1, bias=False, init_seed=21).to(dev).float()
    rowf = RowParallelLinear(F, H, tp1, bias=False, init_seed=22).to(dev).float()
    xf = x.float().clone().requires_grad_()
    yf = torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(xf, colf.weight)), rowf.weight)
    yf.pow(2).mean().backward()
    res = []
    for it in range(2):                                  # twice: buffers, flags and sequence numbers are reused
        xl = x[rank * n:(rank + 1) * n].clone().requires_grad_()
        col.weight.grad = row.weight.grad = None
        y = row(torch.relu(col(xl)))
        (y.float().pow(2).sum() / yf.numel()).backward()
        s = col.shard
        res = [_rel(y, yf[rank * n:(rank + 1) * n]), _rel(xl.grad, xf.grad[rank * n:(rank + 1) * n]),
               _rel(col.weight.grad, colf.weight.grad[rank * s:(rank + 1) * s]),
               _rel(row.weight.grad, rowf.weight.grad[:, rank * row.shard:(rank + 1) * row.shard])]
        assert max(res) < 3e-2, (it, res)
    # the residual rides in the kernel that sums the ranks' partial tiles, and gets the output's gradient
    xl = x[rank * n:(rank + 1) * n].clone()
    resid = (torch.randn(n, H, device=dev) * 0.3).to(torch.bfloat16).requires_grad_()
    with torch.no_grad():
        plain = row(torch.relu(col(xl)))
    y = row(torch.relu(col(xl)), residual=resid)
    assert _rel(y, plain.float() + resid.float()) < 1e-2
    y.float().sum().backward()
    assert torch.allclose(resid.grad.float(), torch.ones_like(resid.grad.float()))
    return res


def case_fsdp_checkpoint(rank, world, dev, symm, pg):
    """Fused FSDP: 2 steps, save, 2 more steps == a fresh engine that loads the checkpoint and takes the same 2 steps."""
    import copy
    import tempfile
    from prometorch_b200.models.llama import Llama, LlamaConfig
    from prometorch_b200.parallel.fsdp_fused import FusedFSDP
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, intermediate_size=768, vocab_size=1024, num_layers=2, max_seq=256)
    torch.manual_seed(0)
    base = Llama(cfg).to(dev).to(torch.bfloat16)
    fresh = copy.deepcopy(base)
    box = [tempfile.mkdtemp(prefix="ptb_ckpt_") if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    d = box[0]
    g = torch.Generator().manual_seed(70 + rank)
    toks = [torch.randint(0, cfg.vocab_size, (2, 257), generator=g).to(dev) for _ in range(4)]

    def run(eng, batch):
        out = []
        for tok in batch:
            loss = eng(tok[:, :-1], tok[:, 1:])
            loss.backward()
            eng.step()
            eng.zero_grad()
            out.append(float(loss))
        return out
    a = FusedFSDP(base, symm, pg, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.0, min_shard_numel=1 << 14)
    run(a, toks[:2])
    a.save_sharded(d, extra={"step": 2})
    la = run(a, toks[2:])
    b = FusedFSDP(fresh, symm, pg, lr=5e-4, betas=(0.9, 0.95), weight_decay=0.0, min_shard_numel=1 << 14)
    extra = b.load_sharded(d)
    assert extra == {"step": 2} and b.param_groups[0]["lr"] == 1e-3 and b.sharded[0].step_count == 2
    lb = run(b, toks[2:])
    torch.cuda.synchronize()
    a.check()
    b.check()
    assert all(abs(x - y) < 2e-3 * abs(x) for x, y in zip(la, lb)), (la, lb)
    for sa, sb in zip(a.sharded, b.sharded):
        assert _rel(sb.master, sa.master) < 1e-4 and _rel(sb.full_weight(), sa.full_weight()) < 1e-3
    for pa, pb in zip(a.rest, b.rest):
        assert _rel(pb, pa) < 1e-3
    return la, lb


CASES = dict(fsdp_checkpoint=case_fsdp_checkpoint, staged_gemm=case_staged_gemm, ddp_fused=case_ddp_fused, fsdp_fused=case_fsdp_fused, fsdp_window=case_fsdp_window,
             tp_sp_fused=case_tp_sp_fused)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from prometorch_b200.distributed import TorchProcessGroup
    from prometorch_b200.parallel.symm import SymmGroup
    symm = SymmGroup(dist.group.WORLD, dev)
    pg = TorchProcessGroup()
    names = sys.argv[1:] or list(CASES)
    ok = True
    for nme in names:
        out = None
        try:
            out = CASES[nme](rank, world, dev, symm, pg)
            torch.cuda.synchronize()
        except Exception as e:                           # report and keep the other ranks out of a hang
            import traceback
            traceback.print_exc()
            print(f"[{nme}] rank {rank} FAILED: {e}", flush=True)
            ok = False
        # every rank takes the same collectives from here on, whether its case passed or not
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(int(flag))
        if not ok:
            break
        dist.barrier()
        symm.check_canaries()                            # nobody wrote outside a symmetric buffer
        if rank == 0:
            print(f"[{nme}] ok {out}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and ok:
        print("MULTI_GPU_OK", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
