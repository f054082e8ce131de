"""Worker bodies for the multi-rank CPU tests.  Each takes ``(rank, world)`` and returns an exit code; they run
as spawned processes over the Gloo backend on 127.0.0.1."""
from __future__ import annotations

import os
import sys

import torch
import torch.nn as nn


def _init(rank, world):
    from .. import distributed as D
    return D.init_process_group("gloo", rank, world, os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), timeout_sec=60)


def _fin():
    from .. import distributed as D
    D.barrier()
    D.destroy_process_group()


def collectives(rank, world):
    from .. import distributed as D
    _init(rank, world)
    t = torch.full((4,), float(rank + 1))
    D.all_reduce(t)
    assert torch.allclose(t, torch.full((4,), float(sum(range(1, world + 1))))), t
    t = torch.full((3,), float(rank))
    D.all_reduce(t, D.ReduceOp.AVG)
    assert torch.allclose(t, torch.full((3,), (world - 1) / 2)), t
    b = torch.arange(5.0) if rank == 0 else torch.zeros(5)
    D.broadcast(b, 0)
    assert torch.equal(b, torch.arange(5.0))
    parts = [torch.zeros(2) for _ in range(world)]
    D.all_gather(parts, torch.full((2,), float(rank)))
    assert all(float(p[0]) == i for i, p in enumerate(parts))
    buf = torch.zeros(world * 3)
    buf.view(world, 3)[rank] = float(rank + 1)
    D.all_gather_inplace(buf)
    assert torch.equal(buf.view(world, 3)[:, 0], torch.arange(1.0, world + 1)), buf
    buf2 = torch.zeros(world * 2)
    buf2.view(world, 2)[rank] = float(10 + rank)
    assert torch.equal(D.all_gather_wait(D.all_gather_post(buf2)).view(world, 2)[:, 1], torch.arange(10.0, 10 + world))
    out = torch.zeros(2)
    D.reduce_scatter(out, [torch.full((2,), float(k + rank)) for k in range(world)])
    assert torch.allclose(out, torch.full((2,), float(sum(rank + r for r in range(world)))))
    _fin()
    return 0


def _mlp(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 32), nn.ReLU(), nn.Linear(32, 4))


def ddp_matches_single(rank, world):
    """DDP over `world` ranks on disjoint halves of a batch == one process on the whole batch; no_sync accumulation too."""
    from .. import distributed as D
    from ..optim import SGD
    _init(rank, world)
    torch.manual_seed(123)
    X, Y = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    ref = _mlp(1)
    model = _mlp(1 + rank)                      # different init per rank: the constructor must broadcast rank 0's
    ddp = D.DistributedDataParallel(model, bucket_mb=0.002)
    assert len(ddp.buckets) > 1
    ro, do = SGD(ref.parameters(), lr=0.1), SGD(model.parameters(), lr=0.1)
    for step in range(3):
        ro.zero_grad()
        ((ref(X) - Y) ** 2).mean().backward()
        ro.step()
        ddp.zero_grad()
        xs, ys = X[rank::world], Y[rank::world]
        if step == 1:                            # two micro-batches, the first under no_sync
            h = xs.shape[0] // 2
            with ddp.no_sync():
                (((ddp(xs[:h]) - ys[:h]) ** 2).mean() / 2).backward()
            (((ddp(xs[h:]) - ys[h:]) ** 2).mean() / 2).backward()
        else:
            ((ddp(xs) - ys) ** 2).mean().backward()
        ddp.finish_gradient_synchronization()
        do.step()
        for a, b in zip(ref.parameters(), model.parameters()):
            assert torch.allclose(a, b, atol=1e-5), (step, (a - b).abs().max())
    _fin()
    return 0


def fsdp_matches_unsharded(rank, world):
    from .. import distributed as D
    from ..optim import SGD
    _init(rank, world)
    torch.manual_seed(7)
    X, Y = torch.randn(4 * world, 16), torch.randn(4 * world, 4)
    ref, model = _mlp(3), _mlp(3)
    for strategy in (D.ShardingStrategy.FULL_SHARD, D.ShardingStrategy.SHARD_GRAD_OP):
        ref, model = _mlp(3), _mlp(3)
        fsdp = D.FullyShardedDataParallel(model, D.FSDPConfig(rank=rank, world_size=world, strategy=strategy))
        ro, so = SGD(ref.parameters(), lr=0.1), D.ZeROOptimizer(fsdp.local_shards(), SGD(fsdp.local_shards(), lr=0.1), stage=3)
        for step in range(2):
            ro.zero_grad()
            ((ref(X) - Y) ** 2).mean().backward()
            ro.step()
            fsdp.all_gather_params()
            ((fsdp(X[rank::world]) - Y[rank::world]) ** 2).mean().backward()
            fsdp.reduce_scatter_grads()
            so.step()
            so.zero_grad()
        fsdp.all_gather_params()
        for a, b in zip(ref.parameters(), model.parameters()):
            assert (a - b).abs().max() < 1e-4, (strategy, (a - b).abs().max())
        sd = fsdp.shard_state_dict()
        fsdp.load_shard_state_dict(sd)
    _fin()
    return 0


def tp_matches_unsharded(rank, world):
    from .. import distributed as D
    from ..nn.parallel import ColumnParallelLinear, RowParallelLinear, TPConfig
    pg = _init(rank, world)
    tp = TPConfig(rank, world, process_group=pg)
    tp1 = TPConfig(0, 1)
    torch.manual_seed(5)
    x = torch.randn(6, 16)
    for sp in (False, True):
        col, row = ColumnParallelLinear(16, 32, tp, gather_output=False, init_seed=11, sequence_parallel=sp), \
            RowParallelLinear(32, 8, tp, init_seed=12, sequence_parallel=sp)
        colf, rowf = ColumnParallelLinear(16, 32, tp1, init_seed=11), RowParallelLinear(32, 8, tp1, init_seed=12)
        xf = x.clone().requires_grad_()
        yf = rowf(torch.relu(colf(xf)))
        yf.pow(2).sum().backward()
        if sp:
            n = x.shape[0] // world
            xl = x[rank * n:(rank + 1) * n].clone().requires_grad_()
            y = row(torch.relu(col(xl)))
            assert torch.allclose(y, yf[rank * n:(rank + 1) * n], atol=1e-5), (y - yf[rank * n:(rank + 1) * n]).abs().max()
            y.pow(2).sum().backward()
            assert torch.allclose(xl.grad, xf.grad[rank * n:(rank + 1) * n], atol=1e-5)
        else:
            xl = x.clone().requires_grad_()
            y = row(torch.relu(col(xl)))
            assert torch.allclose(y, yf, atol=1e-5)
            y.pow(2).sum().backward()
            assert torch.allclose(xl.grad, xf.grad, atol=1e-5)
        s = col.shard
        assert torch.allclose(col.weight.grad, colf.weight.grad[rank * s:(rank + 1) * s], atol=1e-5)
        s = row.shard
        assert torch.allclose(row.weight.grad, rowf.weight.grad[:, rank * s:(rank + 1) * s], atol=1e-5)
    g = ColumnParallelLinear(16, 32, tp, gather_output=True, init_seed=11)
    assert torch.allclose(g(x), ColumnParallelLinear(16, 32, tp1, init_seed=11)(x), atol=1e-6)
    _fin()
    return 0


def pipeline_1f1b(rank, world):
    """Two stages, 1F1B with real gradients == the same layers run sequentially."""
    from .. import distributed as D
    from ..nn.parallel import Pipeline1F1BStage, PipelineScheduleConfig
    pg = _init(rank, world)
    full = _mlp(9)
    layers = list(full.children())
    cut = 2
    stage = nn.Sequential(*(layers[:cut] if rank == 0 else layers[cut:]))
    torch.manual_seed(1)
    X, Y = torch.randn(8, 16), torch.randn(8, 4)
    cfg = PipelineScheduleConfig(num_stages=2, num_micros=4)
    st = Pipeline1F1BStage(stage, cfg, rank, process_group=pg, act_shape=(2, 32), act_dtype=torch.float32)
    loss = st.run(X if rank == 0 else None, loss_fn=lambda o, t: ((o - t) ** 2).mean(), targets=Y if rank == 1 else None)
    ref_loss = sum(((full(X[i * 2:(i + 1) * 2]) - Y[i * 2:(i + 1) * 2]) ** 2).mean() / 4 for i in range(4))
    ref_loss.backward()
    mine = list(stage.parameters())
    refp = [p for l in (layers[:cut] if rank == 0 else layers[cut:]) for p in l.parameters()]
    for a, b in zip(mine, refp):
        assert torch.allclose(a.grad, b.grad, atol=1e-5), (a.grad - b.grad).abs().max()
    if rank == 1:
        assert abs(float(loss) - float(ref_loss)) < 1e-5
    _fin()
    return 0


def rank_that_dies(rank, world):
    """Rank 1 leaves before the collective; rank 0's all-reduce must end with CollectiveTimeout, not hang."""
    from .. import distributed as D
    D.init_process_group("gloo", rank, world, os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), timeout_sec=3)
    if rank == 1:
        os._exit(0)
    try:
        D.all_reduce(torch.ones(4))
    except D.CollectiveTimeout:
        os._exit(0)
    except Exception:
        os._exit(0)
    os._exit(7)


def mlp_ddp_config1(rank, world):
    """The CPU plumbing check of the MLP benchmark config: DDP world_size 2, a few Adam steps, ranks stay in sync."""
    from .. import distributed as D
    from ..models.mlp import MLPClassifier
    from ..optim import Adam
    _init(rank, world)
    torch.manual_seed(rank)
    model = MLPClassifier()
    ddp = D.DistributedDataParallel(model)
    opt = Adam(model.parameters(), lr=1e-3)
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(3):
        x, y = torch.rand(64, 784, generator=g), torch.randint(0, 10, (64,), generator=g)
        ddp.zero_grad()
        nn.functional.cross_entropy(ddp(x), y).backward()
        ddp.finish_gradient_synchronization()
        opt.step()
    w = model[0].weight.detach().clone()
    parts = [torch.zeros_like(w) for _ in range(world)]
    D.all_gather(parts, w)
    assert all(torch.allclose(parts[0], p, atol=1e-6) for p in parts)
    _fin()
    return 0


def local_sgd_averages(rank, world):
    """Ranks drift apart for sync_every - 1 steps, meet on the average at the next; with sync_every = 1 and plain SGD the run
    equals gradient averaging."""
    from .. import distributed as D
    from ..optim import SGD
    _init(rank, world)
    torch.manual_seed(5)
    X, Y = torch.randn(8 * world, 16), torch.randn(8 * world, 4)
    xs, ys = X[rank::world], Y[rank::world]
    model = D.LocalSGD(_mlp(3 + rank), sync_every=3)                 # different init per rank: the constructor broadcasts rank 0's
    opt = SGD(model.parameters(), lr=0.05)
    flat = lambda m: torch.cat([p.detach().reshape(-1) for p in m.parameters()])     # noqa: E731

    def spread():
        f = flat(model)
        parts = [torch.zeros_like(f) for _ in range(world)]
        D.all_gather(parts, f)
        return max(float((p - parts[0]).abs().max()) for p in parts)
    assert spread() == 0.0
    did = []
    for step in range(6):
        opt.zero_grad()
        ((model(xs) - ys) ** 2).mean().backward()
        opt.step()
        did.append(model.step_done())
        assert (spread() == 0.0) == did[-1], (step, spread(), did)
    assert did == [False, False, True, False, False, True] and model.syncs == 2
    # sync_every = 1 with SGD: averaging parameters after the step == averaging gradients before it
    ref, m1 = _mlp(9), D.LocalSGD(_mlp(9), sync_every=1)
    ro, o1 = SGD(ref.parameters(), lr=0.1), SGD(m1.parameters(), lr=0.1)
    for _ in range(3):
        ro.zero_grad()
        ((ref(X) - Y) ** 2).mean().backward()
        ro.step()
        o1.zero_grad()
        ((m1(xs) - ys) ** 2).mean().backward()
        o1.step()
        assert m1.step_done()
    assert torch.allclose(flat(ref), flat(m1), atol=1e-5), float((flat(ref) - flat(m1)).abs().max())
    # outer momentum: the averaged point moves by outer_lr * (momentum * v + displacement)
    m2 = D.LocalSGD(_mlp(11), sync_every=2, outer_momentum=0.5, outer_lr=1.0)
    o2 = SGD(m2.parameters(), lr=0.05)
    start = flat(m2).clone()
    moved = []
    for step in range(4):
        o2.zero_grad()
        ((m2(xs) - ys) ** 2).mean().backward()
        o2.step()
        if m2.step_done():
            moved.append(flat(m2).clone())
    assert len(moved) == 2 and spread() >= 0.0
    f2 = flat(m2)
    parts = [torch.zeros_like(f2) for _ in range(world)]
    D.all_gather(parts, f2)
    assert all(torch.equal(p, parts[0]) for p in parts) and not torch.equal(moved[0], start)
    _fin()
    return 0


def ring_attention_matches_full(rank, world):
    """Context parallelism: output and gradients of ring attention over sequence blocks == attention over the whole sequence."""
    import torch.distributed as dist
    from ..nn.parallel import ring_attention, shard_sequence
    _init(rank, world)
    torch.manual_seed(17)
    B, H, T, Dh = 2, 3, 8 * world, 16
    for causal in (True, False):
        q, k, v = (torch.randn(B, H, T, Dh, dtype=torch.float64) for _ in range(3))
        w = torch.randn(B, H, T, Dh, dtype=torch.float64)                  # weights of the scalar the gradients are taken of
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=causal)
        (ref * w).sum().backward()
        ql, kl, vl = (shard_sequence(t, 2).clone().requires_grad_(True) for t in (q, k, v))
        out = ring_attention(ql, kl, vl, causal=causal)
        (out * shard_sequence(w, 2)).sum().backward()
        assert torch.allclose(out, shard_sequence(ref.detach(), 2), atol=1e-5), float((out - shard_sequence(ref.detach(), 2)).abs().max())
        for got, want, name in ((ql.grad, qf.grad, "dq"), (kl.grad, kf.grad, "dk"), (vl.grad, vf.grad, "dv")):
            assert torch.allclose(got, shard_sequence(want, 2), atol=1e-5), (name, causal, float((got - shard_sequence(want, 2)).abs().max()))
    _fin()
    return 0


def expert_parallel_matches_dense(rank, world):
    """Expert parallelism: tokens routed over all-to-all to the ranks' experts == every expert in one process, gradients too."""
    import torch.distributed as dist
    from ..nn.parallel import Expert, ExpertParallelMoE
    _init(rank, world)
    dim, hidden, E, k = 16, 24, 2 * world, 2
    moe = ExpertParallelMoE(dim, hidden, E, top_k=k, seed=40)
    # the dense oracle holds every expert, built from the same per-expert seeds
    experts = []
    for e in range(E):
        ex = Expert(dim, hidden)
        g = torch.Generator().manual_seed(40 + 1 + e)
        with torch.no_grad():
            for p in ex.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * p.shape[1] ** -0.5)
        experts.append(ex)
    router = moe.router.weight.detach().clone().requires_grad_(True)
    torch.manual_seed(100 + rank)
    x = torch.randn(5 + rank, 3, dim, requires_grad=True)                 # a different number of tokens per rank
    xr = x.detach().clone().requires_grad_(True)
    y = moe(x)
    want = ExpertParallelMoE.dense_forward(xr, router, experts, k)
    assert torch.allclose(y, want, atol=1e-5), float((y - want).abs().max())
    assert int(moe.last_tokens_per_expert.sum()) == x.shape[0] * x.shape[1] * k
    w = torch.randn_like(y)
    (y * w).sum().backward()
    (want * w).sum().backward()
    assert torch.allclose(x.grad, xr.grad, atol=1e-5)
    # an expert's gradient is the sum over the tokens of every rank that chose it; the router's is this rank's share
    for e in range(E):                                                     # the same collectives in the same order on every rank
        local = list(moe.experts[e % moe.local].parameters()) if e // moe.local == rank else None
        for i, p_dense in enumerate(experts[e].parameters()):
            total = p_dense.grad.clone() if p_dense.grad is not None else torch.zeros_like(p_dense)
            dist.all_reduce(total)                                         # the oracle on each rank saw only that rank's tokens
            if local is not None:
                assert torch.allclose(local[i].grad, total, atol=1e-5), (e, i, float((local[i].grad - total).abs().max()))
    assert torch.allclose(moe.router.weight.grad, router.grad, atol=1e-5)
    assert float(moe.load_balance_loss(x.detach())) > 0.5
    _fin()
    return 0


def gguf_tp_oracle_matches_single(rank, world):
    """Tensor-parallel GGUF decode on CPU ranks: the sharded oracle (heads, FFN blocks split unevenly, vocabulary rows) gives
    the single-process logits and the same greedy ids."""
    import tempfile
    from .. import distributed as D
    from ..io.config import tiny_qwen3_config
    from ..io.synthetic import write_synthetic_gguf
    from ..models.gguf_oracle import OracleModel, TPOracleModel
    _init(rank, world)
    path = os.path.join(tempfile.gettempdir(), f"ptb_tp_oracle_{os.environ['MASTER_PORT']}.gguf")
    if rank == 0:
        # 5 FFN blocks of 256: uneven over 2 and 4 ranks; a vocabulary that does not divide by the number of ranks
        write_synthetic_gguf(path, tiny_qwen3_config(layers=2, hidden=256, heads=8, kv_heads=4, inter=1280, vocab=515), seed=21, device="cpu", std=0.05)
    D.barrier()
    prompt = [300, 301, 17, 260, 5, 401]
    tp = TPOracleModel(path, rank, world, max_seq=64)
    assert sum([tp.local_inter]) > 0
    inter = torch.tensor([float(tp.local_inter)])
    D.all_reduce(inter)
    assert int(inter) == 1280
    single = OracleModel(path, max_seq=64)
    want = single.forward(prompt)
    got = tp.forward(prompt)
    assert got.shape == want.shape and torch.allclose(got, want, atol=2e-4, rtol=2e-4), float((got - want).abs().max())
    cos = torch.nn.functional.cosine_similarity(got[-1], want[-1], dim=0)
    assert float(cos) > 0.99999
    ids_tp, ids_one = [], []
    lt, lo = got, want
    for _ in range(5):
        ids_tp.append(int(lt[-1].argmax()))
        ids_one.append(int(lo[-1].argmax()))
        lt, lo = tp.forward([ids_one[-1]]), single.forward([ids_one[-1]])
    assert ids_tp == ids_one, (ids_tp, ids_one)
    D.barrier()
    if rank == 0:
        os.remove(path)
    _fin()
    return 0
