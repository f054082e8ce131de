"""Multi-rank logic on CPU ranks (Gloo over 127.0.0.1, spawned processes) and in-process fakes."""
import os
import random
import threading

import pytest
import torch
import torch.nn as nn

from prometorch_b200 import distributed as D
from prometorch_b200.testing import dist_workers as W


def _launch(fn, world=2, timeout=180):
    port = 29700 + (os.getpid() * 7 + random.randint(0, 200)) % 1200
    return D.launch(world, fn, "127.0.0.1", port, timeout=timeout)


@pytest.mark.parametrize("fn", [W.collectives, W.ddp_matches_single, W.fsdp_matches_unsharded, W.tp_matches_unsharded, W.pipeline_1f1b,
                                W.mlp_ddp_config1], ids=lambda f: f.__name__)
def test_two_ranks(fn):
    assert _launch(fn, 2) == 0


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("fn", [W.ring_attention_matches_full, W.expert_parallel_matches_dense], ids=lambda f: f.__name__)
def test_context_and_expert_parallel(fn, world):
    assert _launch(fn, world) == 0


@pytest.mark.parametrize("world", [2, 4])
def test_gguf_tensor_parallel_oracle_on_cpu_ranks(world):
    assert _launch(W.gguf_tp_oracle_matches_single, world) == 0


def test_local_sgd():
    assert _launch(W.local_sgd_averages, 2) == 0


def test_ring_attention_and_moe_without_a_process_group():
    """One process: ring attention is plain attention, the expert-parallel layer runs all experts locally."""
    from prometorch_b200.nn.parallel import ExpertParallelMoE, ring_attention
    torch.manual_seed(3)
    q, k, v = (torch.randn(2, 2, 12, 8) for _ in range(3))
    for causal in (True, False):
        assert torch.allclose(ring_attention(q, k, v, causal=causal), torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal), atol=1e-5)
    moe = ExpertParallelMoE(8, 12, 4, top_k=2, seed=1)
    x = torch.randn(7, 8, requires_grad=True)
    y = moe(x)
    want = ExpertParallelMoE.dense_forward(x, moe.router.weight, list(moe.experts), 2)
    assert torch.allclose(y, want, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and all(p.grad is not None for p in moe.parameters())


def test_dead_rank_is_detected_not_hung():
    assert _launch(W.rank_that_dies, 2, timeout=60) == 0


def test_launcher_propagates_failure():
    assert _launch(_fail_on_rank1, 2, timeout=60) == 3


def _fail_on_rank1(rank, world):
    return 3 if rank == 1 else 0


def test_no_sync_with_counting_pg():
    pg = D.CountingPG(rank=0, world_size=2)
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    ddp = D.DistributedDataParallel(model, pg, broadcast_parameters=False, bucket_mb=1e-5)
    nb = len(ddp.buckets)
    x = torch.randn(3, 4)
    with ddp.no_sync():
        assert ddp.require_grad_sync is False
        with ddp.no_sync():                       # nests and restores
            ddp(x).sum().backward()
        assert ddp.require_grad_sync is False
        ddp(x).sum().backward()
    assert ddp.require_grad_sync is True and pg.all_reduce_calls == 0
    g_acc = model[0].weight.grad.clone()
    ddp(x).sum().backward()
    ddp.finish_gradient_synchronization()
    assert pg.all_reduce_calls == nb
    assert torch.allclose(model[0].weight.grad * 4, g_acc * 3, atol=1e-6)    # 3 accumulated backwards scaled by 1/2, against 2 unscaled
    with D.DDPNoSyncGuard(ddp):
        assert not ddp.require_grad_sync
    assert ddp.require_grad_sync
    ddp.sync_gradients()
    assert pg.all_reduce_calls == 2 * nb


def test_ddp_logs_every_bucket_reduction(tmp_path):
    """With a metrics writer, each bucket's all-reduce is logged with its bytes on the wire and a roofline fraction."""
    import json
    from prometorch_b200.utils.metrics import MetricsWriter
    pg = D.CountingPG(rank=0, world_size=2)
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    w = MetricsWriter(str(tmp_path / "m.jsonl"))
    ddp = D.DistributedDataParallel(model, pg, broadcast_parameters=False, bucket_mb=1e-5, metrics=w)
    ddp(torch.randn(3, 4)).sum().backward()
    ddp.finish_gradient_synchronization()
    w.close()
    recs = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert len(recs) == len(ddp.buckets) == pg.all_reduce_calls
    total = sum(p.numel() for p in model.parameters())
    assert all(r["kind"] == "collective" and r["op"] == "all_reduce" and r["world"] == 2 and r["seconds"] >= 0 for r in recs)
    assert sum(r["payload_bytes"] for r in recs) >= 4 * total                   # buckets are padded to 64 elements
    assert all(r["wire_bytes_per_gpu"] == r["payload_bytes"] for r in recs)     # 2 (n - 1) / n = 1 at two ranks


def test_shared_memory_backend_threads():
    groups = D.make_shared_memory_groups(3, timeout=10)
    out = [None] * 3

    def run(r):
        t = torch.full((2,), float(r + 1))
        groups[r].all_reduce(t, D.ReduceOp.SUM)
        b = torch.full((2,), float(r))
        groups[r].broadcast(b, 1)
        groups[r].barrier()
        out[r] = (t, b)
    ts = [threading.Thread(target=run, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert all(torch.allclose(o[0], torch.full((2,), 6.0)) and torch.allclose(o[1], torch.full((2,), 1.0)) for o in out)
    g1 = D.make_shared_memory_groups(2, timeout=0.3)
    with pytest.raises(D.CollectiveTimeout):          # the other rank never arrives
        g1[0].barrier()


def test_flag_protocol_model_survives_a_missing_peer_and_a_withheld_flag():
    """The CPU model of the fused collectives' flag protocol: a healthy call reduces; a rank that never launches, a flag write
    that is withheld and a rank that is late beyond the budget each end with a timeout status on the ranks that waited (and
    nobody hangs); the next sequence number on the same channel works again and reduces correctly."""
    from prometorch_b200.testing.symm_fake import ERR_FLAG_TIMEOUT, OK, FakeSymmChannel
    world, n = 3, 12
    ch = FakeSymmChannel(world, n, budget_s=0.4)
    vals = {r: [float(r + 1)] * n for r in range(world)}
    assert ch.run(1, vals) == {0: OK, 1: OK, 2: OK}
    assert all(ch.mem[r].data == [6.0] * n for r in range(world))
    # rank 2 never launches: the others time out, skip the reduction, leave their buffers alone
    t0 = __import__("time").monotonic()
    st = ch.run(2, vals, skip=(2,))
    assert st == {0: ERR_FLAG_TIMEOUT, 1: ERR_FLAG_TIMEOUT} and __import__("time").monotonic() - t0 < 5.0
    assert ch.mem[0].data == [1.0] * n and ch.mem[0].ticket == 0 and ch.mem[1].ticket == 0
    for r in range(world):
        ch.clear_status(r)
    assert ch.run(3, vals) == {0: OK, 1: OK, 2: OK} and ch.mem[1].data == [6.0] * n          # the channel is usable again
    # one flag write is withheld (rank 0's entry word at rank 1): rank 1 gives up, the others finish their slices
    ch.drop = lambda writer, target, phase, seq: seq == 4 and writer == 0 and target == 1 and phase == 0
    st = ch.run(4, vals)
    assert st[1] == ERR_FLAG_TIMEOUT and ch.mem[1].ticket == 0
    ch.drop = None
    for r in range(world):
        ch.clear_status(r)
    assert ch.run(5, vals, scale=0.5) == {0: OK, 1: OK, 2: OK} and ch.mem[2].data == [3.0] * n
    # a rank that is late but inside the budget is waited for; beyond the budget the waiters give up and still recover
    assert ch.run(6, vals, delays={1: 0.05}) == {0: OK, 1: OK, 2: OK}
    st = ch.run(7, vals, delays={1: 1.2})
    assert st[0] == ERR_FLAG_TIMEOUT and st[2] == ERR_FLAG_TIMEOUT
    for r in range(world):
        ch.clear_status(r)
    assert ch.run(8, vals) == {0: OK, 1: OK, 2: OK} and ch.mem[0].data == [6.0] * n


def test_heartbeat_detects_silent_rank():
    store = D.DictStore()
    a = D.Heartbeat(store, 0, 2, interval=0.05, timeout=0.4).start()
    b = D.Heartbeat(store, 1, 2, interval=0.05, timeout=0.4).start()
    import time
    time.sleep(0.2)
    a.check()
    b.stop()                                             # rank 1 goes silent
    time.sleep(0.7)
    with pytest.raises(D.RankFailure) as e:
        a.check()
    assert e.value.ranks == [1]
    a.stop()


def test_gpipe_matches_sequential():
    from prometorch_b200.nn.parallel import Pipeline
    torch.manual_seed(0)
    seq = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 16), nn.ReLU(), nn.Linear(16, 4))
    x = torch.randn(8, 8)
    ref = seq(x)
    pipe = Pipeline(seq, num_stages=2, chunks=4)
    out = pipe(x)
    assert torch.allclose(out, ref, atol=1e-6)
    out.sum().backward()
    assert seq[0].weight.grad is not None


def test_distributed_sampler_disjoint():
    from prometorch_b200.data import DistributedSampler, TensorDataset
    ds = TensorDataset(torch.arange(10))
    idx = [list(DistributedSampler(ds, num_replicas=3, rank=r, shuffle=True, seed=1)) for r in range(3)]
    assert all(len(i) == 4 for i in idx)
    assert set(sum(idx, [])) == set(range(10))
    s = DistributedSampler(ds, num_replicas=3, rank=0, shuffle=True, seed=1)
    a = list(s)
    s.set_epoch(1)
    assert list(s) != a


def test_parse_dist_args():
    a = D.parse_dist_args(["--rank", "2", "--world-size", "4", "--master-port", "1234", "--nprocs", "2"])
    assert (a.rank, a.world_size, a.master_port, a.nprocs) == (2, 4, 1234, 2)


def test_file_backend_collectives_and_timeout(tmp_path):
    """Ranks that meet through a directory: every collective, generations cleaned up, a missing rank times out."""
    import threading
    from prometorch_b200.distributed import CollectiveTimeout, FileBackend, ReduceOp
    W = 3
    results, errors = {}, []

    def worker(r):
        try:
            pg = FileBackend(str(tmp_path / "sync"), r, W, timeout=20.0)
            a = torch.arange(4, dtype=torch.float32) * (r + 1)
            pg.all_reduce(a)
            b = torch.full((3,), float(r))
            pg.broadcast(b, src=1)
            outs = [torch.zeros(2) for _ in range(W)]
            pg.all_gather(outs, torch.tensor([r, r * 10.0]))
            rs = torch.zeros(2)
            pg.reduce_scatter(rs, [torch.full((2,), float(r + k)) for k in range(W)], op=ReduceOp.AVG)
            h = torch.ones(5, dtype=torch.bfloat16) * (r + 1)
            pg.all_reduce(h, op=ReduceOp.MAX)
            for _ in range(4):
                pg.barrier()
            results[r] = (a, b, torch.stack(outs), rs, h)
        except Exception as e:          # noqa: BLE001
            errors.append(e)
    ts = [threading.Thread(target=worker, args=(r,)) for r in range(W)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(60)
    assert not errors, errors
    for r in range(W):
        a, b, g, rs, h = results[r]
        assert torch.equal(a, torch.arange(4, dtype=torch.float32) * 6)
        assert torch.equal(b, torch.full((3,), 1.0))
        assert torch.equal(g, torch.tensor([[0.0, 0.0], [1.0, 10.0], [2.0, 20.0]]))
        assert torch.allclose(rs, torch.full((2,), (0 + 1 + 2) / 3 + r))
        assert torch.equal(h.float(), torch.full((5,), 3.0))
    left = sorted(p.name for p in (tmp_path / "sync").iterdir())
    assert len(left) <= 2 * 2 * W, left                      # only the last two generations remain
    lonely = FileBackend(str(tmp_path / "alone"), 0, 2, timeout=0.2)
    with pytest.raises(CollectiveTimeout):
        lonely.barrier()


def test_data_parallel_step_averages_shard_gradients():
    from prometorch_b200.distributed import data_parallel_step
    torch.manual_seed(0)
    lin = torch.nn.Linear(6, 3)
    x, y = torch.randn(8, 6), torch.randint(0, 3, (8,))

    def fn(rank, xs, ys):
        loss = torch.nn.functional.cross_entropy(lin(xs), ys)
        loss.backward()
        return loss.item()
    loss = data_parallel_step(fn, x, y, list(lin.parameters()), 4)
    got = [p.grad.clone() for p in lin.parameters()]
    lin.zero_grad()
    ref = torch.nn.functional.cross_entropy(lin(x), y)            # equal shards: the mean of shard means is the batch mean
    ref.backward()
    assert abs(loss - ref.item()) < 1e-6
    for g, p in zip(got, lin.parameters()):
        assert torch.allclose(g, p.grad, atol=1e-6)


def _fsdp_train(world, steps, ckpt_dir=None, load_dir=None, seed=0, resume_steps=0):
    """Thread ranks: ``steps`` AdamW steps of a tiny MLP under FSDP; optionally save at the end / load at the start.
    Returns (full parameters after training, extra from the manifest)."""
    import threading
    from prometorch_b200 import optim
    from prometorch_b200.distributed import FullyShardedDataParallel, make_shared_memory_groups
    from prometorch_b200.distributed.checkpoint import load_sharded, save_sharded
    groups = make_shared_memory_groups(world, timeout=60.0)
    out, errs = {}, []
    torch.manual_seed(seed)
    X, Y = torch.randn(24, 10), torch.randn(24, 3)
    init = torch.nn.Sequential(torch.nn.Linear(10, 17), torch.nn.Tanh(), torch.nn.Linear(17, 3)).state_dict()   # one RNG user

    def worker(r):
        try:
            model = torch.nn.Sequential(torch.nn.Linear(10, 17), torch.nn.Tanh(), torch.nn.Linear(17, 3))
            model.load_state_dict(init)
            fsdp = FullyShardedDataParallel(model, process_group=groups[r])
            opt = optim.AdamW(fsdp.local_shards(), lr=1e-2, weight_decay=0.01)
            extra = {}
            if load_dir:
                extra = load_sharded(load_dir, fsdp, opt)
            for it in range(steps):
                fsdp.all_gather_params()
                loss = torch.nn.functional.mse_loss(fsdp(X), Y)        # every rank sees the whole batch: world-size independent
                loss.backward()
                fsdp.reduce_scatter_grads()
                opt.step()
                opt.zero_grad()
            if ckpt_dir:
                save_sharded(ckpt_dir, fsdp, opt, extra={"step": steps + resume_steps, "note": "ok"})
            fsdp.all_gather_params()
            out[r] = ({k: v.clone() for k, v in fsdp.full_state_dict().items()}, extra)
        except Exception as e:          # noqa: BLE001
            import traceback
            errs.append(traceback.format_exc())
    ts = [threading.Thread(target=worker, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(120)
    assert not errs, errs[0]
    return out[0]


def test_sharded_checkpoint_resume_and_reshard(tmp_path):
    """6 steps straight == 3 steps, save (2 ranks), load and 3 more steps, with 2 ranks and re-cut for 3 ranks."""
    straight, _ = _fsdp_train(2, 6)
    d = str(tmp_path / "ckpt")
    _fsdp_train(2, 3, ckpt_dir=d)
    import json
    import os
    man = json.load(open(os.path.join(d, "manifest.json")))
    assert man["format"] == "ptb-sharded-1" and man["world_size"] == 2 and len(man["params"]) == 4 and man["extra"]["step"] == 3
    assert sorted(os.listdir(d)) == ["manifest.json", "rank00000.safetensors", "rank00001.safetensors"]
    same, extra = _fsdp_train(2, 3, load_dir=d)
    other, extra3 = _fsdp_train(3, 3, load_dir=d)
    assert extra == {"step": 3, "note": "ok"} and extra3 == extra
    for k in straight:
        assert torch.allclose(same[k], straight[k], atol=1e-6), k
        assert torch.allclose(other[k], straight[k], atol=1e-5), k
    from prometorch_b200.distributed import FullyShardedDataParallel
    from prometorch_b200.distributed.checkpoint import load_sharded
    wrong = FullyShardedDataParallel(torch.nn.Linear(3, 3))
    with pytest.raises(ValueError):
        load_sharded(d, wrong)
