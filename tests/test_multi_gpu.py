"""Fused compute+collective training paths on 2 GPUs (staged GEMM, DDP bucket kernel, fused FSDP, sequence-parallel
TP), and the bounded wait of the flag barrier on one GPU."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.multigpu
@pytest.mark.parametrize("case", ["staged_gemm", "ddp_fused", "fsdp_fused", "fsdp_window", "fsdp_checkpoint", "tp_sp_fused"])
def test_fused_multi_gpu(case):
    world = 2
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "multi_gpu_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), worker, case]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_flag_barrier_wait_runs_out():
    """A barrier whose peer never arrives (a flag nothing sets) returns with a timeout status; the context stays usable."""
    from prometorch_b200 import _native as N
    from prometorch_b200.distributed import ddp as _ddp  # noqa: F401  (registers the prototypes)
    dev = torch.device("cuda", 0)
    mine = torch.zeros(16, dtype=torch.int32, device=dev)
    ghost = torch.zeros(16, dtype=torch.int32, device=dev)          # stands for a peer that never runs
    flags = (C.c_void_p * 2)(mine.data_ptr(), ghost.data_ptr())
    ticket = torch.zeros(1, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    N.check(N.lib().ptb_peer_barrier(flags, 0, 2, 1, ticket.data_ptr(), status.data_ptr(), st), "peer_barrier")
    torch.cuda.synchronize()
    assert int(status) == 2                                          # flag timeout
    assert int(ghost[0]) == 1                                        # it did signal the peer before giving up
    x = torch.ones(4, device=dev) * 2                                # the context still works
    assert float(x.sum()) == 8.0


class _GhostBuffer:
    """What DDP needs from a symmetric buffer, with a second local allocation standing in for a peer that never runs."""

    def __init__(self, nbytes, dev):
        self.mine = torch.zeros((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=dev)
        self.ghost = torch.zeros_like(self.mine)

    def peer_ptr(self, r):
        return (self.mine if r == 0 else self.ghost).data_ptr()

    def tensor(self, dtype, rank=None):
        return (self.mine if rank in (None, 0) else self.ghost).view(dtype)


class _GhostSymm:
    rank, world = 0, 2

    def __init__(self, dev):
        self.device = dev

    def alloc(self, nbytes):
        return _GhostBuffer(nbytes, self.device)


def test_ddp_raises_before_the_optimizer_steps_when_a_peer_never_arrives():
    """The fused bucket all-reduce gives up after its wait budget; finish_gradient_synchronization() must turn that
    into CollectiveTimeout before the optimizer runs, and the channel must work again afterwards."""
    import prometorch_b200 as pt
    from prometorch_b200.distributed import CollectiveTimeout, CountingPG, DistributedDataParallel
    from prometorch_b200.distributed.ddp import set_collective_timeout
    from prometorch_b200 import _native as N
    dev = torch.device("cuda", 0)
    old_ms = N.lib().ptb_get_collective_timeout_ms()
    set_collective_timeout(0.2)
    try:
        model = torch.nn.Linear(64, 64).to(dev)
        ddp = DistributedDataParallel(model, CountingPG(rank=0, world_size=2), broadcast_parameters=False, symm=_GhostSymm(dev))
        opt = pt.optim.SGD(model.parameters(), lr=0.1)
        before = model.weight.detach().clone()
        ddp(torch.randn(8, 64, device=dev)).sum().backward()
        with pytest.raises(CollectiveTimeout):
            ddp.finish_gradient_synchronization()
            opt.step()                                   # never reached
        assert torch.equal(model.weight.detach(), before)
        # the kernel reset its ticket and told its peer: the same channel can be launched again (and times out again)
        ddp(torch.randn(8, 64, device=dev)).sum().backward()
        with pytest.raises(CollectiveTimeout):
            ddp.finish_gradient_synchronization()
        ch = ddp.buckets[0].channel
        assert int(ch.ticket) == 0 and int(ch.buf.tensor(torch.int32, rank=1).sum()) == 0
    finally:
        N.lib().ptb_set_collective_timeout_ms(old_ms)
