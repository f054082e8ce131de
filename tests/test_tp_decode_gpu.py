"""Tensor-parallel GGUF decode on 2 GPUs: fused GEMV + all-reduce over peer memory against the 1-GPU engine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


@pytest.mark.parametrize("flow", ["plain", "dataflow"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_decode_matches_single_gpu(tmp_path, world, flow):
    """Both hand-over flows at every world size the machine has GPUs for: hidden states against the 1-GPU engine, ids
    equal across ranks, batched prefill, and the NCCL-only arm on the same shards."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "tp_decode_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PTB_DECODE_FLOW=flow)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300), worker, str(tmp_path / "tp.gguf")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "TP_DECODE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
