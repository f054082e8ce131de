"""The C++ torch-style API (prometorch_b200/cpp_api): a C++ program is compiled against the installed libtorch and run.
It trains the benchmark MLP for a few steps, runs all sixteen optimizers and schedulers, round-trips PTOR / .pt
checkpoints and runs DistributedDataParallel with no_sync plus tensor-parallel layers over two forked TCP ranks."""
import os
import shutil
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torch_flags():
    ti = os.path.dirname(torch.__file__)
    return [f"-I{ti}/include", f"-I{ti}/include/torch/csrc/api/include", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
            f"-L{ti}/lib", "-ltorch", "-ltorch_cpu", "-lc10", f"-Wl,-rpath,{ti}/lib"]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_api_trains_and_synchronises(tmp_path):
    exe = str(tmp_path / "train_mlp")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "train_mlp.cpp"), "-o", exe,
           f"-I{ROOT}/prometorch_b200/cpp_api"] + _torch_flags()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(29750 + os.getpid() % 200)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CPP_API_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs g++")
def test_cpp_api_amp_data_fsdp_pipeline(tmp_path):
    """GradScaler / autocast guards, datasets + DataLoader with worker threads, GPipe, and over forked ranks: sharded data
    parallelism with a ZeRO optimizer against a replica, the offload optimizer, the split all-gather, a 1F1B pipeline whose
    stage gradients equal the single-process model's."""
    exe = str(tmp_path / "parallel_api")
    cmd = ["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "parallel_api.cpp"), "-o", exe,
           f"-I{ROOT}/prometorch_b200/cpp_api"] + _torch_flags() + ["-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe, str(30050 + os.getpid() % 200), str(tmp_path / "ckpt")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "CPP_PARALLEL_API_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
