#!/usr/bin/env python
"""Build the reference project's own CUDA decode CLI, unmodified, without network access.

    python baseline/build_reference.py [--src /path/to/PromeTorch] [--jobs 8]

The reference's GGUF decode benchmark is a C++ program (examples/gguf/test_gguf_inference.cpp)
built by its CMake tree.  The tree's two network fetches (googletest, pybind11) sit behind
PT_BUILD_TESTS and PT_BUILD_PYTHON, so with tests off the configure step needs nothing but
cmake, ninja, g++ and nvcc.  The source tree is only read; the build directory is a temporary
one.  The reference's own architecture list (75 80 86 89, CMakeLists.txt:319) is kept: CMake
embeds PTX next to every SASS image, and the driver compiles the compute_89 PTX for the GPU
that is present at first use.

Outputs (three files) land in baseline/_ref/bin/, which is where ``bench.py --impl reference``
looks for them: test_gguf_inference, libaten_cuda.so, libc10.so.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "bin")
ARTIFACTS = ("examples/gguf/test_gguf_inference", "libaten_cuda.so", "libc10.so")


def build(src: str, jobs: int = 8, build_dir: str | None = None, log=sys.stdout) -> str:
    if not os.path.isfile(os.path.join(src, "examples", "gguf", "test_gguf_inference.cpp")):
        raise SystemExit(f"{src} is not a PromeTorch source tree")
    bdir = build_dir or tempfile.mkdtemp(prefix="prometorch_ref_build_")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cfg = ["cmake", "-S", src, "-B", bdir, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release", "-DPT_USE_CUDA=ON",
           "-DPT_USE_CUDNN=OFF", "-DPT_BUILD_TESTS=OFF", f"-DCMAKE_CUDA_COMPILER={nvcc}"]
    for cmd in (cfg, ["ninja", "-C", bdir, f"-j{jobs}", "test_gguf_inference"]):
        print("+", " ".join(cmd), file=log, flush=True)
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        print(r.stdout[-4000:], file=log, flush=True)
        if r.returncode != 0:
            raise SystemExit(f"step failed with exit code {r.returncode}: {' '.join(cmd[:3])}")
    os.makedirs(OUT, exist_ok=True)
    for rel in ARTIFACTS:
        shutil.copy2(os.path.join(bdir, rel), os.path.join(OUT, os.path.basename(rel)))
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=os.environ.get("PROMETORCH_REFERENCE_SRC"), required="PROMETORCH_REFERENCE_SRC" not in os.environ,
                    help="checkout of the reference project (or set PROMETORCH_REFERENCE_SRC)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 8)
    ap.add_argument("--build-dir", default=None)
    a = ap.parse_args()
    print("built into", build(a.src, a.jobs, a.build_dir))
