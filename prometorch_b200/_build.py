"""Builds the native library in-tree with nvcc for sm_100a.

``python -m prometorch_b200._build`` (or ``build()``) compiles every ``.cu`` /
``.cpp`` under ``csrc/`` to an object file and links ``lib/libptb200.so``.
Objects are rebuilt only when their source (or any header) is newer.  The
library has no PyTorch or Python dependency: it exports a C ABI that the Python
side binds with ctypes, so a rebuild takes seconds and the same ``.so`` can be
linked from C++ programs.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
LIB = LIBDIR / "libptb200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


APPS = ROOT / "cpp_api" / "apps"
PROMESERVE = LIBDIR / "promeserve"
GGUF_GENERATE = LIBDIR / "gguf_generate"


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(list(CSRC.rglob("*.cu")) + list(CSRC.rglob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    objdir = LIBDIR / "obj"
    objdir.mkdir(parents=True, exist_ok=True)
    hdr_m = _headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = objdir / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = obj.with_suffix(".log")
        log.write_text(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            print(r.stderr)
        return obj

    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not LIB.exists():
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIB), *[str(o) for o in objs], "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)


def build_promeserve(force: bool = False) -> Path:
    """The native server (``cpp_api/apps/promeserve.cpp``: C++ HTTP server + tokenizer + the CUDA decode engine) as
    ``lib/promeserve``, linked against ``lib/libptb200.so`` and the CUDA runtime."""
    return build_app("promeserve", force)


def build_generate(force: bool = False) -> Path:
    """The native generation CLI (``cpp_api/apps/gguf_generate.cpp``) as ``lib/gguf_generate``."""
    return build_app("gguf_generate", force)


def build_app(name: str, force: bool = False) -> Path:
    build()
    src = APPS / f"{name}.cpp"
    PROMESERVE = LIBDIR / name
    hdrs = list((ROOT / "cpp_api" / "promethorch").glob("*.h")) + [CSRC / "ptb200.h", CSRC / "ptb200_types.h"]
    newest = max([src.stat().st_mtime, LIB.stat().st_mtime] + [h.stat().st_mtime for h in hdrs if h.exists()])
    if not force and PROMESERVE.exists() and PROMESERVE.stat().st_mtime >= newest:
        return PROMESERVE
    cuda = Path(_nvcc()).resolve().parent.parent
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-std=c++17", "-O3", str(src), "-o", str(PROMESERVE), f"-I{ROOT / 'cpp_api'}", f"-I{cuda / 'include'}", f"-L{LIBDIR}", "-lptb200",
           f"-L{cuda / 'lib64'}", "-lcudart", "-lpthread", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{cuda / 'lib64'}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building {name} failed:\n{r.stdout}\n{r.stderr}")
    return PROMESERVE
