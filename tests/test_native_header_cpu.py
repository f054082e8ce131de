"""The public C header of the native library parses as C and as C++, and declares what the library exports."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "prometorch_b200", "csrc")
CUDA_INC = "/usr/local/cuda/include"


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and the CUDA headers")
@pytest.mark.parametrize("lang,cc", [("c", "gcc"), ("c++", "g++")])
def test_header_parses(tmp_path, lang, cc):
    src = tmp_path / ("t.c" if lang == "c" else "t.cpp")
    src.write_text('#include "ptb200.h"\nint main(void) { return ptb_last_error() == 0; }\n')
    r = subprocess.run([cc, "-fsyntax-only", "-x", lang, f"-I{CUDA_INC}", f"-I{CSRC}", str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_header_is_up_to_date():
    from prometorch_b200 import _gen_header
    assert open(os.path.join(CSRC, "ptb200.h")).read() == _gen_header.render(), "run `python -m prometorch_b200._gen_header`"


def test_header_lists_every_entry_point():
    declared = set(re.findall(r"\b(ptb_\w+)\s*\(", open(os.path.join(CSRC, "ptb200.h")).read()))
    defined = set()
    for f in os.listdir(CSRC):
        if f.endswith(".cu"):
            defined |= set(re.findall(r"PTB_API[^;{]*?\b(ptb_\w+)\s*\(", open(os.path.join(CSRC, f)).read()))
    assert defined - declared == set(), sorted(defined - declared)


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INC), reason="needs g++ and the CUDA headers")
def test_c_header_parses_in_a_cpp_program(tmp_path):
    """The public header is plain C that a C++ program can include (the C++ GGUFModel of cpp_api/promethorch/gguf.h does)."""
    src = tmp_path / "t.cpp"
    src.write_text('#include "ptb200.h"\nint main() { return ptb_last_error() == nullptr; }\n')
    r = subprocess.run(["g++", "-std=c++17", "-fsyntax-only", f"-I{CUDA_INC}", f"-I{CSRC}", str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
