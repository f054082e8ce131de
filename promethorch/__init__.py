"""``import promethorch as pt`` — the reference's package name, served by :mod:`prometorch_b200`."""
import sys as _sys

import prometorch_b200 as _impl
from prometorch_b200 import *  # noqa: F401,F403
from prometorch_b200 import (amp, audio, autograd, data, distributed, io, jit, mlir, mobile, nn, onnx, optim, ops, parallel,  # noqa: F401
                             quantization, serve, text, trainer, utils, vision, __version__)

for _name in ("amp", "audio", "autograd", "data", "distributed", "io", "jit", "mlir", "mobile", "nn", "onnx", "optim", "ops", "parallel",
              "quantization", "serve", "text", "trainer", "utils", "vision"):
    _sys.modules[f"promethorch.{_name}"] = getattr(_impl, _name)
from prometorch_b200 import safetensors_reader, transformers_compat  # noqa: E402,F401
from prometorch_b200.serve import llm as _llm  # noqa: E402

_sys.modules["promethorch.transformers_compat"] = transformers_compat
_sys.modules["promethorch.safetensors_reader"] = safetensors_reader
_sys.modules["promethorch.serve.llm"] = _llm
_sys.modules["promethorch.nn.parallel"] = _impl.nn.parallel
_sys.modules["promethorch.nn.functional"] = _impl.nn.functional


def __getattr__(name: str):
    return getattr(_impl, name)
