"""``import promethorch as pt`` — the reference's package name, served by :mod:`prometorch_b200`."""
import sys as _sys

import prometorch_b200 as _impl
from prometorch_b200 import *  # noqa: F401,F403
from prometorch_b200 import (amp, audio, autograd, data, distributed, io, jit, mlir, mobile, nn, onnx, optim, ops, parallel,  # noqa: F401
                             quantization, serve, text, trainer, utils, vision, __version__)

for _name in ("amp", "audio", "autograd", "data", "distributed", "io", "jit", "mlir", "mobile", "nn", "onnx", "optim", "ops", "parallel",
              "quantization", "serve", "text", "trainer", "utils", "vision"):
    _sys.modules[f"promethorch.{_name}"] = getattr(_impl, _name)
_sys.modules["promethorch.nn.parallel"] = _impl.nn.parallel
_sys.modules["promethorch.nn.functional"] = _impl.nn.functional
