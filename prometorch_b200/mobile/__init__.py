"""PTMB: a flat mobile format (``"PTMB"``, u32 version, u32 op count; per op: u8 kind, tensors) and a small
executor for Linear/activation chains (torch/mobile/executor.h in the reference)."""
import struct

import torch
import torch.nn as nn

MAGIC = b"PTMB"
_KINDS = {nn.Linear: 1, nn.ReLU: 2, nn.Sigmoid: 3, nn.Tanh: 4, nn.GELU: 5, nn.SiLU: 6, nn.Softmax: 7}


def _wt(f, t):
    t = t.detach().float().contiguous().cpu()
    f.write(struct.pack("<I", t.dim()))
    for s in t.shape:
        f.write(struct.pack("<q", s))
    f.write(t.numpy().tobytes())


def save(model: nn.Module, path: str):
    ops = [m for m in model.modules() if type(m) in _KINDS]
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<II", 1, len(ops)))
        for m in ops:
            f.write(struct.pack("<B", _KINDS[type(m)]))
            if isinstance(m, nn.Linear):
                _wt(f, m.weight)
                f.write(struct.pack("<B", m.bias is not None))
                if m.bias is not None:
                    _wt(f, m.bias)


def _rt(f):
    nd = struct.unpack("<I", f.read(4))[0]
    shape = [struct.unpack("<q", f.read(8))[0] for _ in range(nd)]
    n = 1
    for s in shape:
        n *= s
    return torch.frombuffer(bytearray(f.read(4 * n)), dtype=torch.float32).reshape(shape).clone()


class Executor:
    def __init__(self, path: str):
        self.ops = []
        with open(path, "rb") as f:
            if f.read(4) != MAGIC:
                raise ValueError("not a PTMB file")
            _, n = struct.unpack("<II", f.read(8))
            for _ in range(n):
                kind = struct.unpack("<B", f.read(1))[0]
                if kind == 1:
                    w = _rt(f)
                    b = _rt(f) if struct.unpack("<B", f.read(1))[0] else None
                    self.ops.append((kind, w, b))
                else:
                    self.ops.append((kind, None, None))

    @torch.no_grad()
    def run(self, x: torch.Tensor) -> torch.Tensor:
        fns = {2: torch.relu, 3: torch.sigmoid, 4: torch.tanh, 5: torch.nn.functional.gelu, 6: torch.nn.functional.silu,
               7: lambda t: torch.softmax(t, -1)}
        for kind, w, b in self.ops:
            x = torch.nn.functional.linear(x, w, b) if kind == 1 else fns[kind](x)
        return x


MobileExecutor = Executor                  # the reference's names (torch/mobile/executor.h)
export_model = save
