"""ONNX export.  ``export(model, args, path)`` uses PyTorch's exporter when its dependencies are present and
otherwise writes the MLP subset (Linear/ReLU/Sigmoid/Tanh/Softmax chains) with a hand-rolled protobuf writer,
which is the subset the reference's own exporter covers (torch/onnx/export.h)."""
from __future__ import annotations

import struct

import torch
import torch.nn as nn


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field(num: int, wt: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wt) + (_varint(len(payload)) + payload if wt == 2 else payload)


def _str(num, s):
    return _field(num, 2, s.encode())


def _tensor(name, t: torch.Tensor) -> bytes:
    t = t.detach().float().contiguous().cpu()
    b = b"".join(_field(1, 0, _varint(d)) for d in t.shape) + _field(2, 0, _varint(1)) + _str(8, name) + _field(9, 2, t.numpy().tobytes())
    return b


def _value_info(name, shape) -> bytes:
    dims = b"".join(_field(1, 2, _field(1, 0, _varint(d))) for d in shape)
    ttype = _field(1, 0, _varint(1)) + _field(2, 2, dims)
    return _str(1, name) + _field(2, 2, _field(1, 2, ttype))


def _node(op, ins, outs, attrs=b"") -> bytes:
    return b"".join(_str(1, i) for i in ins) + b"".join(_str(2, o) for o in outs) + _str(4, op) + attrs


def export_mlp(model: nn.Module, input_shape, path: str, opset: int = 13):
    nodes, inits, cur, k = [], [], "input", 0
    shape = list(input_shape)
    for m in model.modules():
        if isinstance(m, nn.Linear):
            w, b, out = f"w{k}", f"b{k}", f"h{k}"
            inits += [_tensor(w, m.weight.t()), _tensor(b, m.bias if m.bias is not None else torch.zeros(m.out_features))]
            nodes.append(_node("Gemm", [cur, w, b], [out]))
            cur, shape, k = out, shape[:-1] + [m.out_features], k + 1
        elif isinstance(m, (nn.ReLU, nn.Sigmoid, nn.Tanh)):
            out = f"a{k}"
            nodes.append(_node(type(m).__name__.replace("ReLU", "Relu"), [cur], [out]))
            cur, k = out, k + 1
        elif isinstance(m, nn.Softmax):
            out = f"a{k}"
            nodes.append(_node("Softmax", [cur], [out]))
            cur, k = out, k + 1
    graph = b"".join(_field(1, 2, n) for n in nodes) + _str(2, "prometorch_b200") + b"".join(_field(5, 2, t) for t in inits) + \
        _field(11, 2, _value_info("input", input_shape)) + _field(12, 2, _value_info(cur, shape))
    model_pb = _field(1, 0, _varint(8)) + _str(2, "prometorch_b200") + _field(7, 2, graph) + _field(8, 2, _str(1, "") + _field(2, 0, _varint(opset)))
    with open(path, "wb") as f:
        f.write(model_pb)
    return path


def export(model: nn.Module, args, path: str, **kw):
    try:
        torch.onnx.export(model, args, path, **kw)
        return path
    except Exception:
        shape = list(args.shape if torch.is_tensor(args) else args[0].shape)
        return export_mlp(model, shape, path)


def export_model(model: nn.Module, input_shape, path: str, opset: int = 13):
    """The reference's entry point (torch/onnx/export.h): ``export_model(model, input shape, path)``."""
    return export(model, torch.zeros(*input_shape), path, opset_version=opset) if not _is_chain(model) else export_mlp(model, list(input_shape), path, opset)


def _is_chain(model: nn.Module) -> bool:
    leaves = [m for m in model.modules() if not list(m.children())]
    return all(isinstance(m, (nn.Linear, nn.ReLU, nn.Sigmoid, nn.Tanh, nn.Softmax, nn.Identity, nn.Flatten, nn.Dropout)) for m in leaves)
