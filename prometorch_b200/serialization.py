"""Checkpoint I/O.

* ``save`` / ``load`` / ``save_state_dict`` / ``load_state_dict``: the PTOR container
  (``"PTOR"``, u32 version 1, u64 count, then per tensor: u32 name length, name, u8 dtype code, u32
  ndim, i64 sizes, u64 nbytes, raw little-endian data; torch/serialization.h:17-197), byte-compatible
  with files the reference writes.
* ``save_pytorch`` / ``load_pytorch``: PyTorch ``.pt`` zip checkpoints.  Loading is restricted to
  tensors and plain containers (``weights_only``), the same policy as the reference's unpickler
  white-list (torch/serialization_pytorch.h:734-878).
"""
from __future__ import annotations

import io
import struct
from collections import OrderedDict
from typing import Dict, Union

import numpy as np
import torch

MAGIC = b"PTOR"
VERSION = 1

# dtype codes of the container (c10/core/ScalarType.h:540-569)
_CODE = {torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4, torch.float16: 5,
         torch.float32: 6, torch.float64: 7, torch.complex64: 9, torch.complex128: 10, torch.bool: 11,
         torch.bfloat16: 12, torch.float8_e4m3fn: 17, torch.float8_e5m2: 18}
_DTYPE = {v: k for k, v in _CODE.items()}


def _write_tensor(f, name: str, t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    nb = name.encode("utf-8")
    f.write(struct.pack("<I", len(nb)))
    f.write(nb)
    f.write(struct.pack("<B", _CODE[t.dtype]))
    f.write(struct.pack("<I", t.dim()))
    for s in t.shape:
        f.write(struct.pack("<q", s))
    raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
    f.write(struct.pack("<Q", len(raw)))
    f.write(raw)


def _read_exact(f, n):
    b = f.read(n)
    if len(b) != n:
        raise RuntimeError("serialization: read failed (unexpected EOF)")
    return b


def _read_tensor(f):
    (nl,) = struct.unpack("<I", _read_exact(f, 4))
    name = _read_exact(f, nl).decode("utf-8")
    (code,) = struct.unpack("<B", _read_exact(f, 1))
    (nd,) = struct.unpack("<I", _read_exact(f, 4))
    sizes = [struct.unpack("<q", _read_exact(f, 8))[0] for _ in range(nd)]
    (nbytes,) = struct.unpack("<Q", _read_exact(f, 8))
    if code not in _DTYPE:
        raise RuntimeError(f"serialization: unknown dtype code {code}")
    dt = _DTYPE[code]
    t = torch.empty(sizes, dtype=dt)
    if nbytes != t.numel() * t.element_size():
        raise RuntimeError("serialization: nbytes mismatch")
    if nbytes:
        raw = np.frombuffer(_read_exact(f, nbytes), dtype=np.uint8).copy()
        t = torch.from_numpy(raw).view(dt).reshape(sizes)
    return name, t


def _header(f, count):
    f.write(MAGIC)
    f.write(struct.pack("<I", VERSION))
    f.write(struct.pack("<Q", count))


def _check_header(f, what):
    if _read_exact(f, 4) != MAGIC:
        raise RuntimeError(f"{what}: invalid file format (bad magic)")
    (v,) = struct.unpack("<I", _read_exact(f, 4))
    if v != VERSION:
        raise RuntimeError(f"{what}: unsupported format version")
    return struct.unpack("<Q", _read_exact(f, 8))[0]


def save(obj: Union[torch.Tensor, Dict[str, torch.Tensor]], path: str):
    """A single tensor (stored under the name ``tensor``) or a state dict."""
    if torch.is_tensor(obj):
        with open(path, "wb") as f:
            _header(f, 1)
            _write_tensor(f, "tensor", obj)
    else:
        save_state_dict(obj, path)


def load(path: str):
    with open(path, "rb") as f:
        n = _check_header(f, "load")
        items = [_read_tensor(f) for _ in range(n)]
    if n == 1 and items[0][0] == "tensor":
        return items[0][1]
    return OrderedDict(items)


def save_state_dict(state_dict: Dict[str, torch.Tensor], path: str):
    with open(path, "wb") as f:
        _header(f, len(state_dict))
        for k, v in state_dict.items():
            _write_tensor(f, k, v if torch.is_tensor(v) else torch.as_tensor(v))


def load_state_dict(path: str) -> "OrderedDict[str, torch.Tensor]":
    with open(path, "rb") as f:
        n = _check_header(f, "load_state_dict")
        return OrderedDict(_read_tensor(f) for _ in range(n))


def save_pytorch(obj, path: str):
    """Write a checkpoint ``torch.load`` (any PyTorch) can read."""
    torch.save(obj, path)


def load_pytorch(path: str, map_location="cpu"):
    """Read a PyTorch ``.pt``/``.pth`` checkpoint; only tensors and plain containers are accepted."""
    # libtorch's C++ pickler wraps dictionaries in torch.jit._pickle.restore_type_tag(value, type string), which returns the
    # value unchanged; allowing that one function lets files written by the C++ API (save_pytorch) load under the same
    # tensors-and-plain-containers policy
    from torch.jit._pickle import restore_type_tag
    with torch.serialization.safe_globals([restore_type_tag]):
        return torch.load(path, map_location=map_location, weights_only=True)
