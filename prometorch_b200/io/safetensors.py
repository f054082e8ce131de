"""``.safetensors`` reader and writer without the ``safetensors`` package.

File layout: 8-byte little-endian header length, a JSON header (``name -> {dtype, shape, data_offsets}``), then the
raw little-endian tensor bytes.  ``SafeTensorsFile`` maps the file and materialises one tensor at a time, so a
sharded checkpoint never sits in memory twice (python/promethorch/safetensors_reader.py:67-175 is the
reference's reader; it returns numpy arrays, this one returns torch tensors and also writes).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterator, List, Optional

import numpy as np
import torch

_DTYPES = {"F64": (torch.float64, np.float64), "F32": (torch.float32, np.float32), "F16": (torch.float16, np.float16),
           "BF16": (torch.bfloat16, np.uint16), "I64": (torch.int64, np.int64), "I32": (torch.int32, np.int32),
           "I16": (torch.int16, np.int16), "I8": (torch.int8, np.int8), "U8": (torch.uint8, np.uint8), "BOOL": (torch.bool, np.bool_)}
_NAMES = {t: n for n, (t, _) in _DTYPES.items()}


class SafeTensorsFile:
    """``with SafeTensorsFile(path) as f: f.keys(); f.get_tensor(name)``."""

    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > os.path.getsize(path) - 8:
            self._fh.close()
            raise ValueError(f"{path}: header length {n} exceeds the file")
        header = json.loads(self._fh.read(n))
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self._header: Dict[str, dict] = header
        self._base = 8 + n
        size = os.path.getsize(path)
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def __enter__(self) -> "SafeTensorsFile":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.close()

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        if self._fh is not None:
            self._fh.close()
            self._fh = None

    def keys(self) -> Iterator[str]:
        return iter(self._header.keys())

    def __contains__(self, name: str) -> bool:
        return name in self._header

    def __len__(self) -> int:
        return len(self._header)

    def info(self, name: str) -> dict:
        return dict(self._header[name])

    def get_tensor(self, name: str) -> torch.Tensor:
        meta = self._header[name]
        if meta["dtype"] not in _DTYPES:
            raise TypeError(f"{self.path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        tdt, ndt = _DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        count = int(np.prod(meta["shape"])) if meta["shape"] else 1
        if hi - lo != count * np.dtype(ndt).itemsize:
            raise ValueError(f"{self.path}: tensor {name!r} spans {hi - lo} bytes, its shape needs {count * np.dtype(ndt).itemsize}")
        arr = np.frombuffer(self._mm, dtype=ndt, count=count, offset=self._base + lo).reshape(meta["shape"]).copy()
        t = torch.from_numpy(arr)
        return t.view(torch.bfloat16) if tdt == torch.bfloat16 else t


def load_file(path: str) -> Dict[str, torch.Tensor]:
    with SafeTensorsFile(path) as f:
        return {k: f.get_tensor(k) for k in f.keys()}


def load_index(index_json_path: str) -> Dict[str, torch.Tensor]:
    """Every tensor of a sharded checkpoint described by ``model.safetensors.index.json``."""
    with open(index_json_path, encoding="utf-8") as fp:
        weight_map = json.load(fp)["weight_map"]
    base = os.path.dirname(os.path.abspath(index_json_path))
    out: Dict[str, torch.Tensor] = {}
    for shard in sorted(set(weight_map.values())):
        with SafeTensorsFile(os.path.join(base, shard)) as f:
            for k in f.keys():
                if weight_map.get(k, shard) == shard:
                    out[k] = f.get_tensor(k)
    return out


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None):
    header: Dict[str, dict] = {}
    blobs: List[bytes] = []
    off = 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise TypeError(f"save_file: dtype {t.dtype} of {name!r} has no safetensors name")
        b = (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def load_checkpoint_dir(model_dir: str) -> Dict[str, torch.Tensor]:
    """``model.safetensors``, else the shards of ``model.safetensors.index.json``, else ``pytorch_model.bin`` through the
    restricted ``.pt`` reader; an empty dict when the directory holds no weights."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    legacy = os.path.join(model_dir, "pytorch_model.bin")
    if os.path.exists(single):
        return load_file(single)
    if os.path.exists(index):
        return load_index(index)
    if os.path.exists(legacy):
        from ..serialization import load_pytorch
        sd = load_pytorch(legacy)
        return dict(sd.get("state_dict", sd)) if isinstance(sd, dict) else {}
    return {}
