"""GGUF container: reader (mmap-backed) and writer.

File layout (GGUF v2/v3, little-endian): magic ``GGUF`` (0x46554747), u32
version, u64 tensor count, u64 key/value count, the key/value table (13 value
types), the tensor-info table, padding to ``general.alignment`` (default 32),
then tensor data at the recorded offsets.  Tensor dimensions are stored
innermost-first and are reversed here so ``shape`` reads like a torch shape.
The reference implements the same container in torch/io/gguf_loader.h:96-121
(dimension order), :129-384 (mmap) and :386-693 (reader API).
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Any, Dict, Iterable, List, Optional, Tuple

import numpy as np
import torch

from .gguf_quant import BLOCK_INFO, GGMLType, dequantize, tensor_bytes

GGUF_MAGIC = 0x46554747
DEFAULT_ALIGNMENT = 32

# value type ids
T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)
_SCALAR_FMT = {
    T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i",
    T_F32: "<f", T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d",
}
_NP_FMT = {
    T_U8: np.uint8, T_I8: np.int8, T_U16: np.uint16, T_I16: np.int16, T_U32: np.uint32,
    T_I32: np.int32, T_F32: np.float32, T_BOOL: np.bool_, T_U64: np.uint64, T_I64: np.int64, T_F64: np.float64,
}


@dataclass
class TensorInfo:
    name: str
    shape: Tuple[int, ...]      # torch order (outermost first)
    qtype: GGMLType
    offset: int                 # absolute file offset
    nbytes: int


class GGUFReader:
    """Memory-mapped GGUF file.  ``metadata`` is a plain dict, ``tensors`` maps
    names to :class:`TensorInfo`; raw bytes come back as zero-copy uint8 views."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = memoryview(self._mm)
        self.metadata: Dict[str, Any] = {}
        self.tensors: Dict[str, TensorInfo] = {}
        self._parse()

    # -- low-level cursor helpers
    def _rd(self, fmt: str):
        v = struct.unpack_from(fmt, self._buf, self._pos)[0]
        self._pos += struct.calcsize(fmt)
        return v

    def _rd_str(self) -> str:
        n = self._rd("<Q")
        s = bytes(self._buf[self._pos:self._pos + n]).decode("utf-8", errors="replace")
        self._pos += n
        return s

    def _rd_value(self, vt: int):
        if vt == T_STR:
            return self._rd_str()
        if vt == T_ARR:
            et = self._rd("<I")
            n = self._rd("<Q")
            if et == T_STR:
                return [self._rd_str() for _ in range(n)]
            if et == T_ARR:
                return [self._rd_value(T_ARR) for _ in range(n)]
            dt = np.dtype(_NP_FMT[et])
            arr = np.frombuffer(self._buf, dtype=dt, count=n, offset=self._pos)
            self._pos += n * dt.itemsize
            return arr.tolist() if n <= 64 else arr
        if vt not in _SCALAR_FMT:
            raise ValueError(f"GGUF: unknown value type {vt}")
        return self._rd(_SCALAR_FMT[vt])

    def _parse(self):
        self._pos = 0
        magic = self._rd("<I")
        if magic != GGUF_MAGIC:
            raise ValueError(f"{self.path}: not a GGUF file (magic {magic:#x})")
        self.version = self._rd("<I")
        if self.version not in (2, 3):
            raise ValueError(f"GGUF version {self.version} not supported")
        n_tensors = self._rd("<Q")
        n_kv = self._rd("<Q")
        for _ in range(n_kv):
            key = self._rd_str()
            vt = self._rd("<I")
            self.metadata[key] = self._rd_value(vt)
        infos = []
        for _ in range(n_tensors):
            name = self._rd_str()
            nd = self._rd("<I")
            dims = [self._rd("<Q") for _ in range(nd)]
            qt = GGMLType(self._rd("<I"))
            off = self._rd("<Q")
            infos.append((name, tuple(reversed(dims)), qt, off))
        self.alignment = int(self.metadata.get("general.alignment", DEFAULT_ALIGNMENT))
        self.data_start = (self._pos + self.alignment - 1) // self.alignment * self.alignment
        for name, shape, qt, off in infos:
            self.tensors[name] = TensorInfo(name, shape, qt, self.data_start + off, tensor_bytes(qt, shape))

    # -- public API
    def get(self, key: str, default=None):
        return self.metadata.get(key, default)

    def arch(self) -> str:
        return self.metadata.get("general.architecture", "llama")

    def get_arch(self, suffix: str, default=None):
        """``<arch>.<suffix>`` lookup, e.g. ``get_arch('embedding_length')``."""
        return self.metadata.get(f"{self.arch()}.{suffix}", default)

    def has_tensor(self, name: str) -> bool:
        return name in self.tensors

    def raw(self, name: str) -> torch.Tensor:
        """Zero-copy uint8 view ``[rows..., row_bytes]`` over the mapped file."""
        ti = self.tensors[name]
        arr = np.frombuffer(self._buf, dtype=np.uint8, count=ti.nbytes, offset=ti.offset)
        t = torch.from_numpy(arr)
        lead = ti.shape[:-1]
        return t.reshape(*lead, -1) if lead else t

    def load(self, name: str, device="cpu") -> torch.Tensor:
        """Dequantised fp32 tensor."""
        ti = self.tensors[name]
        raw = self.raw(name).to(device)
        return dequantize(raw, ti.qtype, ti.shape[-1]).reshape(ti.shape)

    def close(self):
        self._buf.release()
        self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class GGUFWriter:
    """Streams a GGUF v3 file: metadata first, then tensors in insertion order."""

    def __init__(self, path: str, alignment: int = DEFAULT_ALIGNMENT):
        self.path = path
        self.alignment = alignment
        self._kv: List[Tuple[str, int, Any, Optional[int]]] = []
        self._tensors: List[Tuple[str, Tuple[int, ...], GGMLType, Any]] = []

    def add(self, key: str, value, vtype: Optional[int] = None, elem_type: Optional[int] = None):
        if vtype is None:
            if isinstance(value, bool):
                vtype = T_BOOL
            elif isinstance(value, int):
                vtype = T_U32 if 0 <= value < 2**32 else T_I64
            elif isinstance(value, float):
                vtype = T_F32
            elif isinstance(value, str):
                vtype = T_STR
            elif isinstance(value, (list, tuple, np.ndarray)):
                vtype = T_ARR
                if elem_type is None:
                    first = value[0] if len(value) else 0
                    elem_type = T_STR if isinstance(first, str) else (T_F32 if isinstance(first, float) else T_I32)
            else:
                raise TypeError(f"GGUFWriter.add: unsupported value {type(value)}")
        self._kv.append((key, vtype, value, elem_type))

    def add_tensor(self, name: str, shape: Iterable[int], qtype: GGMLType, data):
        """``data``: uint8 tensor/ndarray of raw block bytes, or a zero-argument
        callable returning one (lets a large model be produced tensor by tensor)."""
        self._tensors.append((name, tuple(int(s) for s in shape), GGMLType(qtype), data))

    @staticmethod
    def _wstr(f, s: str):
        b = s.encode("utf-8")
        f.write(struct.pack("<Q", len(b)))
        f.write(b)

    def _wvalue(self, f, vtype, value, elem_type):
        if vtype == T_STR:
            self._wstr(f, value)
        elif vtype == T_ARR:
            f.write(struct.pack("<IQ", elem_type, len(value)))
            if elem_type == T_STR:
                for s in value:
                    self._wstr(f, s)
            else:
                f.write(np.asarray(value, dtype=_NP_FMT[elem_type]).tobytes())
        else:
            f.write(struct.pack(_SCALAR_FMT[vtype], value))

    def write(self):
        al = self.alignment
        offsets, off = [], 0
        for _, shape, qt, _ in self._tensors:
            offsets.append(off)
            off += (tensor_bytes(qt, shape) + al - 1) // al * al
        with open(self.path, "wb") as f:
            f.write(struct.pack("<IIQQ", GGUF_MAGIC, 3, len(self._tensors), len(self._kv)))
            for key, vt, val, et in self._kv:
                self._wstr(f, key)
                f.write(struct.pack("<I", vt))
                self._wvalue(f, vt, val, et)
            for (name, shape, qt, _), o in zip(self._tensors, offsets):
                self._wstr(f, name)
                f.write(struct.pack("<I", len(shape)))
                for dim in reversed(shape):
                    f.write(struct.pack("<Q", dim))
                f.write(struct.pack("<IQ", int(qt), o))
            pos = f.tell()
            f.write(b"\0" * ((pos + al - 1) // al * al - pos))
            for (name, shape, qt, data), o in zip(self._tensors, offsets):
                if callable(data):
                    data = data()
                if isinstance(data, torch.Tensor):
                    data = data.detach().cpu().contiguous().view(torch.uint8).numpy()
                data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
                want = tensor_bytes(qt, shape)
                if data.size != want:
                    raise ValueError(f"{name}: {data.size} bytes given, {want} expected for {qt.name}{list(shape)}")
                f.write(data.tobytes() if data.size < (1 << 20) else memoryview(data))
                f.write(b"\0" * ((want + al - 1) // al * al - want))
        return self.path
