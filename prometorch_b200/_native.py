"""ctypes binding of the native library ``lib/libptb200.so``.

The library is built in-tree by :mod:`prometorch_b200._build`.  On a machine
with a GPU a missing library is an error (there is no PyTorch fallback for the
kernels); on a CPU-only machine ``lib()`` still loads it (the host-side code —
planners, GGUF helpers, servers — works without a device).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

_LIB: Optional[C.CDLL] = None
MAX_PEERS = 8


class NativeError(RuntimeError):
    pass


class WeightDesc(C.Structure):
    _fields_ = [("w", C.c_void_p), ("bias", C.c_void_p), ("qtype", C.c_int), ("rows", C.c_int),
                ("cols", C.c_int), ("rowbytes", C.c_int), ("layout", C.c_int), ("pad", C.c_int)]


class LayerDesc(C.Structure):
    _fields_ = [("q", WeightDesc), ("k", WeightDesc), ("v", WeightDesc), ("o", WeightDesc),
                ("gate", WeightDesc), ("up", WeightDesc), ("down", WeightDesc),
                ("attn_norm", C.c_void_p), ("ffn_norm", C.c_void_p), ("q_norm", C.c_void_p),
                ("k_norm", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
                ("window", C.c_int), ("pad", C.c_int), ("post_attn_norm", C.c_void_p), ("post_ffn_norm", C.c_void_p)]


class ModelDesc(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("hidden", C.c_int), ("n_heads", C.c_int), ("n_kv_heads", C.c_int),
                ("head_dim", C.c_int), ("inter", C.c_int), ("vocab", C.c_int), ("max_seq", C.c_int),
                ("eps", C.c_float), ("emb_scale", C.c_float),
                ("neox", C.c_int), ("act_gelu", C.c_int), ("norm_add_one", C.c_int), ("want_logits", C.c_int),
                ("embed", WeightDesc), ("lm_head", WeightDesc), ("out_norm", C.c_void_p),
                ("tp_rank", C.c_int), ("tp_world", C.c_int), ("vocab_offset", C.c_int), ("pad", C.c_int),
                ("peer_inbox", (C.c_void_p * MAX_PEERS) * 3),
                ("slot_elems", C.c_int), ("pad2", C.c_int)]


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "lib" / "libptb200.so"


def _declare(L: C.CDLL):
    vp, ci, cf, cl = C.c_void_p, C.c_int, C.c_float, C.c_long
    L.ptb_last_error.restype = C.c_char_p
    L.ptb_gemv.argtypes = [vp, vp, ci, ci, ci, ci, ci, vp, vp, cf, vp, vp, vp, ci, ci, ci, vp, vp, vp]
    L.ptb_gemv.restype = ci
    L.ptb_attn_decode.argtypes = [vp] * 14 + [ci, ci, ci, ci, ci, cf, ci, vp]
    L.ptb_attn_decode.restype = ci
    L.ptb_engine_create.argtypes = [C.POINTER(ModelDesc), C.POINTER(LayerDesc), vp]
    L.ptb_engine_create.restype = vp
    L.ptb_engine_destroy.argtypes = [vp]
    L.ptb_engine_destroy.restype = None
    for name in ("ptb_engine_capture", "ptb_engine_sync", "ptb_engine_status"):
        getattr(L, name).argtypes = [vp]
        getattr(L, name).restype = ci
    L.ptb_engine_set_ctrl.argtypes = [vp, ci, ci, ci, ci]
    L.ptb_engine_set_ctrl.restype = ci
    L.ptb_engine_run.argtypes = [vp, ci]
    L.ptb_engine_run.restype = ci
    L.ptb_engine_step.argtypes = [vp, ci, ci]
    L.ptb_engine_step.restype = ci
    L.ptb_engine_begin_script.argtypes = [vp, C.POINTER(ci), ci, ci]
    L.ptb_engine_begin_script.restype = ci
    L.ptb_engine_read_log.argtypes = [vp, C.POINTER(ci), ci]
    L.ptb_engine_read_log.restype = ci
    for name in ("ptb_engine_stream", "ptb_engine_logits", "ptb_engine_hidden", "ptb_engine_result"):
        getattr(L, name).argtypes = [vp]
        getattr(L, name).restype = vp
    L.ptb_engine_enqueue_range.argtypes = [vp, ci, ci]
    L.ptb_engine_enqueue_range.restype = ci
    L.ptb_engine_buffer.argtypes = [vp, ci]
    L.ptb_engine_buffer.restype = vp
    L.ptb_engine_finish_token.argtypes = [vp, vp, ci]
    L.ptb_engine_finish_token.restype = ci
    L.ptb_engine_launches_per_token.argtypes = [vp]
    L.ptb_engine_launches_per_token.restype = cl
    L.ptb_gemv_plan.argtypes = [ci, ci, ci, ci, ci, ci, ci, C.POINTER(ci)]
    L.ptb_gemv_plan.restype = ci
    L.ptb_engine_kv_cache.argtypes = [vp, ci, C.POINTER(vp), C.POINTER(vp)]
    L.ptb_engine_kv_cache.restype = ci
    L.ptb_dequant_weight.argtypes = [vp, ci, ci, ci, ci, vp, vp]
    L.ptb_dequant_weight.restype = ci
    L.ptb_dequant_rows.argtypes = [vp, ci, ci, ci, vp, ci, cf, ci, vp, vp, vp]
    L.ptb_dequant_rows.restype = ci


def lib(build_if_missing: bool = True) -> C.CDLL:
    """Load (building first if needed) the native library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    p = lib_path()
    if not p.exists():
        if not build_if_missing:
            raise NativeError(f"{p} is missing: run `python -m prometorch_b200._build`")
        from ._build import build
        build()
    L = C.CDLL(str(p))
    _declare(L)
    for decl in _EXTRA_DECLS:
        decl(L)
    _LIB = L
    return L


_EXTRA_DECLS = []


def register_decls(fn):
    """Other modules add their own prototypes (called once when the library loads)."""
    _EXTRA_DECLS.append(fn)
    if _LIB is not None:
        fn(_LIB)
    return fn


def check(rc: int, what: str = "native call"):
    if rc != 0:
        msg = lib().ptb_last_error()
        raise NativeError(f"{what}: {msg.decode() if msg else 'failed'}")


def ptr(t) -> int:
    """Device/host address of a tensor (or 0 for None)."""
    return 0 if t is None else t.data_ptr()
