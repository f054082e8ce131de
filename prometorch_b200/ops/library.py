"""The package's kernels as dispatcher ops: ``torch.ops.ptb200.<name>``.

The reference routes its CUDA wrappers through a dispatch header that allocates outputs and launches on the default
stream (aten/src/ATen/cuda/CUDADispatch.h:213-1136).  Here the launchers are registered with PyTorch's dispatcher under
the ``ptb200`` namespace, so they can be called by schema from Python, from TorchScript-free C++ (``c10::Dispatcher``)
and show up by name in profiler traces.  Each op is registered as a composite: its implementation is the wrapper in
``ops/`` whose ``autograd.Function`` carries the hand-written backward kernel, so gradients flow through an op call as
they do through the Python function, and on a CPU tensor the wrapper's plain-math path answers.
"""
from __future__ import annotations

import torch

_LIB = None

SCHEMAS = {
    "linear": "(Tensor x, Tensor weight, Tensor? bias=None) -> Tensor",
    "rms_norm": "(Tensor x, Tensor weight, float eps=1e-6) -> Tensor",
    "add_rms_norm": "(Tensor x, Tensor resid, Tensor weight, float eps=1e-6) -> (Tensor, Tensor)",
    "rope": "(Tensor x, Tensor cos, Tensor sin, bool neox=True, int pos_offset=0) -> Tensor",
    "swiglu": "(Tensor gate_up, bool gelu=False) -> Tensor",
    "cross_entropy": "(Tensor logits, Tensor target, int ignore_index=-100) -> Tensor",
    "flash_attention": "(Tensor q, Tensor k, Tensor v, bool causal=True, int q_offset=0, float? scale=None) -> Tensor",
    "linear_swiglu": "(Tensor x, Tensor w_gate_up, bool gelu=False) -> Tensor",
}


def register() -> "torch.library.Library":
    """Define and implement the ops once per process; returns the library handle."""
    global _LIB
    if _LIB is not None:
        return _LIB
    from . import attention, fused_ops, gemm
    lib = torch.library.Library("ptb200", "DEF")
    impls = {
        "linear": gemm.linear,
        "rms_norm": fused_ops.rms_norm,
        "add_rms_norm": fused_ops.add_rms_norm,
        "rope": fused_ops.rope,
        "swiglu": fused_ops.swiglu,
        "cross_entropy": lambda logits, target, ignore_index=-100: fused_ops.cross_entropy(logits, target, ignore_index),
        "flash_attention": lambda q, k, v, causal=True, q_offset=0, scale=None: attention.flash_attention(q, k, v, causal, q_offset, scale),
        "linear_swiglu": gemm.linear_swiglu,
    }
    for name, schema in SCHEMAS.items():
        lib.define(name + schema)
        lib.impl(name, impls[name], "CompositeImplicitAutograd")
    _LIB = lib
    return lib
