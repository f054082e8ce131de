"""Autograd surface: custom functions, hooks, anomaly mode, checkpointing, forward-mode AD and vmap.

PyTorch's engine does the graph walk the reference implements in torch/csrc/autograd/engine.h; the
names below are the reference's (``Function``/``FunctionCtx``, ``AnomalyGuard``, ``NoGradGuard``,
``checkpoint``/``checkpoint_sequential``, ``forward_ad.make_dual/unpack_dual/jvp``, ``vmap``)."""
import torch
from torch.autograd import Function, backward, grad
from torch.autograd.function import FunctionCtx
from torch.autograd import forward_ad
from torch.func import jvp, vjp, vmap
from torch.utils.checkpoint import checkpoint as _checkpoint, checkpoint_sequential as _checkpoint_sequential

no_grad, enable_grad, set_grad_enabled, is_grad_enabled = torch.no_grad, torch.enable_grad, torch.set_grad_enabled, torch.is_grad_enabled
NoGradGuard = torch.no_grad
set_detect_anomaly, detect_anomaly = torch.autograd.set_detect_anomaly, torch.autograd.detect_anomaly
AnomalyGuard = torch.autograd.detect_anomaly


class AnomalyMode:
    @staticmethod
    def is_enabled():
        return torch.is_anomaly_enabled()

    @staticmethod
    def set_enabled(v: bool):
        torch.autograd.set_detect_anomaly(bool(v))


def checkpoint(fn, *args, **kw):
    """Recompute ``fn`` in backward instead of storing its activations (torch/utils/checkpoint.h:24-200)."""
    kw.setdefault("use_reentrant", False)
    return _checkpoint(fn, *args, **kw)


def checkpoint_sequential(functions, segments, input, **kw):
    kw.setdefault("use_reentrant", False)
    return _checkpoint_sequential(functions, segments, input, **kw)


def register_hook(tensor, fn):
    """Gradient hook on a tensor; returns a removable handle (torch/csrc/autograd/hooks.h:43-62)."""
    return tensor.register_hook(fn)
