"""``compile`` / ``trace``: capture instead of code generation.

The reference's JIT traces element-wise chains and emits C++ through a subprocess compiler, and its
"PromePile" flattens Sequential MLPs and the LLM decode step (torch/jit/*.h, torch/compile/*.h).  On a B200
the launch-bound inner loops are captured as CUDA graphs: ``compile(module)`` returns a ``CompiledModule``
that records one forward per input signature into a graph (static buffers, replay on later calls); on CPU it
returns the module unchanged.  The decode engine captures its own per-token graph natively."""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.nn as nn


class CompiledModule(nn.Module):
    def __init__(self, module: nn.Module, warmup: int = 2):
        super().__init__()
        self.module, self.warmup = module, warmup
        self._graphs: Dict[Tuple, Tuple] = {}

    def forward(self, *args):
        if not args or not all(torch.is_tensor(a) and a.is_cuda for a in args) or torch.is_grad_enabled() and any(
                p.requires_grad for p in self.module.parameters()):
            return self.module(*args)
        key = tuple((tuple(a.shape), a.dtype) for a in args)
        ent = self._graphs.get(key)
        if ent is None:
            static_in = [a.clone() for a in args]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s), torch.no_grad():
                for _ in range(self.warmup):
                    self.module(*static_in)
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g), torch.no_grad():
                static_out = self.module(*static_in)
            ent = self._graphs[key] = (g, static_in, static_out)
        g, static_in, static_out = ent
        for d, a in zip(static_in, args):
            d.copy_(a)
        g.replay()
        return static_out.clone() if torch.is_tensor(static_out) else static_out


def compile(module, **kw):
    """Graph-capturing wrapper for inference modules (see :class:`CompiledModule`)."""
    if isinstance(module, nn.Module):
        return CompiledModule(module)
    return module


def trace(fn, example_inputs):
    return torch.jit.trace(fn, example_inputs)


def script(fn):
    return torch.jit.script(fn)


CompiledFn = CompiledModule                # the reference's name for what compile() returns


def tracing_active() -> bool:
    """Whether a CUDA-graph capture is in progress on the current stream (the recorder state of the reference's tracer)."""
    return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()


# ---------------------------------------------------------------------------------------------- the PromePile entry points (torch/compile/promepile.h)
CompiledForward = CompiledModule


def promepile(module: nn.Module) -> CompiledModule:
    """The reference flattens a model into one compiled forward; here the forward is captured as a CUDA graph per input
    signature (eager on CPU)."""
    return CompiledModule(module)


class CompiledTrainingStep:
    """One call = one optimisation step: zero the gradients, forward, loss, backward, (optional) gradient clipping, optimizer
    step; returns the loss as a detached tensor, so a caller that does not read it never waits for the device.  The kernels
    behind it are the fused ones of this package (multi-tensor optimizer, fused clip); the step itself is not re-traced."""

    def __init__(self, model: nn.Module, optimizer, loss_fn, max_grad_norm: float = 0.0, scaler=None):
        self.model, self.optimizer, self.loss_fn, self.max_grad_norm, self.scaler = model, optimizer, loss_fn, max_grad_norm, scaler
        self.steps = 0

    def __call__(self, *inputs, target=None):
        self.optimizer.zero_grad(set_to_none=True)
        out = self.model(*inputs)
        loss = self.loss_fn(out, target) if target is not None else self.loss_fn(out)
        (self.scaler.scale(loss) if self.scaler is not None else loss).backward()
        if self.scaler is not None:
            self.scaler.unscale(self.optimizer)
        if self.max_grad_norm > 0:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.max_grad_norm)
        if self.scaler is not None:
            self.scaler.step(self.optimizer)
            self.scaler.update()
        else:
            self.optimizer.step()
        self.steps += 1
        return loss.detach()


def promepile_train(model: nn.Module, optimizer, loss_fn, max_grad_norm: float = 0.0, scaler=None) -> CompiledTrainingStep:
    return CompiledTrainingStep(model, optimizer, loss_fn, max_grad_norm, scaler)


class CompiledDecodeStep:
    """The decode step of a GGUF model as one captured CUDA graph per token: ``step(token, pos)`` returns the next id.  The
    capture is the decode engine's own (``GGUFModel.capture``); this class only gives it the reference's name and call shape."""

    def __init__(self, model):
        self.model = model
        if hasattr(model, "capture"):
            model.capture()

    def __call__(self, token: int, pos: int) -> int:
        return self.model.forward_decode(int(token), int(pos))
