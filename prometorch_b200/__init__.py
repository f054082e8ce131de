"""prometorch_b200 — a Blackwell-native training and inference framework with the public surface of
PromeTorch (``import prometorch_b200 as pt`` or ``import promethorch as pt``).

PyTorch is the tensor/autograd layer; the hot operators are hand-written sm_100a kernels in the
native library ``lib/libptb200.so`` (tcgen05/TMEM GEMM, FlashAttention, fused norms/activations/loss,
multi-tensor optimizers, Q4_K/Q6_K decode engine, peer-memory collectives).  The names exported here
follow python/promethorch/__init__.py:356-460 of the reference."""
from __future__ import annotations

import torch as _torch
from torch import (Tensor, arange, bmm, cat, chunk, clamp, cos, cumsum, device, dot, dtype, einsum, empty, exp, eye, from_numpy,
                   full, gather, isfinite, isinf, isnan, linspace, log, masked_fill, matmul, max, mean, min, mm, multinomial,
                   nan_to_num, norm, ones, ones_like, rand, randint, randn, relu, rsqrt, scatter, sigmoid, sin, softmax, sort, split,
                   sqrt, stack, sum, tanh, tensor, topk, where, zeros, zeros_like)
from torch import bfloat16, bool, float16, float32, float64, int8, int16, int32, int64, uint8  # noqa: F401
from torch import Generator, enable_grad, is_grad_enabled, manual_seed, no_grad, set_grad_enabled  # noqa: F401
from torch.autograd import backward, grad  # noqa: F401
from torch.nn.utils.rnn import pack_padded_sequence, pack_sequence, pad_packed_sequence, pad_sequence  # noqa: F401

__version__ = "0.1.0"

from . import amp, nn, optim  # noqa: E402
from . import autograd, data, distributed, io, ops, parallel, quantization, serve, trainer, utils  # noqa: E402
from . import jit, mlir, mobile, onnx, vision, text, audio  # noqa: E402
from .serialization import load, load_pytorch, load_state_dict, save, save_pytorch, save_state_dict  # noqa: E402
from .jit import compile  # noqa: E402

TensorOptions = dict


def __getattr__(name: str):
    """Every other tensor function or factory (``randn_like``, ``full_like``, ``tril``, ...) is PyTorch's."""
    if name.startswith("__"):
        raise AttributeError(name)
    try:
        return getattr(_torch, name)
    except AttributeError:
        raise AttributeError(f"module 'prometorch_b200' has no attribute '{name}'") from None


class DeviceType:
    CPU, CUDA = "cpu", "cuda"


class cuda:
    """``pt.cuda.is_available()`` / ``device_count()`` / ``synchronize()``."""
    is_available = staticmethod(_torch.cuda.is_available)
    device_count = staticmethod(_torch.cuda.device_count)
    synchronize = staticmethod(_torch.cuda.synchronize)
    current_device = staticmethod(_torch.cuda.current_device)
    set_device = staticmethod(_torch.cuda.set_device)
    empty_cache = staticmethod(_torch.cuda.empty_cache)
    memory_allocated = staticmethod(_torch.cuda.memory_allocated)


def cuda_is_available() -> bool:
    return _torch.cuda.is_available()


def cuda_device_count() -> int:
    return _torch.cuda.device_count()


def mps_is_available() -> bool:
    return False


def _smoke_train():
    """One tiny forward + backward + optimizer step of the Llama-style model on cuda:0 (used by the
    build entry point's smoke test)."""
    from .models.llama import Llama, LlamaConfig
    cfg = LlamaConfig.tiny(hidden_size=256, num_heads=4, num_kv_heads=2, intermediate_size=512, vocab_size=1024, max_seq=128)
    m = Llama(cfg).cuda().bfloat16()
    masters = [nn.Parameter(p.detach().float()) for p in m.parameters()]
    opt = optim.AdamW(masters, lr=1e-3, fused=True)
    tok = _torch.randint(0, 1024, (2, 65), device="cuda")
    loss = m(tok[:, :-1], tok[:, 1:])
    loss.backward()
    for mp, p in zip(masters, m.parameters()):
        opt.set_grad_source(mp, p.grad)
        opt.attach_lowp(mp, p.data)
    opt.step()
    _torch.cuda.synchronize()
    print("smoke train ok: loss", float(loss))
