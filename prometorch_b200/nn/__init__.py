"""``nn``: the module system and layers.

``torch.nn`` provides the Module base (named parameters/buffers/submodules, ``state_dict``,
``to``, ``train/eval``, forward pre/post hooks, backward hooks) and the standard layers; everything
the reference lists in torch/nn/modules/*.h is importable from here under the same name.  Added on
top: the layers the reference has and PyTorch lacks (``LowRankLinear``, ``FocalLoss``, ``DiceLoss``,
``GlobalAvgPool2d``, ``PositionalEncoding``, ``QuantizedLinear``, ``QuantizedConv2d``) and the fused
sm_100a building blocks (``FusedRMSNorm``, ``FusedSwiGLU``, ``FusedCrossEntropyLoss``,
``FlashSelfAttention``) used by the model zoo."""
from torch.nn import *  # noqa: F401,F403
from torch.nn import Module, Parameter, functional, init, utils  # noqa: F401
from torch.nn import parameter, modules  # noqa: F401

from .extras import (DiceLoss, FocalLoss, GlobalAvgPool2d, LowRankLinear, PositionalEncoding, QuantizedConv2d,
                     QuantizedLinear, num_parameters)
from .fused import FlashSelfAttention, FusedCrossEntropyLoss, FusedRMSNorm, FusedSwiGLU
import importlib as _importlib

parallel = _importlib.import_module(__name__ + ".parallel")     # our package, not torch.nn.parallel from the star import

F = functional
