"""Optimizers (16), LR schedulers (16), EMA and gradient utilities."""
from .optimizers import *  # noqa: F401,F403
from .optimizers import Optimizer, ParamGroup
from . import lr_scheduler
from .lr_scheduler import *  # noqa: F401,F403
from .grad_utils import clip_grad_norm_, clip_grad_value_, GradNormClipper
