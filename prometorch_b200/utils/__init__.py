"""Utilities: profiling (CUDA-event section timers, NVTX ranges), JSONL metrics, environment registry."""
from .profiler import InferenceProfiler, ScopedTimer, Timer, nvtx_range
from .metrics import MetricsWriter
from .env import ENV, env_flag, env_int, env_str
from torch.utils.checkpoint import checkpoint, checkpoint_sequential  # noqa: F401
