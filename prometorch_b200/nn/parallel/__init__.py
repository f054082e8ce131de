"""Model parallelism: tensor-parallel linear layers and pipelines."""
from torch.nn.parallel import DataParallel  # noqa: F401  (kept importable from the same place as in torch)

from .tensor_parallel import (ColumnParallelLinear, RowParallelLinear, TPConfig, tp_all_gather, tp_all_reduce_sum, tp_barrier)
from .pipeline import Pipeline, Pipeline1F1BStage, PipelineScheduleConfig
from ...distributed.ddp import DistributedDataParallel
from .context_parallel import ring_attention, shard_sequence  # noqa: E402,F401
from .expert_parallel import Expert, ExpertParallelMoE  # noqa: E402,F401
