"""B200-specific parallel runtime: symmetric peer memory and the fused FSDP engine.  (Tensor-parallel
layers and pipelines live in :mod:`prometorch_b200.nn.parallel`; DDP/FSDP front ends in
:mod:`prometorch_b200.distributed`.)"""
