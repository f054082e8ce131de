"""B200-specific parallel runtime: symmetric peer memory and the fused FSDP engine.  (Tensor-parallel
layers and pipelines live in :mod:`prometorch_b200.nn.parallel`; DDP/FSDP front ends in
:mod:`prometorch_b200.distributed`.)"""


_LAZY = {"FusedFSDP": "fsdp_fused", "ShardedLinear": "fsdp_fused", "WindowPool": "fsdp_fused", "SymmGroup": "symm"}


def __getattr__(name):
    """``parallel.FusedFSDP`` / ``ShardedLinear`` / ``WindowPool`` / ``SymmGroup`` without importing them at package import."""
    if name in _LAZY:
        import importlib
        return getattr(importlib.import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
