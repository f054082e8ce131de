"""Sharded checkpoints: one file per rank plus a manifest, readable by a run with a different number of ranks.

The reference saves whole-model ``.ptor`` files only and has no sharded format (torch/serialization.h:113-197,
torch/trainer/trainer.h); a ZeRO-3 job whose parameters never exist in one place needs one.  Layout of a directory::

    manifest.json            format tag, world size, per-parameter (name, shape, numel, shard length, dtype), optimizer
                             hyper-parameters and state keys, and the caller's ``extra`` (epoch, step, scheduler, RNG ...)
    rank00000.safetensors    this rank's flat shard of every parameter ("shard.<i>") and the optimizer state of those shards
    rank00001.safetensors    ...

Every rank calls :func:`save_sharded` / :func:`load_sharded`.  Loading with the writer's world size copies the rank's own
file; with another world size each rank reads the pieces it needs from all files and re-cuts them (flat shards are
element-wise, so parameters and their optimizer state re-shard the same way).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from ..io.safetensors import SafeTensorsFile, save_file

FORMAT = "ptb-sharded-1"


def _rank_file(directory: str, rank: int) -> str:
    return os.path.join(directory, f"rank{rank:05d}.safetensors")


def _opt_state_tensors(optimizer, shards) -> Dict[str, torch.Tensor]:
    """Tensor state of the optimizer keyed ``opt.<shard index>.<key>``; scalars (step counts) become 0-dim tensors."""
    out: Dict[str, torch.Tensor] = {}
    inner = getattr(optimizer, "inner", optimizer)
    state = getattr(inner, "state", {})
    for i, p in enumerate(shards):
        for k, v in (state.get(p) or {}).items():
            if torch.is_tensor(v):
                out[f"opt.{i}.{k}"] = v.detach().cpu()
            elif isinstance(v, (int, float)):
                out[f"opt.{i}.{k}"] = torch.tensor(float(v), dtype=torch.float64)
    return out


def save_sharded(directory: str, fsdp, optimizer=None, extra: Optional[dict] = None):
    """Write this rank's shards (and the optimizer state of those shards); rank 0 also writes the manifest."""
    os.makedirs(directory, exist_ok=True)
    shards = fsdp.local_shards()
    tensors = {f"shard.{i}": s.data.detach().cpu() for i, s in enumerate(shards)}
    if optimizer is not None:
        tensors.update(_opt_state_tensors(optimizer, shards))
    tmp = _rank_file(directory, fsdp.rank) + ".tmp"
    save_file(tensors, tmp, metadata={"rank": str(fsdp.rank), "world": str(fsdp.world)})
    os.replace(tmp, _rank_file(directory, fsdp.rank))
    if fsdp.rank == 0:
        names = [n for n, _ in fsdp.module.named_parameters()]
        inner = getattr(optimizer, "inner", optimizer)
        groups = []
        for g in getattr(inner, "param_groups", []) if optimizer is not None else []:
            groups.append({k: v for k, v in g.items() if k != "params" and isinstance(v, (int, float, bool, str, list, tuple))})
        manifest = {"format": FORMAT, "world_size": fsdp.world,
                    "params": [{"name": n, "shape": list(sh), "numel": int(ne), "shard_len": int(sl), "dtype": str(p.dtype).replace("torch.", "")}
                               for n, sh, ne, sl, p in zip(names, fsdp._shapes, fsdp._numels, fsdp._shard_len, shards)],
                    "optimizer": {"param_groups": groups}, "extra": extra or {}}
        with open(os.path.join(directory, "manifest.json.tmp"), "w") as f:
            json.dump(manifest, f, indent=1)
        os.replace(os.path.join(directory, "manifest.json.tmp"), os.path.join(directory, "manifest.json"))
    fsdp.pg.barrier()


def _recut(files: List[SafeTensorsFile], key: str, numel: int, new_len: int, new_rank: int) -> Optional[torch.Tensor]:
    """Elements [new_rank*new_len, (new_rank+1)*new_len) of the flat tensor whose old shards are ``key`` in ``files``."""
    if key not in files[0]:
        return None
    first = files[0].get_tensor(key)
    if first.dim() == 0:                                   # a scalar (step count): the same on every rank
        return first
    old_len = first.numel()
    lo, hi = new_rank * new_len, (new_rank + 1) * new_len
    out = torch.zeros(new_len, dtype=first.dtype)
    for r in range(lo // old_len, min(len(files), (hi - 1) // old_len + 1)):
        piece = first if r == 0 else files[r].get_tensor(key)
        a, b = max(lo, r * old_len), min(hi, (r + 1) * old_len)
        out[a - lo:b - lo] = piece.reshape(-1)[a - r * old_len:b - r * old_len]
    valid = max(0, min(hi, numel) - lo)                    # what lies past the parameter's end is padding
    out[valid:] = 0
    return out


def load_sharded(directory: str, fsdp, optimizer=None) -> dict:
    """Restore shards (and optimizer state) written by :func:`save_sharded`; returns the manifest's ``extra``."""
    with open(os.path.join(directory, "manifest.json")) as f:
        manifest = json.load(f)
    if manifest.get("format") != FORMAT:
        raise ValueError(f"{directory}: not a {FORMAT} checkpoint")
    if len(manifest["params"]) != len(fsdp._shards):
        raise ValueError(f"{directory}: {len(manifest['params'])} parameters in the checkpoint, {len(fsdp._shards)} in the model")
    for meta, ne in zip(manifest["params"], fsdp._numels):
        if meta["numel"] != ne:
            raise ValueError(f"{directory}: parameter {meta['name']} has {meta['numel']} elements in the checkpoint, {ne} in the model")
    old_world = int(manifest["world_size"])
    same = old_world == fsdp.world
    files = [SafeTensorsFile(_rank_file(directory, fsdp.rank))] if same else [SafeTensorsFile(_rank_file(directory, r)) for r in range(old_world)]
    inner = getattr(optimizer, "inner", optimizer)
    try:
        with torch.no_grad():
            for i, (sh, ne, sl) in enumerate(zip(fsdp._shards, fsdp._numels, fsdp._shard_len)):
                t = files[0].get_tensor(f"shard.{i}") if same else _recut(files, f"shard.{i}", ne, sl, fsdp.rank)
                sh.data.copy_(t.to(sh.dtype))
                if optimizer is None:
                    continue
                keys = [k[len(f"opt.{i}."):] for k in files[0].keys() if k.startswith(f"opt.{i}.")]
                st = inner.state.setdefault(sh, {}) if hasattr(inner, "state") else {}
                for k in keys:
                    v = files[0].get_tensor(f"opt.{i}.{k}") if same else _recut(files, f"opt.{i}.{k}", ne, sl, fsdp.rank)
                    if v.dim() == 0 and not torch.is_tensor(st.get(k)):
                        st[k] = int(v) if float(v).is_integer() else float(v)
                    else:
                        st[k] = v.to(device=sh.device, dtype=st[k].dtype if torch.is_tensor(st.get(k)) else v.dtype).view_as(sh) if v.dim() else v.to(sh.device)
    finally:
        for f in files:
            f.close()
    if optimizer is not None:
        for g, saved in zip(getattr(inner, "param_groups", []), manifest.get("optimizer", {}).get("param_groups", [])):
            for k, v in saved.items():
                g[k] = tuple(v) if isinstance(g.get(k), tuple) and isinstance(v, list) else v
    fsdp._gathered = False
    fsdp.pg.barrier()
    return manifest.get("extra", {})
