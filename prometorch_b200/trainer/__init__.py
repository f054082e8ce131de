"""Trainer: ``LightningModule`` hooks, ``TrainerConfig``, ``Trainer.fit/test/save_checkpoint/load_checkpoint``
(torch/trainer/trainer.h:48-86, python/promethorch/trainer/__init__.py:199-216 in the reference).
Gradient accumulation, clipping, per-epoch checkpoints ``epoch_N.ptor``; on top of the reference a
checkpoint also carries optimizer, scheduler, RNG and step so that a run resumes exactly."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import serialization
from ..optim import clip_grad_norm_


class LightningModule(nn.Module):
    def training_step(self, batch, batch_idx):
        raise NotImplementedError

    def validation_step(self, batch, batch_idx):
        return None

    def test_step(self, batch, batch_idx):
        return self.validation_step(batch, batch_idx)

    def configure_optimizer(self):
        """Return the optimizer, or ``(optimizer, scheduler)``.  ``configure_optimizers`` is the same hook under
        the plural name; override either."""
        if type(self).configure_optimizers is not LightningModule.configure_optimizers:
            return self.configure_optimizers()
        raise NotImplementedError

    def configure_optimizers(self):
        return self.configure_optimizer()

    def on_train_start(self): ...
    def on_train_end(self): ...
    def on_epoch_start(self, epoch): ...
    def on_epoch_end(self, epoch, metrics): ...


@dataclass
class TrainerConfig:
    max_epochs: int = 1
    accumulate_grad_batches: int = 1
    gradient_clip_val: float = 0.0
    log_every_n_steps: int = 50
    save_every_n_epochs: int = 0
    checkpoint_dir: str = "checkpoints"
    device: str = "cpu"
    enable_progress_bar: bool = False
    max_steps: int = -1


class Trainer:
    def __init__(self, config: Optional[TrainerConfig] = None, **kw):
        self.config = config or TrainerConfig(**kw)
        self.global_step = 0
        self.current_epoch = 0
        self.optimizer = None
        self.scheduler = None
        self.history = []

    def _to(self, batch, dev):
        if torch.is_tensor(batch):
            return batch.to(dev, non_blocking=True)
        if isinstance(batch, (list, tuple)):
            return type(batch)(self._to(b, dev) for b in batch)
        return batch

    def fit(self, module: LightningModule, train_loader, val_loader=None):
        c = self.config
        dev = torch.device(c.device)
        module.to(dev)
        if self.optimizer is None:
            opt = module.configure_optimizer()
            if isinstance(opt, (tuple, list)):
                opt, self.scheduler = opt[0], (opt[1] if len(opt) > 1 else None)
            self.optimizer = opt
        module.on_train_start()
        for epoch in range(self.current_epoch, c.max_epochs):
            self.current_epoch = epoch
            module.train()
            module.on_epoch_start(epoch)
            t0, total, n = time.time(), 0.0, 0
            self.optimizer.zero_grad()
            for i, batch in enumerate(train_loader):
                loss = module.training_step(self._to(batch, dev), i)
                (loss / c.accumulate_grad_batches).backward()
                if (i + 1) % c.accumulate_grad_batches == 0:
                    if c.gradient_clip_val > 0:
                        clip_grad_norm_(module.parameters(), c.gradient_clip_val)
                    self.optimizer.step()
                    self.optimizer.zero_grad()
                    self.global_step += 1
                    if self.scheduler is not None and not hasattr(self.scheduler, "mode"):
                        self.scheduler.step()
                total += float(loss.detach())
                n += 1
                if c.log_every_n_steps and (i + 1) % c.log_every_n_steps == 0:
                    print(f"[Trainer] epoch {epoch} step {i + 1} loss {total / n:.4f}")
                if 0 < c.max_steps <= self.global_step:
                    break
            metrics = {"epoch": epoch, "train_loss": total / max(n, 1), "seconds": time.time() - t0}
            if val_loader is not None:
                metrics.update(self.test(module, val_loader, prefix="val"))
            self.history.append(metrics)
            module.on_epoch_end(epoch, metrics)
            if c.save_every_n_epochs and (epoch + 1) % c.save_every_n_epochs == 0:
                self.save_checkpoint(module, os.path.join(c.checkpoint_dir, f"epoch_{epoch + 1}.ptor"))
            if 0 < c.max_steps <= self.global_step:
                break
        self.current_epoch = c.max_epochs
        module.on_train_end()
        return self.history

    @torch.no_grad()
    def test(self, module: LightningModule, loader, prefix: str = "test"):
        dev = torch.device(self.config.device)
        module.eval()
        tot, n = 0.0, 0
        for i, batch in enumerate(loader):
            out = module.validation_step(self._to(batch, dev), i)
            if out is not None:
                if isinstance(out, dict):
                    out = out["loss"] if "loss" in out else next(iter(out.values()))
                tot += float(out)
                n += 1
        return {f"{prefix}_loss": tot / max(n, 1)}

    def save_checkpoint(self, module: nn.Module, path: str):
        """Weights go to ``path`` in the PTOR container; optimizer/scheduler/RNG/step go to ``path + '.state'``."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        serialization.save_state_dict(module.state_dict(), path)
        extra = {"epoch": self.current_epoch, "global_step": self.global_step, "rng": torch.get_rng_state(),
                 "optimizer": self.optimizer.state_dict() if self.optimizer is not None else None,
                 "scheduler": self.scheduler.state_dict() if self.scheduler is not None and hasattr(self.scheduler, "state_dict") else None}
        torch.save(extra, path + ".state")

    def load_checkpoint(self, module: nn.Module, path: str, strict: bool = False):
        module.load_state_dict(serialization.load_state_dict(path), strict=strict)
        sp = path + ".state"
        if os.path.exists(sp):
            extra = torch.load(sp, weights_only=True)
            self.current_epoch, self.global_step = extra["epoch"] + 1, extra["global_step"]
            torch.set_rng_state(extra["rng"])
            if self.optimizer is not None and extra.get("optimizer") is not None:
                self.optimizer.load_state_dict(extra["optimizer"])
            if self.scheduler is not None and extra.get("scheduler") is not None:
                self.scheduler.load_state_dict(extra["scheduler"])
