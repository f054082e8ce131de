"""The sixteen learning-rate schedulers with the constructors and closed forms of the reference
(torch/optim/lr_scheduler.h).  They are host-side scalar programs: ``step()`` advances
``last_epoch`` (which starts at -1) and writes ``group['lr']``; ``state_dict`` makes them resumable.
Works with any optimizer object that exposes ``param_groups``."""
from __future__ import annotations

import math
from typing import Callable, List, Sequence, Union

__all__ = ["LRScheduler", "StepLR", "MultiStepLR", "ExponentialLR", "CosineAnnealingLR", "LinearLR", "ConstantLR",
           "ReduceLROnPlateau", "WarmupCosineAnnealingLR", "OneCycleLR", "CosineAnnealingWarmRestarts", "CyclicLR",
           "PolynomialLR", "LambdaLR", "MultiplicativeLR", "SequentialLR", "ChainedScheduler"]


class LRScheduler:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.last_epoch = -1
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]

    def get_lr(self) -> List[float]:
        raise NotImplementedError

    def step(self, epoch: int = -1):
        self.last_epoch = self.last_epoch + 1 if epoch == -1 else epoch
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr

    def step_group(self, group_idx: int, epoch: int = -1):
        self.last_epoch = self.last_epoch + 1 if epoch == -1 else epoch
        lrs = self.get_lr()
        if group_idx < len(lrs):
            self.optimizer.param_groups[group_idx]["lr"] = lrs[group_idx]

    def get_last_lr(self) -> float:
        return self.optimizer.param_groups[0]["lr"] if self.optimizer.param_groups else 0.0

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer" and not callable(v) and k not in ("fns", "schedulers")}

    def load_state_dict(self, sd):
        self.__dict__.update(sd)


class StepLR(LRScheduler):
    def __init__(self, optimizer, step_size: int, gamma: float = 0.1):
        super().__init__(optimizer)
        self.step_size, self.gamma = step_size, gamma

    def get_lr(self):
        f = self.gamma ** (self.last_epoch // self.step_size)
        return [b * f for b in self.base_lrs]


class MultiStepLR(LRScheduler):
    def __init__(self, optimizer, milestones: Sequence[int], gamma: float = 0.1):
        super().__init__(optimizer)
        self.milestones, self.gamma = sorted(milestones), gamma

    def get_lr(self):
        n = sum(1 for m in self.milestones if self.last_epoch >= m)
        return [b * self.gamma ** n for b in self.base_lrs]


class ExponentialLR(LRScheduler):
    def __init__(self, optimizer, gamma: float):
        super().__init__(optimizer)
        self.gamma = gamma

    def get_lr(self):
        return [b * self.gamma ** self.last_epoch for b in self.base_lrs]


class CosineAnnealingLR(LRScheduler):
    def __init__(self, optimizer, T_max: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.T_max, self.eta_min = T_max, eta_min

    def get_lr(self):
        c = (1 + math.cos(math.pi * self.last_epoch / self.T_max)) / 2
        return [self.eta_min + (b - self.eta_min) * c for b in self.base_lrs]


class LinearLR(LRScheduler):
    def __init__(self, optimizer, start_factor: float = 1.0 / 3, end_factor: float = 1.0, total_iters: int = 5):
        super().__init__(optimizer)
        self.start_factor, self.end_factor, self.total_iters = start_factor, end_factor, total_iters

    def get_lr(self):
        if self.last_epoch >= self.total_iters:
            f = self.end_factor
        else:
            f = self.start_factor + self.last_epoch / self.total_iters * (self.end_factor - self.start_factor)
        return [b * f for b in self.base_lrs]


class ConstantLR(LRScheduler):
    def __init__(self, optimizer, factor: float = 1.0 / 3, total_iters: int = 5):
        super().__init__(optimizer)
        self.factor, self.total_iters = factor, total_iters

    def get_lr(self):
        m = self.factor if self.last_epoch < self.total_iters else 1.0
        return [b * m for b in self.base_lrs]


class ReduceLROnPlateau:
    def __init__(self, optimizer, mode: str = "min", factor: float = 0.1, patience: int = 10, threshold: float = 1e-4,
                 min_lr: float = 0.0):
        self.optimizer, self.mode, self.factor, self.patience = optimizer, str(mode).lower(), factor, patience
        self.threshold, self.min_lr = threshold, min_lr
        self.num_bad_epochs = 0
        self.best = math.inf if self.mode == "min" else -math.inf

    def step(self, metric: float):
        better = metric < self.best - self.threshold if self.mode == "min" else metric > self.best + self.threshold
        if better:
            self.best, self.num_bad_epochs = metric, 0
            return
        self.num_bad_epochs += 1
        if self.num_bad_epochs > self.patience:
            for g in self.optimizer.param_groups:
                g["lr"] = max(g["lr"] * self.factor, self.min_lr)
            self.num_bad_epochs = 0

    def get_last_lr(self):
        return self.optimizer.param_groups[0]["lr"]

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, sd):
        self.__dict__.update(sd)


class WarmupCosineAnnealingLR(LRScheduler):
    """``lr = base*(e+1)/warmup`` during warm-up, then cosine from base to ``eta_min``
    (torch/optim/lr_scheduler.h:359-398)."""

    def __init__(self, optimizer, warmup_epochs: int, total_epochs: int, eta_min: float = 0.0):
        super().__init__(optimizer)
        self.warmup_epochs, self.total_epochs, self.eta_min = warmup_epochs, total_epochs, eta_min

    def get_lr(self):
        e, w, T = self.last_epoch, self.warmup_epochs, self.total_epochs
        if e < w:
            return [b * (e + 1) / w for b in self.base_lrs]
        prog = min(1.0, (e - w) / max(T - w, 1))
        c = (1 + math.cos(math.pi * prog)) / 2
        return [self.eta_min + (b - self.eta_min) * c for b in self.base_lrs]


class OneCycleLR:
    def __init__(self, optimizer, max_lr: float, total_steps: int, pct_start: float = 0.3, div_factor: float = 25.0,
                 final_div_factor: float = 1e4):
        self.optimizer, self.max_lr, self.total_steps, self.pct_start = optimizer, max_lr, total_steps, pct_start
        self.initial_lr = max_lr / div_factor
        self.min_lr = self.initial_lr / final_div_factor
        self.step_count = 0
        for g in optimizer.param_groups:
            g["lr"] = self.initial_lr

    def step(self):
        self.step_count += 1
        warm = int(self.total_steps * self.pct_start)
        if self.step_count <= warm:
            lr = self.initial_lr + self.step_count / max(warm, 1) * (self.max_lr - self.initial_lr)
        else:
            c = (1 + math.cos(math.pi * (self.step_count - warm) / max(self.total_steps - warm, 1))) / 2
            lr = self.min_lr + (self.max_lr - self.min_lr) * c
        for g in self.optimizer.param_groups:
            g["lr"] = lr

    def get_last_lr(self):
        return self.optimizer.param_groups[0]["lr"]

    def state_dict(self):
        return {k: v for k, v in self.__dict__.items() if k != "optimizer"}

    def load_state_dict(self, sd):
        self.__dict__.update(sd)


class CosineAnnealingWarmRestarts(LRScheduler):
    def __init__(self, optimizer, T_0: int, T_mult: int = 1, eta_min: float = 0.0):
        if T_0 <= 0:
            raise ValueError("T_0 must be positive")
        if T_mult < 1:
            raise ValueError("T_mult must be >= 1")
        super().__init__(optimizer)
        self.T_0, self.T_mult, self.eta_min = T_0, T_mult, eta_min
        self.T_i, self.T_cur = T_0, 0

    def step(self, epoch: int = -1):
        if epoch == -1:
            self.last_epoch += 1
            self.T_cur += 1
            if self.T_cur >= self.T_i:
                self.T_cur = 0
                self.T_i *= self.T_mult
        else:
            self.last_epoch = epoch
            rem, T_i = epoch, self.T_0
            while rem >= T_i:
                rem -= T_i
                T_i *= self.T_mult
            self.T_cur, self.T_i = rem, T_i
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr

    def get_lr(self):
        c = (1 + math.cos(math.pi * self.T_cur / self.T_i)) / 2
        return [self.eta_min + (b - self.eta_min) * c for b in self.base_lrs]


class CyclicLR(LRScheduler):
    def __init__(self, optimizer, base_lr: float, max_lr: float, step_size_up: int = 2000, step_size_down: int = -1,
                 mode: str = "triangular", gamma: float = 1.0):
        super().__init__(optimizer)
        self.base_lr, self.max_lr, self.step_size_up = base_lr, max_lr, step_size_up
        self.step_size_down = step_size_up if step_size_down < 0 else step_size_down
        self.mode, self.gamma = str(mode).lower(), gamma
        for g in optimizer.param_groups:
            g["lr"] = base_lr
        self.base_lrs = [base_lr] * len(self.base_lrs)

    def get_lr(self):
        total = self.step_size_up + self.step_size_down
        cycle = self.last_epoch // total
        pos = self.last_epoch - cycle * total
        x = pos / self.step_size_up if pos < self.step_size_up else 1 - (pos - self.step_size_up) / self.step_size_down
        scale = 1.0
        if self.mode == "triangular2":
            scale = 1 / 2 ** cycle
        elif self.mode in ("exprange", "exp_range"):
            scale = self.gamma ** self.last_epoch
        return [self.base_lr + (self.max_lr - self.base_lr) * x * scale] * len(self.base_lrs)


class PolynomialLR(LRScheduler):
    def __init__(self, optimizer, total_iters: int, power: float = 1.0):
        super().__init__(optimizer)
        self.total_iters, self.power = total_iters, power

    def get_lr(self):
        f = 0.0 if self.last_epoch >= self.total_iters else (1 - self.last_epoch / self.total_iters) ** self.power
        return [b * f for b in self.base_lrs]


def _fn_list(fn, n):
    fns = list(fn) if isinstance(fn, (list, tuple)) else [fn] * n
    if len(fns) != n:
        raise ValueError("lambda count must match param_groups")
    return fns


class LambdaLR(LRScheduler):
    def __init__(self, optimizer, lr_lambda: Union[Callable[[int], float], Sequence[Callable[[int], float]]]):
        super().__init__(optimizer)
        self.fns = _fn_list(lr_lambda, len(self.base_lrs))

    def get_lr(self):
        return [b * f(self.last_epoch) for b, f in zip(self.base_lrs, self.fns)]


class MultiplicativeLR(LRScheduler):
    def __init__(self, optimizer, lr_lambda):
        super().__init__(optimizer)
        self.fns = _fn_list(lr_lambda, len(self.base_lrs))

    def step(self, epoch: int = -1):
        self.last_epoch = self.last_epoch + 1 if epoch == -1 else epoch
        if self.last_epoch == 0:
            return
        for g, f in zip(self.optimizer.param_groups, self.fns):
            g["lr"] *= f(self.last_epoch)

    def get_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]


class SequentialLR:
    def __init__(self, optimizer, schedulers: Sequence[LRScheduler], milestones: Sequence[int]):
        if not schedulers:
            raise ValueError("SequentialLR: schedulers must not be empty")
        if len(milestones) + 1 != len(schedulers):
            raise ValueError("SequentialLR: len(milestones) must equal len(schedulers) - 1")
        if any(b <= a for a, b in zip(milestones, milestones[1:])):
            raise ValueError("SequentialLR: milestones must be strictly increasing")
        self.optimizer, self.schedulers, self.milestones = optimizer, list(schedulers), list(milestones)
        self.step_count = -1

    def step(self):
        self.step_count += 1
        active = len(self.schedulers) - 1
        for i, m in enumerate(self.milestones):
            if self.step_count < m:
                active = i
                break
        self.schedulers[active].step()

    def get_last_lr(self):
        return self.optimizer.param_groups[0]["lr"]


class ChainedScheduler:
    """Every scheduler steps; the group's lr is its base lr times the product of each scheduler's
    (current lr / base lr)."""

    def __init__(self, optimizer, schedulers: Sequence[LRScheduler]):
        if not schedulers:
            raise ValueError("ChainedScheduler: schedulers must not be empty")
        self.optimizer, self.schedulers = optimizer, list(schedulers)
        self.base_lrs = [g["lr"] for g in optimizer.param_groups]

    def step(self):
        comb = [1.0] * len(self.base_lrs)
        for s in self.schedulers:
            s.step()
            for i, (post, base) in enumerate(zip(s.get_lr(), s.base_lrs)):
                comb[i] *= post / (base if base != 0 else 1.0)
        for g, b, c in zip(self.optimizer.param_groups, self.base_lrs, comb):
            g["lr"] = b * c

    def get_last_lr(self):
        return self.optimizer.param_groups[0]["lr"]
