"""Learning-rate schedules (reference: savanna/learning_rates.py:7-108, savanna/schedulers.py:13-45).

AnnealingLR: linear warm-up over `warmup_iter` steps, then constant / linear / cosine / exponential
decay measured against `end_iter` (the reference divides by `end_iter`, not `end_iter - warmup`,
learning_rates.py:42-61), floored at `min_lr`.  Parameter groups carrying a fixed `lr` of their own
(Hyena-MR filter lr, wd-free lr) are scaled by the same factor.
"""
from __future__ import annotations

import math
from typing import Dict, List


class AnnealingLR:
    def __init__(self, optimizer, start_lr: float, warmup_iter: int, total_iters: int, decay_style: str,
                 last_iter: int = 0, min_lr: float = 0.0, use_checkpoint_lr_scheduler: bool = True,
                 override_lr_scheduler: bool = False):
        self.optimizer = optimizer
        self.start_lr, self.min_lr = start_lr, min_lr
        self.warmup_iter, self.end_iter = warmup_iter, total_iters
        self.decay_style = decay_style
        self.num_iters = last_iter
        self.use_checkpoint_lr_scheduler = use_checkpoint_lr_scheduler
        self.override_lr_scheduler = override_lr_scheduler
        if override_lr_scheduler and use_checkpoint_lr_scheduler:
            raise ValueError("override_lr_scheduler and use_checkpoint_lr_scheduler are mutually exclusive")
        self.step(self.num_iters)

    def factor(self) -> float:
        # as the reference counts (learning_rates.py:47-52): the step count saturates at end_iter - warmup_iter, so the
        # decay runs over end_iter - 2 * warmup_iter steps after the warm-up and then holds its value
        it = min(self.num_iters, self.end_iter - self.warmup_iter)
        if self.warmup_iter > 0 and self.num_iters <= self.warmup_iter:
            return it / self.warmup_iter
        it = it - self.warmup_iter
        if self.decay_style == "linear":
            f = (self.end_iter - it) / self.end_iter
        elif self.decay_style == "cosine":
            f = 0.5 * (math.cos(math.pi * it / self.end_iter) + 1)
        elif self.decay_style == "exponential":
            f = math.exp(-0.693 * it / self.end_iter)
        else:
            f = 1.0
        return f

    def in_warmup(self) -> bool:
        return self.warmup_iter > 0 and self.num_iters <= self.warmup_iter

    def get_lr(self, base: float = None) -> float:
        base = self.start_lr if base is None else base
        if self.in_warmup():
            return base * self.factor()             # the floor applies to the decay only: warm-up starts at zero
        return max(base * self.factor(), self.min_lr)

    def step(self, step_num: int = None) -> None:
        self.num_iters = self.num_iters + 1 if step_num is None else step_num
        for g in self.optimizer.param_groups:
            if g.get("fixed_lr", False):
                g["lr"] = self.get_lr(self.start_lr * g.get("lr_mult", 1.0))     # same shape and floor, own peak
            else:
                g["lr"] = self.get_lr()

    def state_dict(self) -> Dict:
        return {"start_lr": self.start_lr, "warmup_iter": self.warmup_iter, "num_iters": self.num_iters,
                "decay_style": self.decay_style, "end_iter": self.end_iter, "min_lr": self.min_lr}

    def _check(self, mine, theirs, name):
        if self.override_lr_scheduler:
            return mine
        if not self.use_checkpoint_lr_scheduler and mine != theirs:
            raise ValueError(f"lr scheduler: {name} differs between config ({mine}) and checkpoint ({theirs}); "
                             "set override_lr_scheduler or use_checkpoint_lr_scheduler")
        return theirs

    def load_state_dict(self, sd: Dict) -> None:
        self.start_lr = self._check(self.start_lr, sd["start_lr"], "learning rate")
        self.min_lr = self._check(self.min_lr, sd["min_lr"], "minimum learning rate")
        self.warmup_iter = self._check(self.warmup_iter, sd["warmup_iter"], "warmup iterations")
        self.end_iter = self._check(self.end_iter, sd["end_iter"], "total iterations")
        self.decay_style = self._check(self.decay_style, sd["decay_style"], "decay style")
        self.num_iters = sd["num_iters"]
        self.step(self.num_iters)


class MultiLR:
    """Several schedulers stepped together (one per optimizer / group family)."""

    def __init__(self, schedulers: List):
        self.schedulers = list(schedulers)

    def step(self, step_num: int = None):
        for s in self.schedulers:
            s.step(step_num)

    def state_dict(self):
        return {"schedulers": [s.state_dict() for s in self.schedulers]}

    def load_state_dict(self, sd):
        for s, d in zip(self.schedulers, sd["schedulers"]):
            s.load_state_dict(d)


def build_lr_scheduler(optimizer, cfg) -> AnnealingLR:
    num_iters = max(1, cfg.lr_decay_iters or cfg.train_iters or 1)
    warmup_iter = int((cfg.warmup or 0.0) * num_iters)
    return AnnealingLR(optimizer, start_lr=cfg.lr, warmup_iter=warmup_iter, total_iters=num_iters,
                       decay_style=cfg.lr_decay_style, last_iter=0, min_lr=cfg.min_lr,
                       use_checkpoint_lr_scheduler=cfg.use_checkpoint_lr_scheduler,
                       override_lr_scheduler=cfg.override_lr_scheduler)
