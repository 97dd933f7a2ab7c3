"""Loss scaling for fp16 training.

fp16 gradients underflow without a scale on the loss and overflow with too large a one.  The loss is multiplied by
`scale` before the backward; the optimizer divides the gradients by it again (folded into its clip coefficient), checks
the gradient norm for inf / nan, and skips the update when one is found.  The dynamic scaler halves the scale after
overflows and doubles it after `window` clean steps (the policy of DeepSpeed's fp16 optimizer, which the reference
configures through its `fp16` block: `loss_scale` (0 = dynamic), `initial_scale_power`, `loss_scale_window`,
`hysteresis`, `min_loss_scale`; reference: savanna/arguments/deepspeed_args.py fp16 dict, savanna/utils.py:702-716 for the
abort after 50 skipped steps).

The overflow check reads one scalar on the host per step.  bf16 training, the path this framework is tuned for, has no
scaler and keeps its step free of host synchronisation.
"""
from __future__ import annotations

import math
from typing import Dict, Optional


class LossScaler:
    """Static scale: overflows are reported (and the step skipped) but the scale never moves."""

    dynamic = False

    def __init__(self, scale: float = 1.0):
        self.scale = float(scale)
        self.overflows = 0

    def update(self, overflow: bool) -> None:
        self.overflows += int(bool(overflow))

    def check(self, grad_norm) -> bool:
        """True when the (already reduced) gradient norm is inf / nan; updates the scale."""
        v = float(grad_norm)
        bad = math.isinf(v) or math.isnan(v)
        self.update(bad)
        return bad

    def state_dict(self) -> Dict:
        return {"cur_scale": self.scale, "dynamic": self.dynamic, "overflows": self.overflows}

    def load_state_dict(self, sd: Dict) -> None:
        self.scale = float(sd.get("cur_scale", self.scale))
        self.overflows = int(sd.get("overflows", self.overflows))


class DynamicLossScaler(LossScaler):
    """scale starts at 2 ** initial_scale_power.  An overflow consumes one unit of `hysteresis`; when none is left the
    scale is halved (not below `min_scale`).  After `window` steps since the last overflow the scale doubles (and, with
    `consecutive_hysteresis`, the hysteresis budget is refilled)."""

    dynamic = True

    def __init__(self, initial_scale_power: int = 16, window: int = 1000, hysteresis: int = 2, min_scale: float = 1.0,
                 scale_factor: float = 2.0, consecutive_hysteresis: bool = False):
        super().__init__(2.0 ** initial_scale_power)
        self.window, self.min_scale, self.factor = int(window), float(min_scale), float(scale_factor)
        self.hysteresis = self.budget = int(hysteresis)
        self.consecutive = bool(consecutive_hysteresis)
        self.iter = 0
        self.last_overflow_iter = -1

    def update(self, overflow: bool) -> None:
        if overflow:
            self.overflows += 1
            if self.hysteresis == 1 or self.budget == 1:
                self.scale = max(self.scale / self.factor, self.min_scale)
            else:
                self.budget -= 1
            self.last_overflow_iter = self.iter
        else:
            if self.consecutive:
                self.budget = self.hysteresis
            if (self.iter - self.last_overflow_iter) % self.window == 0:
                if not self.consecutive:
                    self.budget = self.hysteresis
                self.scale *= self.factor
        self.iter += 1

    def state_dict(self) -> Dict:
        sd = super().state_dict()
        sd.update(cur_iter=self.iter, last_overflow_iter=self.last_overflow_iter, cur_hysteresis=self.budget,
                  scale_window=self.window, min_scale=self.min_scale, scale_factor=self.factor)
        return sd

    def load_state_dict(self, sd: Dict) -> None:
        super().load_state_dict(sd)
        self.iter = int(sd.get("cur_iter", self.iter))
        self.last_overflow_iter = int(sd.get("last_overflow_iter", self.last_overflow_iter))
        self.budget = int(sd.get("cur_hysteresis", self.budget))


def from_config(cfg) -> Optional[LossScaler]:
    """A scaler for fp16 runs, None otherwise.  Values come from the `fp16` block, with the top-level `loss_scale`,
    `loss_scale_window`, `hysteresis` and `min_scale` keys as fall-backs."""
    if cfg.precision != "fp16":
        return None
    d = dict(cfg.fp16 or {})
    static = d.get("loss_scale", cfg.loss_scale if cfg.loss_scale is not None else 0)
    if static:
        return LossScaler(float(static))
    return DynamicLossScaler(
        initial_scale_power=int(d.get("initial_scale_power", 16)),
        window=int(d.get("loss_scale_window", cfg.loss_scale_window or 1000)),
        hysteresis=int(d.get("hysteresis", cfg.hysteresis or 2)),
        min_scale=float(d.get("min_loss_scale", cfg.min_scale or 1.0)),
        consecutive_hysteresis=bool(d.get("consecutive_hysteresis", False)))
