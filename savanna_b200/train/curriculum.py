"""Sequence-length curriculum: training starts on short prefixes of every sample and the length grows with the step count.

Role of DeepSpeed's legacy curriculum scheduler as the reference drives it (savanna/training.py:910-924, 957-963: the
batch is cut to `update_difficulty(iteration + 1)` tokens, the loss sees the same prefix).  Configuration
(`curriculum_learning` in the YAML):

    enabled: true
    curriculum_type: seqlen
    min_difficulty: 64            # first length
    max_difficulty: 8192          # final length (the model's seq_length)
    schedule_type: fixed_linear | fixed_root | fixed_discrete
    schedule_config:
      total_curriculum_step: 10000      # fixed_linear / fixed_root: steps until max_difficulty
      difficulty_step: 64               #   lengths are rounded down to a multiple of this
      root_degree: 2                    #   fixed_root only (fixed_linear is degree 1)
      difficulty: [64, 512, 8192]       # fixed_discrete: lengths ...
      max_step: [1000, 5000]            #   ... and the last step of each but the final one
"""
from __future__ import annotations

import math
from typing import Dict, Optional


class CurriculumScheduler:
    def __init__(self, config: Dict):
        self.min = int(config["min_difficulty"])
        self.max = int(config["max_difficulty"])
        if self.min > self.max or self.min <= 0:
            raise ValueError(f"curriculum: need 0 < min_difficulty <= max_difficulty (got {self.min}, {self.max})")
        self.kind = config.get("schedule_type", "fixed_linear")
        sc = dict(config.get("schedule_config") or {})
        if self.kind in ("fixed_linear", "fixed_root"):
            self.total = int(sc["total_curriculum_step"])
            self.quantum = int(sc.get("difficulty_step", 8))
            self.degree = 1.0 if self.kind == "fixed_linear" else float(sc["root_degree"])
            if self.total <= 0 or self.quantum <= 0 or self.degree <= 0:
                raise ValueError("curriculum: total_curriculum_step, difficulty_step and root_degree must be positive")
        elif self.kind == "fixed_discrete":
            self.levels = [int(d) for d in sc["difficulty"]]
            self.last_steps = [int(s) for s in sc["max_step"]]
            if len(self.levels) != len(self.last_steps) + 1 or not self.levels:
                raise ValueError("curriculum: fixed_discrete needs one more `difficulty` entry than `max_step` entries")
        else:
            raise ValueError(f"curriculum schedule_type {self.kind!r} unknown (fixed_linear | fixed_root | fixed_discrete)")
        self.current = self.min

    def difficulty(self, step: int) -> int:
        """Sequence length at optimizer step `step` (1-based)."""
        if self.kind == "fixed_discrete":
            for level, last in zip(self.levels, self.last_steps):
                if step <= last:
                    return level
            return self.levels[-1]
        frac = min(1.0, max(0.0, step / self.total)) ** (1.0 / self.degree)
        d = math.floor(frac * (self.max - self.min) + self.min)
        d -= d % self.quantum
        return max(min(d, self.max), min(self.min, self.max))

    def update_difficulty(self, step: int) -> int:
        self.current = self.difficulty(step)
        return self.current

    def state_dict(self) -> Dict:
        return {"current_difficulty": self.current}

    def load_state_dict(self, sd: Dict) -> None:
        self.current = int(sd.get("current_difficulty", self.current))


def from_config(cfg) -> Optional[CurriculumScheduler]:
    c = cfg.curriculum_learning
    if not c or not c.get("enabled", False):
        return None
    if c.get("curriculum_type", "seqlen") != "seqlen":
        raise ValueError("curriculum_type: only `seqlen` (sequence-length curriculum) exists")
    return CurriculumScheduler(c)
