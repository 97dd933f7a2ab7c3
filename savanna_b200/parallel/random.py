"""Random-number streams for tensor parallelism (role of the reference's savanna/mpu/random.py shim over
DeepSpeed's CUDA RNG tracker): a named generator state per purpose, so dropout inside tensor-parallel regions
differs per rank while everything else stays identical."""
from __future__ import annotations

import contextlib
from typing import Dict

import torch

from . import state

_MODEL_PARALLEL_RNG = "model-parallel-rng"


class RNGStatesTracker:
    def __init__(self):
        self.states: Dict[str, torch.Tensor] = {}
        self.seeds = set()

    def reset(self):
        self.states.clear()
        self.seeds.clear()

    def get_states(self):
        return {k: v.clone() for k, v in self.states.items()}

    def set_states(self, states):
        self.states = {k: v.clone() for k, v in states.items()}

    def _get(self):
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    def _set(self, s):
        if torch.cuda.is_available():
            torch.cuda.set_rng_state(s)
        else:
            torch.set_rng_state(s)

    def add(self, name: str, seed: int):
        if seed in self.seeds or name in self.states:
            raise ValueError(f"seed {seed} or state {name!r} already registered")
        self.seeds.add(seed)
        orig = self._get()
        if torch.cuda.is_available():
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states[name] = self._get()
        self._set(orig)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG):
        if name not in self.states:
            raise KeyError(f"rng state {name!r} is not registered")
        orig = self._get()
        self._set(self.states[name])
        try:
            yield
        finally:
            self.states[name] = self._get()
            self._set(orig)


_TRACKER = RNGStatesTracker()


def get_cuda_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def model_parallel_cuda_manual_seed(seed: int) -> None:
    """Default stream: same on all tensor-parallel ranks; tracked stream: seed + 2718 + tp_rank."""
    _TRACKER.reset()
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    else:
        torch.manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, seed + 2718 + state.get_model_parallel_rank())


def checkpoint(function, *args):
    """Activation checkpointing entry point (non-reentrant torch implementation)."""
    import torch.utils.checkpoint as ckpt
    return ckpt.checkpoint(function, *args, use_reentrant=False)
