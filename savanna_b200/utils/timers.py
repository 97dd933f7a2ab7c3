"""Named wall-clock timers with optional device synchronisation (reference: savanna/utils.py:586-670)
and a device-event timer whose result is the maximum over ranks, the rule for every multi-GPU number."""
from __future__ import annotations

import time
from typing import Dict, List

import torch
import torch.distributed as dist


class Timer:
    def __init__(self, name: str, sync: bool = True):
        self.name, self.sync = name, sync
        self.elapsed_, self.started_, self.start_time = 0.0, False, 0.0

    def _sync(self):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()

    def start(self):
        if self.started_:
            raise RuntimeError(f"timer {self.name} has already been started")
        self._sync()
        self.start_time = time.time()
        self.started_ = True

    def stop(self):
        if not self.started_:
            raise RuntimeError(f"timer {self.name} is not started")
        self._sync()
        self.elapsed_ += time.time() - self.start_time
        self.started_ = False

    def reset(self):
        self.elapsed_, self.started_ = 0.0, False

    def elapsed(self, reset: bool = True) -> float:
        was = self.started_
        if was:
            self.stop()
        e = self.elapsed_
        if reset:
            self.reset()
        if was:
            self.start()
        return e


class Timers:
    def __init__(self, use_wandb: bool = False, tensorboard_writer=None, sync: bool = True):
        self.timers: Dict[str, Timer] = {}
        self.use_wandb, self.tensorboard_writer, self.sync = use_wandb, tensorboard_writer, sync

    def __call__(self, name: str) -> Timer:
        if name not in self.timers:
            self.timers[name] = Timer(name, self.sync)
        return self.timers[name]

    def write(self, names: List[str], iteration: int, normalizer: float = 1.0, reset: bool = False):
        for n in names:
            v = self.timers[n].elapsed(reset=reset) / normalizer
            if self.tensorboard_writer:
                self.tensorboard_writer.add_scalar(f"timers/{n}", v, iteration)

    def log(self, names: List[str], normalizer: float = 1.0, reset: bool = True) -> str:
        s = "time (ms)"
        for n in names:
            s += f" | {n}: {self.timers[n].elapsed(reset=reset) * 1000.0 / normalizer:.2f}"
        if not dist.is_initialized() or dist.get_rank() == 0:
            print(s, flush=True)
        return s


class DeviceTimer:
    """CUDA-event timer on the current stream; `elapsed_ms_max()` is the maximum over all ranks."""

    def __init__(self):
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.t0 = self.t1 = 0.0

    def start(self):
        if self.cuda:
            self.e0.record()
        self.t0 = time.perf_counter()

    def stop(self):
        if self.cuda:
            self.e1.record()
        self.t1 = time.perf_counter()

    def elapsed_ms(self) -> float:
        if self.cuda:
            self.e1.synchronize()
            return self.e0.elapsed_time(self.e1)
        return (self.t1 - self.t0) * 1e3

    def elapsed_ms_max(self, group=None) -> float:
        ms = self.elapsed_ms()
        if dist.is_available() and dist.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if self.cuda and dist.get_backend() == "nccl" else "cpu"
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            ms = float(t.item())
        return ms
