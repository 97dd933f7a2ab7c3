"""Profilers behind one interface: start / stop / step / mark(name).

EmptyProfiler  does nothing.
TorchProfiler  torch.profiler with a (wait, warmup, active, repeat) schedule; the trace handler writes a
               per-rank Chrome trace (and optionally memory timeline, stacks, key-averages table).
CudaProfiler   for an external capture tool driven by cudaProfilerStart/Stop: starts after
               `nsys_warmup_steps`, stops after `nsys_num_steps`, emits NVTX ranges for the marks.
`train_step` wraps forward / backward / optimizer in marks named TRAIN_STEP_FORWARD, TRAIN_STEP_BACKWARD,
TRAIN_STEP_OPTIMIZER_STEP (reference: savanna/profiler.py:26-455, savanna/training.py:1444-1495).
"""
from __future__ import annotations

import contextlib
import os
import shutil
from typing import Optional

import torch

from .. import print_rank_0

MARKS = ("TRAIN_STEP_FORWARD", "TRAIN_STEP_BACKWARD", "TRAIN_STEP_OPTIMIZER_STEP", "TRAIN_STEP")


class EmptyProfiler:
    def start(self): pass
    def stop(self): pass
    def step(self): pass

    def mark(self, name: str):
        return contextlib.nullcontext()


class TorchProfiler(EmptyProfiler):
    def __init__(self, cfg, rank: int):
        self.cfg, self.rank = cfg, rank
        out = cfg.profiler_output_dir
        if cfg.profiler_clean_output_dir and rank == 0 and os.path.isdir(out):
            shutil.rmtree(out, ignore_errors=True)
        os.makedirs(out, exist_ok=True)
        acts = []
        if cfg.profile_cpu:
            acts.append(torch.profiler.ProfilerActivity.CPU)
        if cfg.profile_cuda and torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self.prof = torch.profiler.profile(
            activities=acts,
            schedule=torch.profiler.schedule(wait=cfg.profiler_schedule_wait, warmup=cfg.profiler_schedule_warmup,
                                             active=cfg.profiler_schedule_active, repeat=cfg.profiler_schedule_repeat),
            on_trace_ready=self._on_trace, record_shapes=cfg.profile_record_shapes, profile_memory=cfg.profile_memory,
            with_stack=cfg.profile_with_stack, with_flops=cfg.profile_with_flops)
        self.traces = 0

    def _on_trace(self, prof):
        out = self.cfg.profiler_output_dir
        path = os.path.join(out, f"rank{self.rank}_step{prof.step_num}.pt.trace.json.gz")
        prof.export_chrome_trace(path)
        self.traces += 1
        if self.rank == 0:
            rows = self.cfg.profiler_num_rows
            table = prof.key_averages().table(sort_by="self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total",
                                              row_limit=rows if rows and rows > 0 else 50)
            with open(os.path.join(out, f"key_averages_step{prof.step_num}.txt"), "w") as fh:
                fh.write(table)
            if self.cfg.profile_memory:
                try:
                    prof.export_memory_timeline(os.path.join(out, f"memory_timeline_step{prof.step_num}.html"))
                except Exception as exc:
                    print_rank_0(f"memory timeline export failed: {exc}")

    def start(self):
        self.prof.start()

    def stop(self):
        self.prof.stop()

    def step(self):
        self.prof.step()

    def mark(self, name: str):
        return torch.profiler.record_function(name)


class CudaProfiler(EmptyProfiler):
    def __init__(self, cfg, rank: int):
        self.cfg, self.rank = cfg, rank
        self.steps = 0
        self.running = False
        self.done = False
        if cfg.disable_autograd_multithreading:
            torch.autograd.set_multithreading_enabled(False)     # NVTX ranges nest only on one thread
        self._nvtx_ctx = None

    def start(self):
        pass

    def _begin(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
            from ..ops import cuda_ops
            cuda_ops.set_nvtx(True)                  # one range per native kernel launcher inside the capture window
            if self.cfg.emit_nvtx:
                self._nvtx_ctx = torch.autograd.profiler.emit_nvtx(record_shapes=self.cfg.profile_record_shapes)
                self._nvtx_ctx.__enter__()
        self.running = True

    def _end(self):
        if self.running and torch.cuda.is_available():
            torch.cuda.synchronize()
            if self._nvtx_ctx is not None:
                self._nvtx_ctx.__exit__(None, None, None)
                self._nvtx_ctx = None
            torch.cuda.cudart().cudaProfilerStop()
            from ..ops import cuda_ops
            cuda_ops.set_nvtx(False)
        self.running, self.done = False, True

    def step(self):
        self.steps += 1
        if not self.running and not self.done and self.steps == self.cfg.nsys_warmup_steps:
            self._begin()
        elif self.running and self.steps == self.cfg.nsys_warmup_steps + self.cfg.nsys_num_steps:
            self._end()

    def stop(self):
        if self.running:
            self._end()

    @contextlib.contextmanager
    def mark(self, name: str):
        on = self.running and torch.cuda.is_available()
        if on:
            torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            if on:
                torch.cuda.nvtx.range_pop()


def setup_profiler(cfg) -> EmptyProfiler:
    rank = cfg.rank or 0
    if not cfg.should_profile or cfg.profiler_type == "none":
        return EmptyProfiler()
    if cfg.profile_ranks is not None and rank not in cfg.profile_ranks:
        return EmptyProfiler()
    if cfg.profiler_type == "torch":
        return TorchProfiler(cfg, rank)
    if cfg.profiler_type == "nsys":
        return CudaProfiler(cfg, rank)
    raise ValueError(f"profiler type {cfg.profiler_type!r} unknown")


def build_nsys_command(cfg, train_cmd: list, output: str = "nsys_profile") -> list:
    """Command line that wraps a training command in an external capture driven by cudaProfilerApi
    (the launcher adds it with --nsys; reference: profiler.py:487-620)."""
    cmd = ["nsys", "profile", "--capture-range=cudaProfilerApi", "--trace=cuda,nvtx", "-o", output, "--force-overwrite=true"]
    if cfg.nsys_stop_on_exit:
        cmd.append("--capture-range-end=stop")
    return cmd + list(train_cmd)
