"""CUDA allocator statistics, cross-rank summaries and memory-history snapshots
(reference: savanna/memory_stats.py:106-268)."""
from __future__ import annotations

import os
import pickle
from contextlib import contextmanager
from typing import Dict

import torch
import torch.distributed as dist

GB = float(1 << 30)


def memory_stats(device=None) -> Dict[str, float]:
    if not torch.cuda.is_available():
        return {}
    s = torch.cuda.memory_stats(device)
    return {
        "allocated_gb": s.get("allocated_bytes.all.current", 0) / GB,
        "max_allocated_gb": s.get("allocated_bytes.all.peak", 0) / GB,
        "reserved_gb": s.get("reserved_bytes.all.current", 0) / GB,
        "max_reserved_gb": s.get("reserved_bytes.all.peak", 0) / GB,
        "num_alloc_retries": s.get("num_alloc_retries", 0),
        "num_ooms": s.get("num_ooms", 0),
        "alloc_count": s.get("allocation.all.allocated", 0),
        "free_count": s.get("allocation.all.freed", 0),
    }


def format_memory_stats(stats: Dict[str, float]) -> str:
    if not stats:
        return "mem: n/a"
    return (f"mem alloc {stats['allocated_gb']:.1f} (max {stats['max_allocated_gb']:.1f}) GB | reserved "
            f"{stats['reserved_gb']:.1f} (max {stats['max_reserved_gb']:.1f}) GB | retries {stats['num_alloc_retries']}")


def gather_alloc_counts(group=None) -> Dict[str, float]:
    """min / max / mean of allocator call counts over ranks: differing counts between ranks are an early
    sign of divergent control flow."""
    st = memory_stats()
    v = torch.tensor([float(st.get("alloc_count", 0))], dtype=torch.float64)
    if dist.is_available() and dist.is_initialized():
        if dist.get_backend() == "nccl":
            v = v.cuda()
        vs = [torch.zeros_like(v) for _ in range(dist.get_world_size(group))]
        dist.all_gather(vs, v, group=group)
        v = torch.cat(vs)
    return {"min": float(v.min()), "max": float(v.max()), "mean": float(v.mean())}


@contextmanager
def memory_snapshot(folder: str, tag: str, enabled: bool = True, max_entries: int = 100000):
    """Record allocator history for the enclosed region and dump a snapshot pickle (also on OOM)."""
    if not (enabled and torch.cuda.is_available()):
        yield
        return
    os.makedirs(folder, exist_ok=True)
    torch.cuda.memory._record_memory_history(max_entries=max_entries)
    try:
        yield
    except torch.cuda.OutOfMemoryError:
        _dump(folder, tag + "_oom")
        raise
    finally:
        _dump(folder, tag)
        torch.cuda.memory._record_memory_history(enabled=None)


class MemorySnapshotter:
    """Allocator-history snapshots during training (keys `enable_memory_snapshot`, `save_memory_snapshot_folder`,
    `memory_snapshot_freq`, `memory_snapshot_max_entries`, `memory_snapshot_rank0_only`; role of the reference's
    savanna/memory_stats.py:207-268): history recording is switched on at construction, `step()` writes
    `<folder>/rank<r>/iteration_<n>/rank<r>_memory_snapshot.pickle` every `freq` steps, `on_oom()` writes
    `iteration_<n>_exit` when a step ran out of memory, `close()` stops the recording.  The pickles open in PyTorch's
    memory visualiser.  `recorder` / `snapshot` are the two allocator calls, replaceable in tests."""

    def __init__(self, folder: str, rank: int = 0, step: int = 0, freq: int = 3, max_entries: int = 100000,
                 recorder=None, snapshot=None, printer=print):
        self.folder = os.path.join(folder, f"rank{rank}")
        self.rank, self.step_num, self.freq = rank, int(step), max(1, int(freq))
        self._record = recorder or (lambda **kw: torch.cuda.memory._record_memory_history(**kw))
        self._snapshot = snapshot or (lambda: torch.cuda.memory._snapshot())
        self.printer = printer
        os.makedirs(self.folder, exist_ok=True)
        self._record(max_entries=max_entries)
        self.written = []

    @classmethod
    def from_config(cls, cfg, rank: int, step: int = 0):
        """None unless the run asks for snapshots on this rank (and has a CUDA allocator to record)."""
        if not cfg.enable_memory_snapshot or not torch.cuda.is_available():
            return None
        if cfg.memory_snapshot_rank0_only and rank != 0:
            return None
        return cls(cfg.save_memory_snapshot_folder or "memory_snapshot", rank, step, cfg.memory_snapshot_freq or 3,
                   cfg.memory_snapshot_max_entries or 100000)

    def _write(self, name: str) -> str:
        d = os.path.join(self.folder, name)
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"rank{self.rank}_memory_snapshot.pickle")
        try:
            with open(path, "wb") as fh:
                pickle.dump(self._snapshot(), fh)
            self.written.append(path)
            self.printer(f"rank {self.rank}: memory snapshot written to {path}")
        except Exception as exc:                    # a failed snapshot never takes the run down
            self.printer(f"rank {self.rank}: memory snapshot failed: {exc}")
        return path

    def step(self) -> None:
        self.step_num += 1
        if self.step_num % self.freq == 0:
            self._write(f"iteration_{self.step_num}")

    def on_oom(self) -> None:
        self._write(f"iteration_{self.step_num}_exit")

    def close(self) -> None:
        try:
            self._record(enabled=None)
        except Exception:
            pass


def _dump(folder, tag):
    try:
        snap = torch.cuda.memory._snapshot()
        with open(os.path.join(folder, f"{tag}.pickle"), "wb") as fh:
            pickle.dump(snap, fh)
    except Exception as exc:  # snapshotting must never take the run down
        print(f"memory snapshot failed: {exc}", flush=True)
