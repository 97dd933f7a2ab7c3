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


def _dump(folder, tag):
    try:
        snap = torch.cuda.memory._snapshot()
        with open(os.path.join(folder, f"{tag}.pickle"), "wb") as fh:
            pickle.dump(snap, fh)
    except Exception as exc:  # snapshotting must never take the run down
        print(f"memory snapshot failed: {exc}", flush=True)
