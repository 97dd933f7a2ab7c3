"""Run-time observability: straggler detection, collective-operation logging, allocator-churn watching, recycled CUDA events.

The reference delegates these to external packages and to DeepSpeed (savanna/training.py:87-201 event recycling and the
allocation watcher, :517-551 and :1608-1639 Heimdall / nvidia_resiliency_ext straggler detectors, savanna/logging.py:536-595
DeepSpeed's comms logger).  Here they are small in-tree pieces driven by the same configuration keys:

    StragglerDetector   per-rank section and step times over a reporting window; at a report every rank contributes its
                        medians (one small all-gather) and rank 0 prints min / median / max per section, each rank's
                        relative score (group median / own median, 1.0 = typical, lower = slower) and its individual score
                        (own best window / own current window), and names the ranks below the thresholds
                        (keys: heimdall_log_straggler, heimdall_log_interval, heimdall_straggler_minmax_count, use_next,
                        next_report_interval, next_*_threshold)
    CommsLogger         wraps the torch.distributed collectives in place, records per (operation, message size) the call
                        count and latencies (CUDA events on the calling stream, or wall time on CPU), derives algorithm and
                        bus bandwidth, prints `COMMS:<op>,<rank>,<bytes>,<latencies...>` lines in the reference's format
                        (keys: deepspeed_enable_comms_logging, deepspeed_comms_ops_to_log, deepspeed_comms_ranks_to_log,
                        deepspeed_comms_logging_interval, deepspeed_comms_print_summary)
    AllocStats          compares the caching allocator's device-allocation counters between steps and warns when they
                        move after warm-up (a sign of memory pressure that slows the step); empties the cache once at step 6
                        as the reference does (key: print_mem_alloc_stats)
    EventPool           timing events that are reused instead of created and destroyed every step (key: recycle_events)
"""
from __future__ import annotations

import contextlib
import statistics
import time
from collections import defaultdict
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------- recycled events


class EventPool:
    """CUDA timing events handed out and taken back; creating and destroying events every step costs driver calls and,
    with many streams, allocator churn."""

    def __init__(self):
        self._free: List["torch.cuda.Event"] = []
        self.created = 0

    def get(self):
        if self._free:
            return self._free.pop()
        self.created += 1
        return torch.cuda.Event(enable_timing=True)

    def put(self, *events) -> None:
        self._free.extend(e for e in events if e is not None)


EVENTS = EventPool()


# ----------------------------------------------------------------------------- straggler detection


class StragglerDetector:
    def __init__(self, world: int, rank: int, group=None, interval: int = 10, minmax_count: int = 32,
                 rel_threshold: float = 0.7, individual_threshold: float = 0.7, enabled: bool = True,
                 use_cuda_events: Optional[bool] = None, printer: Callable[[str], None] = print):
        self.world, self.rank, self.group = world, rank, group
        self.interval = max(1, int(interval))
        self.minmax_count = max(1, int(minmax_count))
        self.rel_threshold, self.individual_threshold = rel_threshold, individual_threshold
        self.enabled = enabled
        self.cuda = torch.cuda.is_available() if use_cuda_events is None else use_cuda_events
        self.printer = printer
        self.window: Dict[str, List[float]] = defaultdict(list)      # section -> times (ms) in the current window
        self._pending = []                                           # (section, start event, end event) not yet read
        self.best: Dict[str, float] = {}                             # section -> best (lowest) window median so far
        self.steps = 0
        self._t_step = None
        self.last_report: Optional[Dict] = None

    # -- recording ----------------------------------------------------------------
    @contextlib.contextmanager
    def section(self, name: str):
        """Times a named part of the step: on the device (events on the current stream, read at the next report, so
        nothing synchronises) and on the host."""
        if not self.enabled:
            yield
            return
        t0 = time.perf_counter()
        e0 = e1 = None
        if self.cuda:
            e0, e1 = EVENTS.get(), EVENTS.get()
            e0.record()
        try:
            yield
        finally:
            if self.cuda:
                e1.record()
                self._pending.append((name, e0, e1))
            self.window["host/" + name].append((time.perf_counter() - t0) * 1e3)

    def step(self) -> Optional[Dict]:
        """Call once per optimizer step; returns a report every `interval` steps (collective over the group)."""
        if not self.enabled:
            return None
        now = time.perf_counter()
        if self._t_step is not None:
            self.window["host/step"].append((now - self._t_step) * 1e3)
        self._t_step = now
        self.steps += 1
        if self.steps % self.interval:
            return None
        return self.report()

    def _drain(self) -> None:
        for name, e0, e1 in self._pending:
            e1.synchronize()
            self.window["gpu/" + name].append(e0.elapsed_time(e1))
            EVENTS.put(e0, e1)
        self._pending.clear()

    # -- reporting ----------------------------------------------------------------
    def report(self) -> Dict:
        self._drain()
        names = sorted(self.window)
        if self.world > 1 and dist.is_initialized():
            # every rank must contribute the same sections: agree on the union
            gathered: List = [None] * self.world
            dist.all_gather_object(gathered, names, group=self.group)
            names = sorted(set().union(*[set(g) for g in gathered]))
        mine = [statistics.median(self.window[n]) if self.window.get(n) else float("nan") for n in names]
        table = [mine]
        if self.world > 1 and dist.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else torch.device("cpu")
            t = torch.tensor(mine, dtype=torch.float64, device=dev)
            out = [torch.empty_like(t) for _ in range(self.world)]
            dist.all_gather(out, t, group=self.group)
            table = [o.cpu().tolist() for o in out]
        report = {"steps": self.steps, "sections": {}, "stragglers": {}}
        for j, n in enumerate(names):
            col = [row[j] for row in table]
            valid = [v for v in col if v == v]
            if not valid:
                continue
            med = statistics.median(valid)
            rel = [(med / v if v == v and v > 0 else float("nan")) for v in col]
            order = sorted(range(len(col)), key=lambda r: (col[r] != col[r], col[r]))
            k = min(self.minmax_count, len(order))
            report["sections"][n] = {"min_ms": min(valid), "median_ms": med, "max_ms": max(valid),
                                     "fastest_ranks": order[:k], "slowest_ranks": order[::-1][:k],
                                     "relative_perf_scores": rel}
            slow = [r for r, s in enumerate(rel) if s == s and s < self.rel_threshold]
            if slow:
                report["stragglers"][n] = slow
        # individual score: this rank against its own best window
        indiv = {}
        for j, n in enumerate(names):
            v = mine[j]
            if v == v and v > 0:
                best = min(self.best.get(n, v), v)
                self.best[n] = best
                indiv[n] = best / v
        report["individual_perf_scores"] = indiv
        report["individual_stragglers"] = sorted(n for n, s in indiv.items() if s < self.individual_threshold)
        self.window.clear()
        self.last_report = report
        if self.rank == 0:
            for n, s in report["sections"].items():
                self.printer(f"[straggler] step {self.steps} {n}: min {s['min_ms']:.2f} / median {s['median_ms']:.2f} / "
                             f"max {s['max_ms']:.2f} ms; slowest ranks {s['slowest_ranks'][:4]}")
            for n, ranks in report["stragglers"].items():
                self.printer(f"[straggler] step {self.steps} {n}: ranks {ranks} run below {self.rel_threshold:.2f} of the median speed")
        if report["individual_stragglers"]:
            self.printer(f"[straggler] rank {self.rank} step {self.steps}: slower than its own best in {report['individual_stragglers']}")
        return report


# ----------------------------------------------------------------------------- collective logging

_COLLECTIVES = ("all_reduce", "all_gather", "all_gather_into_tensor", "reduce_scatter", "reduce_scatter_tensor",
                "all_to_all_single", "broadcast", "reduce", "send", "recv", "barrier")


def _message_bytes(name: str, args, kwargs) -> int:
    def nbytes(x):
        if isinstance(x, torch.Tensor):
            return x.numel() * x.element_size()
        if isinstance(x, (list, tuple)):
            return sum(nbytes(v) for v in x)
        return 0
    if name in ("all_gather", "all_gather_into_tensor", "reduce_scatter", "reduce_scatter_tensor"):
        return max(nbytes(args[0]) if args else 0, nbytes(args[1]) if len(args) > 1 else 0)
    return nbytes(args[0]) if args else 0


def bus_bandwidth_factor(op: str, n: int) -> float:
    """busbw = algbw * factor (the convention of nccl-tests, which DeepSpeed's logger follows)."""
    if n <= 1:
        return 1.0
    if op == "all_reduce":
        return 2.0 * (n - 1) / n
    if op in ("all_gather", "all_gather_into_tensor", "reduce_scatter", "reduce_scatter_tensor", "all_to_all_single"):
        return (n - 1) / n
    return 1.0


class CommsLogger:
    def __init__(self, rank: int = 0, ops: Optional[Sequence[str]] = None, rank_stride: int = 1, world: int = 1,
                 verbose: bool = False, printer: Callable[[str], None] = print):
        self.rank, self.world = rank, world
        self.ops = set(ops) if ops else None                          # None = all collectives
        self.log_this_rank = rank % max(1, rank_stride) == 0
        self.verbose, self.printer = verbose, printer
        self.enabled = False
        self.records: Dict[str, Dict[int, List]] = defaultdict(dict)  # op -> bytes -> [count, [latencies ms]]
        self._pending = []
        self._orig = {}

    # -- patching ----------------------------------------------------------------
    def install(self) -> None:
        """Wrap the torch.distributed collectives (idempotent).  The wrappers time a call only while `enabled`."""
        if self._orig:
            return
        for name in _COLLECTIVES:
            fn = getattr(dist, name, None)
            if fn is None:
                continue
            self._orig[name] = fn
            setattr(dist, name, self._wrap(name, fn))

    def uninstall(self) -> None:
        for name, fn in self._orig.items():
            setattr(dist, name, fn)
        self._orig.clear()

    def _wrap(self, name, fn):
        logger = self

        def wrapped(*args, **kwargs):
            if not logger.enabled or (logger.ops is not None and name not in logger.ops):
                return fn(*args, **kwargs)
            size = _message_bytes(name, args, kwargs)
            on_gpu = torch.cuda.is_available() and any(isinstance(a, torch.Tensor) and a.is_cuda for a in args)
            if on_gpu:
                e0, e1 = EVENTS.get(), EVENTS.get()
                e0.record()
                out = fn(*args, **kwargs)
                e1.record()
                logger._pending.append((name, size, e0, e1))
            else:
                t0 = time.perf_counter()
                out = fn(*args, **kwargs)
                logger._add(name, size, (time.perf_counter() - t0) * 1e3)
            return out
        wrapped._sb_comms_original = fn
        return wrapped

    def _add(self, name: str, size: int, ms: float) -> None:
        rec = self.records[name].setdefault(size, [0, []])
        rec[0] += 1
        rec[1].append(ms)
        if self.verbose and self.log_this_rank:
            self.printer(f"COMMS-CALL:{name},{self.rank},{size},{ms:.4f}")

    def _drain(self) -> None:
        for name, size, e0, e1 in self._pending:
            e1.synchronize()
            self._add(name, size, e0.elapsed_time(e1))
            EVENTS.put(e0, e1)
        self._pending.clear()

    # -- output ------------------------------------------------------------------
    def serialize(self, ops: Optional[Sequence[str]] = None, prefix: str = "COMMS", reset: bool = True) -> List[str]:
        """`<prefix>:<op>,<rank>,<bytes>,<latency ms>,...` per (operation, message size), as the reference prints."""
        self._drain()
        lines = []
        for op in sorted(self.records):
            if ops is not None and op not in ops:
                continue
            for size in sorted(self.records[op]):
                lat = self.records[op][size][1]
                lines.append(f"{prefix}:{op},{self.rank},{size}," + ",".join(f"{v:.4f}" for v in lat))
        if self.log_this_rank:
            for ln in lines:
                self.printer(ln)
        if reset:
            self.records.clear()
        return lines

    def summary(self) -> Dict[str, Dict[int, Dict[str, float]]]:
        """Count, mean latency, algorithm and bus bandwidth (GB/s) per (operation, message size)."""
        self._drain()
        out: Dict[str, Dict[int, Dict[str, float]]] = {}
        for op, by_size in self.records.items():
            for size, (count, lat) in by_size.items():
                mean = sum(lat) / max(1, len(lat))
                alg = size / (mean * 1e-3) / 1e9 if mean > 0 else 0.0
                out.setdefault(op, {})[size] = {"count": count, "mean_ms": mean, "algbw_gbs": alg,
                                                "busbw_gbs": alg * bus_bandwidth_factor(op, self.world)}
        return out


# ----------------------------------------------------------------------------- allocator churn


class AllocStats:
    KEYS = ("num_alloc_retries", "num_device_alloc", "num_device_free")

    def __init__(self, rank: int = 0, enabled: bool = True, warmup_steps: int = 7, reader: Optional[Callable[[], Dict]] = None,
                 printer: Callable[[str], None] = print):
        self.rank, self.enabled, self.warmup = rank, enabled, warmup_steps
        self.reader = reader or (lambda: torch.cuda.memory_stats() if torch.cuda.is_available() else {})
        self.printer = printer
        self.last = None
        self.changes = 0

    def step(self, iteration: int) -> bool:
        """Returns True when the allocation counters moved since the previous step (after the warm-up steps)."""
        s = self.reader()
        stats = {k: s.get(k, 0) for k in self.KEYS}
        if iteration == self.warmup - 1 and torch.cuda.is_available():
            torch.cuda.empty_cache()                # one clean-up after the first steps have shown the working set
        changed = iteration > self.warmup and self.last is not None and stats != self.last
        if changed:
            self.changes += 1
            if self.enabled:
                self.printer(f"[rank={self.rank}] device allocations changed between iteration {iteration - 1} and {iteration} "
                             f"({self.last} -> {stats}): the caching allocator went back to the driver, which usually means "
                             "memory pressure and slower steps")
        self.last = stats
        return changed


# ----------------------------------------------------------------------------- wiring


def build_from_config(cfg, rank: int, world: int):
    """(straggler detector or None, comms logger or None, alloc watcher or None) for a training run."""
    det = None
    if cfg.heimdall_log_straggler or cfg.use_next:
        interval = cfg.heimdall_log_interval if cfg.heimdall_log_straggler else cfg.next_report_interval
        det = StragglerDetector(world, rank, interval=interval, minmax_count=cfg.heimdall_straggler_minmax_count,
                                rel_threshold=cfg.next_section_rel_threshold,
                                individual_threshold=cfg.next_section_individual_threshold)
    comms = None
    if cfg.deepspeed_enable_comms_logging:
        comms = CommsLogger(rank, cfg.deepspeed_comms_ops_to_log, cfg.deepspeed_comms_ranks_to_log or 1, world,
                            verbose=bool(cfg.deepspeed_comms_logging_verbose))
        comms.install()
        comms.enabled = True
    # every `mem_alloc_stats_ranks`-th rank reports (1 = all ranks); the others stay silent
    every = max(1, int(cfg.mem_alloc_stats_ranks or 1))
    alloc = AllocStats(rank, enabled=True) if cfg.print_mem_alloc_stats and rank % every == 0 else None
    return det, comms, alloc
