"""Host-side failure detection: a per-rank watchdog thread with a step deadline and a heartbeat file.

Every optimizer step calls `beat(iteration)`.  If no beat arrives within `timeout` seconds the watchdog
writes a poison file `<dir>/poison.rank<r>` naming the stalled iteration and terminates the process with a
non-zero exit code, so a launcher with restart-on-failure (torchrun --max-restarts, the relaunch loop of
launch_multinode.sh) resumes from the latest checkpoint; other ranks see the poison file at their next
beat and exit too instead of waiting inside a collective.  Poison files belong to one launch: each carries the
launch generation (`TORCHELASTIC_RESTART_COUNT`) in its name, `start()` removes this rank's leftovers, and a file
older than this watchdog's start is ignored, so a relaunch into the same heartbeat directory is not stopped by the
previous attempt's files.  Long host-side phases that are not steps (checkpoint save, evaluation) run inside
`paused()`, which suspends the deadline.  Nothing here touches a GPU: device-side waits
are bounded on their own (csrc/sm100.cuh) and report through a status word that `ops.cuda_ops.check_status`
turns into an exception.  The reference relies on external tools for this role (Heimdall /
nvidia_resiliency_ext straggler detectors and SLURM requeue, savanna/training.py:517-551).
"""
from __future__ import annotations

import contextlib
import glob
import os
import threading
import time
from typing import Callable, Optional


class Watchdog:
    def __init__(self, timeout: float, heartbeat_dir: Optional[str] = None, rank: int = 0,
                 on_timeout: Optional[Callable[[int], None]] = None, poll: float = 0.25):
        self.timeout, self.dir, self.rank, self.poll = float(timeout), heartbeat_dir, rank, poll
        self.on_timeout = on_timeout
        self._last = time.monotonic()
        self._iter = 0
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.fired = False
        self._paused = 0
        self.generation = os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")
        self._started_wall = time.time()
        if self.dir:
            os.makedirs(self.dir, exist_ok=True)

    # -- public ---------------------------------------------------------------
    def start(self) -> None:
        self._last = time.monotonic()
        self._started_wall = time.time()
        if self.dir:
            # leftovers of an earlier launch of this rank
            for p in glob.glob(os.path.join(self.dir, f"poison.rank{self.rank}")) + \
                    glob.glob(os.path.join(self.dir, f"poison.rank{self.rank}.gen*")) + \
                    [os.path.join(self.dir, f"heartbeat.rank{self.rank}")]:
                with contextlib.suppress(OSError):
                    os.remove(p)
        self._thread = threading.Thread(target=self._run, name=f"watchdog-{self.rank}", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def beat(self, iteration: int) -> None:
        self._last = time.monotonic()
        self._iter = iteration
        if self.dir:
            with open(os.path.join(self.dir, f"heartbeat.rank{self.rank}"), "w") as fh:
                fh.write(f"{iteration} {time.time():.3f}\n")
            poisoned = self.poisoned_by()
            if poisoned is not None and poisoned != self.rank:
                raise RuntimeError(f"rank {poisoned} reported a stalled step; stopping rank {self.rank}")

    @contextlib.contextmanager
    def paused(self):
        """Suspend the deadline around a host-side phase that is not a training step (checkpoint save, evaluation);
        the clock restarts when the phase ends."""
        self._paused += 1
        try:
            yield
        finally:
            self._last = time.monotonic()
            self._paused -= 1

    def _poison_path(self) -> str:
        return os.path.join(self.dir, f"poison.rank{self.rank}.gen{self.generation}")

    def poisoned_by(self) -> Optional[int]:
        """Rank that reported a stall in THIS launch (same generation, file not older than this watchdog), if any."""
        if not self.dir:
            return None
        for p in glob.glob(os.path.join(self.dir, "poison.rank*")):
            name = os.path.basename(p)[len("poison.rank"):]
            rank_s, _, gen = name.partition(".gen")
            try:
                rank = int(rank_s)
                if gen != self.generation or os.path.getmtime(p) < self._started_wall - 1.0:
                    continue
            except (ValueError, OSError):
                continue
            return rank
        return None

    # -- thread ---------------------------------------------------------------
    def _run(self) -> None:
        while not self._stop.wait(self.poll):
            if self._paused:
                self._last = time.monotonic()
                continue
            if time.monotonic() - self._last > self.timeout:
                self.fired = True
                if self.dir:
                    with open(self._poison_path(), "w") as fh:
                        fh.write(f"iteration {self._iter} exceeded {self.timeout}s\n")
                if self.on_timeout is not None:
                    self.on_timeout(self._iter)
                else:
                    print(f"[watchdog] rank {self.rank}: step after iteration {self._iter} exceeded "
                          f"{self.timeout}s; exiting", flush=True)
                    os._exit(17)
                return


class OverflowMonitor:
    """Abort after `n` consecutive skipped (overflowed) steps (reference: savanna/utils.py:702-716)."""

    def __init__(self, n: int = 50):
        self.n, self.history = n, []

    def check(self, skipped: bool) -> None:
        self.history.append(bool(skipped))
        self.history = self.history[-self.n:]
        if len(self.history) == self.n and all(self.history):
            raise RuntimeError(f"{self.n} consecutive steps were skipped because of overflow; aborting")
