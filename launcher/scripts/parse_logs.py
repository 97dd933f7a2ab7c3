"""Scrape training logs into tables: per-iteration metrics, checkpoint save times, start-up time.

    python -m launcher.scripts.parse_logs train.log [more.log ...] [--csv out.csv] [--what iterations|checkpoints|startup]

Lines understood (this framework's `utils/logging.py` and `ckpt/io.py`, and the reference's equivalents):
    ` iteration      12/    1000 | ... | lm_loss: 2.345E+00 | ... tokens/s/gpu: 4.1E+04 | ...`   any `name: value` pairs
    `SAVE_CHECKPOINT: iteration: 500, ckpt saving takes 12.3 seconds`
    `time (ms) | model and optimizer: 1234.5 | train/valid/test data iterators: 56.7`             start-up timers
Role of the reference's launcher/scripts/parse_checkpoint_times.py:6-24, search_logs.py, parse_hsd_logs.py and the
`search_*_times.sh` greps.  Output is a list of dicts (and optionally a CSV); no pandas needed.
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from typing import Dict, List

ITER = re.compile(r"iteration\s+(\d+)\s*/\s*(\d+)\s*\|(.*)")
PAIR = re.compile(r"([A-Za-z_][\w /().-]*?):\s*([-+]?\d[\d.]*(?:[eE][-+]?\d+)?)")
CKPT = re.compile(r"SAVE_CHECKPOINT: iteration: (\d+), ckpt saving takes ([\d.]+) seconds")
STARTUP = re.compile(r"time \(ms\)\s*\|(.*)")


def parse_iterations(lines) -> List[Dict]:
    rows = []
    for line in lines:
        m = ITER.search(line)
        if not m:
            continue
        row = {"iteration": int(m.group(1)), "train_iters": int(m.group(2))}
        for part in m.group(3).split("|"):
            pm = PAIR.search(part)
            if pm:
                row[pm.group(1).strip().replace(" ", "_")] = float(pm.group(2))
        rows.append(row)
    return rows


def parse_checkpoint_times(lines) -> List[Dict]:
    return [{"iteration": int(m.group(1)), "checkpoint_time": float(m.group(2))} for m in map(CKPT.search, lines) if m]


def parse_startup(lines) -> List[Dict]:
    rows = []
    for line in lines:
        m = STARTUP.search(line)
        if not m or "iteration" in line:
            continue
        row = {}
        for part in m.group(1).split("|"):
            pm = PAIR.search(part)
            if pm:
                row[pm.group(1).strip().replace(" ", "_")] = float(pm.group(2))
        if row:
            rows.append(row)
    return rows


def describe(rows: List[Dict], key: str) -> Dict[str, float]:
    vals = sorted(r[key] for r in rows if key in r)
    if not vals:
        return {}
    n = len(vals)
    return {"count": n, "mean": sum(vals) / n, "min": vals[0], "median": vals[n // 2], "max": vals[-1]}


def write_csv(rows: List[Dict], path: str) -> None:
    keys: List[str] = []
    for r in rows:
        for k in r:
            if k not in keys:
                keys.append(k)
    with open(path, "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=keys)
        w.writeheader()
        w.writerows(rows)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--what", choices=["iterations", "checkpoints", "startup"], default="iterations")
    ap.add_argument("--csv", default=None)
    a = ap.parse_args(argv)
    lines: List[str] = []
    for p in a.logs:
        with open(p, errors="replace") as fh:
            lines.extend(fh)
    rows = {"iterations": parse_iterations, "checkpoints": parse_checkpoint_times, "startup": parse_startup}[a.what](lines)
    if a.csv:
        write_csv(rows, a.csv)
    for r in rows[:5] + ([{"...": "..."}] if len(rows) > 10 else []) + (rows[-5:] if len(rows) > 5 else []):
        print(r)
    if a.what == "checkpoints":
        print(describe(rows, "checkpoint_time"))
    print(f"{len(rows)} rows", file=sys.stderr)
    return rows


if __name__ == "__main__":
    main()
