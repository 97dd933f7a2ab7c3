"""Summarise the checkpoints under a save directory: steps, files, sizes, `latest`, upload markers, incomplete steps.

    python -m launcher.scripts.summarize_checkpoints /path/to/save [--csv files.csv] [--expect-mp 2 --expect-dp 4]

A step counts as complete when it holds one `mp_rank_XX_model_states.pt` per tensor-parallel rank (or the pipeline
layout's `layer_*` files) and one `*_optim_states.pt` per (data-parallel, tensor-parallel) pair; the expected counts are
read from the first model file unless given.  Role of the reference's launcher/scripts/collect_local_chkpts.py and the
`summarize_*` / `list_num_uploaded` shell helpers (which do the same against S3 buckets).
"""
from __future__ import annotations

import argparse
import csv
import os
import re
from typing import Dict, List, Optional

STEP = re.compile(r"^global_step(\d+)$")


def collect(save_dir: str) -> List[Dict]:
    rows = []
    for name in sorted(os.listdir(save_dir)):
        m = STEP.match(name)
        step_dir = os.path.join(save_dir, name)
        if not m or not os.path.isdir(step_dir):
            continue
        for root, _, files in os.walk(step_dir):
            for f in files:
                path = os.path.join(root, f)
                rows.append({"checkpoint_dir": save_dir, "step": int(m.group(1)), "filename": os.path.relpath(path, step_dir),
                             "size": os.path.getsize(path)})
    return rows


def summarize(save_dir: str, expect_mp: Optional[int] = None, expect_dp: Optional[int] = None) -> Dict:
    rows = collect(save_dir)
    steps: Dict[int, Dict] = {}
    for r in rows:
        s = steps.setdefault(r["step"], {"files": 0, "bytes": 0, "model": 0, "optim": 0, "layers": 0})
        s["files"] += 1
        s["bytes"] += r["size"]
        base = os.path.basename(r["filename"])
        if re.match(r"mp_rank_\d+_model_states\.pt$", base):
            s["model"] += 1
        elif base.endswith("_optim_states.pt"):
            s["optim"] += 1
        elif re.match(r"layer_\d+-model_\d+-model_states\.pt$", base):
            s["layers"] += 1
    latest = None
    lp = os.path.join(save_dir, "latest")
    if os.path.isfile(lp):
        with open(lp) as fh:
            latest = fh.read().strip()
    for step, s in steps.items():
        d = os.path.join(save_dir, f"global_step{step}")
        s["uploaded"] = os.path.exists(d + ".uploaded") or os.path.exists(os.path.join(d, ".uploaded"))
        s["uploading"] = os.path.exists(d + ".uploading") or os.path.exists(os.path.join(d, ".uploading"))
        mp = expect_mp or max(s["model"], 1)
        ok_model = s["model"] >= mp or s["layers"] > 0
        ok_optim = True if expect_dp is None else s["optim"] >= mp * expect_dp
        s["complete"] = bool(ok_model and ok_optim and s["files"] > 0)
    return {"save_dir": save_dir, "latest": latest, "steps": dict(sorted(steps.items())),
            "total_bytes": sum(s["bytes"] for s in steps.values()), "files": rows}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("save_dir")
    ap.add_argument("--csv", default=None)
    ap.add_argument("--expect-mp", type=int, default=None)
    ap.add_argument("--expect-dp", type=int, default=None)
    a = ap.parse_args(argv)
    res = summarize(a.save_dir, a.expect_mp, a.expect_dp)
    print(f"{len(res['files'])} files in {len(res['steps'])} checkpoints, {res['total_bytes'] / 1e9:.2f} GB; latest = {res['latest']}")
    for step, s in res["steps"].items():
        flags = ("complete" if s["complete"] else "INCOMPLETE") + (", uploaded" if s["uploaded"] else "") + \
                (", uploading" if s["uploading"] else "")
        print(f"  global_step{step}: {s['files']} files, {s['bytes'] / 1e9:.2f} GB, {s['model']} model / {s['optim']} optimizer "
              f"/ {s['layers']} layer files ({flags})")
    if a.csv:
        with open(a.csv, "w", newline="") as fh:
            w = csv.DictWriter(fh, fieldnames=["checkpoint_dir", "step", "filename", "size"])
            w.writeheader()
            w.writerows(res["files"])
    return res


if __name__ == "__main__":
    main()
