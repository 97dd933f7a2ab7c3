"""Check, and repair, the stored length of Hyena-MR explicit filters (`mixer.mixer.filter.h`) in a checkpoint after a
context-length extension.

    python -m launcher.scripts.filter_lens check <dir> --num-groups 256 --seq-len 8192 --target-seq-len 32768
    python -m launcher.scripts.filter_lens fix   <dir> --num-groups 256 --seq-len 8192 --target-seq-len 32768

`<dir>` holds one `*model_states.pt` file (key `module`) and, for a universal checkpoint, `zero/<parameter name>/*.pt`
files (the fp32 weight and the Adam moments per parameter).  `check` verifies for every tensor whose name contains the
pattern: shape [num_groups, target_seq_len], zeros beyond `seq_len`, non-zero content before it.  `fix` zero-pads
tensors that still have the old shape [num_groups, seq_len] (or the same number of elements, flattened) to the target
shape and rewrites the files in place.  Role of the reference's launcher/scripts/check_filter_lens.py:14-62 and
fix_filter_lens.py.
"""
from __future__ import annotations

import argparse
import glob
import os
from typing import Dict, List

import torch

PATTERN = "mixer.mixer.filter.h"


def _files(ckpt_dir: str, pat: str):
    models = sorted(glob.glob(os.path.join(ckpt_dir, "*model_states.pt")))
    zero = sorted(p for p in glob.glob(os.path.join(ckpt_dir, "zero", "**", "*.pt"), recursive=True) if pat in p)
    return models, zero


def _check_tensor(name: str, w: torch.Tensor, G: int, L: int, LT: int) -> List[str]:
    bad = []
    if w.dim() != 2 or tuple(w.shape) != (G, LT):
        return [f"{name}: shape {tuple(w.shape)} != {(G, LT)}"]
    if float(w[:, L:].abs().sum()) != 0.0:
        bad.append(f"{name}: non-zero values in the padding region [{L}:{LT})")
    if float(w[:, :L].abs().sum()) == 0.0:
        bad.append(f"{name}: only zeros in the filter region [0:{L})")
    return bad


def check(ckpt_dir: str, num_groups: int, seq_len: int, target_seq_len: int, pat: str = PATTERN) -> List[str]:
    models, zero = _files(ckpt_dir, pat)
    problems: List[str] = []
    for mf in models:
        module = torch.load(mf, map_location="cpu", weights_only=False)["module"]
        for k, w in module.items():
            if pat in k:
                problems += _check_tensor(f"{os.path.basename(mf)}:{k}", w, num_groups, seq_len, target_seq_len)
    for zf in zero:
        sd = torch.load(zf, map_location="cpu", weights_only=False)
        items = sd.items() if isinstance(sd, dict) else [("param", sd)]
        for k, w in items:
            if hasattr(w, "shape") and w.numel() > 1:
                problems += _check_tensor(f"{os.path.relpath(zf, ckpt_dir)}:{k}", w, num_groups, seq_len, target_seq_len)
    return problems


def _pad(w: torch.Tensor, G: int, L: int, LT: int) -> torch.Tensor:
    if tuple(w.shape) == (G, LT):
        return w
    if w.numel() != G * L:
        raise ValueError(f"tensor of shape {tuple(w.shape)} is neither [{G}, {L}] nor [{G}, {LT}]")
    out = torch.zeros(G, LT, dtype=w.dtype)
    out[:, :L] = w.reshape(G, L)
    return out


def fix(ckpt_dir: str, num_groups: int, seq_len: int, target_seq_len: int, pat: str = PATTERN) -> Dict[str, int]:
    models, zero = _files(ckpt_dir, pat)
    changed = {"model_tensors": 0, "zero_tensors": 0}
    for mf in models:
        sd = torch.load(mf, map_location="cpu", weights_only=False)
        touched = False
        for k in list(sd["module"].keys()):
            if pat in k:
                new = _pad(sd["module"][k], num_groups, seq_len, target_seq_len)
                if new is not sd["module"][k]:
                    sd["module"][k] = new
                    changed["model_tensors"] += 1
                    touched = True
                    for grp in sd.get("param_shapes") or []:
                        if k in grp:
                            grp[k] = new.shape
        if touched:
            torch.save(sd, mf)
    for zf in zero:
        sd = torch.load(zf, map_location="cpu", weights_only=False)
        if isinstance(sd, dict):
            touched = False
            for k in list(sd.keys()):
                if hasattr(sd[k], "shape") and sd[k].numel() > 1:
                    new = _pad(sd[k], num_groups, seq_len, target_seq_len)
                    if new is not sd[k]:
                        sd[k], touched = new, True
                        changed["zero_tensors"] += 1
            if touched:
                torch.save(sd, zf)
        elif hasattr(sd, "shape"):
            new = _pad(sd, num_groups, seq_len, target_seq_len)
            if new is not sd:
                torch.save(new, zf)
                changed["zero_tensors"] += 1
    return changed


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("action", choices=["check", "fix"])
    ap.add_argument("checkpoint_dir")
    ap.add_argument("--num-groups", type=int, default=256)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--target-seq-len", type=int, default=32768)
    ap.add_argument("--pat", default=PATTERN)
    a = ap.parse_args(argv)
    if a.action == "fix":
        print(fix(a.checkpoint_dir, a.num_groups, a.seq_len, a.target_seq_len, a.pat))
    problems = check(a.checkpoint_dir, a.num_groups, a.seq_len, a.target_seq_len, a.pat)
    for p in problems:
        print("PROBLEM:", p)
    print("filter lengths OK" if not problems else f"{len(problems)} problems")
    return problems


if __name__ == "__main__":
    main()
