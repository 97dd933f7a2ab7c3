"""Print the structure of checkpoint files: keys, tensor shapes / dtypes / norms, optional diff of two files
(reference: tools/inspect_checkpoints.py).

    python -m savanna_b200.tools.inspect_checkpoints <file-or-dir> [--diff other] [--values]
"""
from __future__ import annotations

import argparse
import os

import torch


def describe(obj, indent=0, values=False, out=None, max_items=400):
    out = [] if out is None else out
    pad = "  " * indent
    if isinstance(obj, torch.Tensor):
        s = f"{pad}Tensor{tuple(obj.shape)} {obj.dtype}"
        if values and obj.numel() and obj.is_floating_point():
            s += f" norm={obj.float().norm().item():.6g} mean={obj.float().mean().item():.3g}"
        out.append(s)
    elif isinstance(obj, dict):
        for i, (k, v) in enumerate(obj.items()):
            if i >= max_items:
                out.append(f"{pad}... ({len(obj) - max_items} more)")
                break
            if isinstance(v, (dict, list, tuple, torch.Tensor)):
                out.append(f"{pad}{k}:")
                describe(v, indent + 1, values, out, max_items)
            else:
                out.append(f"{pad}{k}: {str(v)[:100]}")
    elif isinstance(obj, (list, tuple)):
        out.append(f"{pad}{type(obj).__name__}[{len(obj)}]")
        for v in obj[:8]:
            describe(v, indent + 1, values, out, max_items)
    else:
        out.append(f"{pad}{str(obj)[:100]}")
    return out


def diff_modules(a: dict, b: dict, atol=0.0):
    lines = []
    for k in sorted(set(a) | set(b)):
        if k not in a:
            lines.append(f"only in second: {k}")
        elif k not in b:
            lines.append(f"only in first: {k}")
        elif isinstance(a[k], torch.Tensor):
            if a[k].shape != b[k].shape:
                lines.append(f"shape differs: {k} {tuple(a[k].shape)} vs {tuple(b[k].shape)}")
            else:
                d = (a[k].float() - b[k].float()).abs().max().item() if a[k].numel() else 0.0
                if d > atol:
                    lines.append(f"values differ: {k} max|d|={d:.4g}")
    return lines


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("path")
    ap.add_argument("--diff", default=None)
    ap.add_argument("--values", action="store_true")
    a = ap.parse_args(argv)
    paths = [a.path] if os.path.isfile(a.path) else sorted(os.path.join(a.path, f) for f in os.listdir(a.path) if f.endswith(".pt"))
    for p in paths:
        print(f"== {p}")
        sd = torch.load(p, map_location="cpu", weights_only=False)
        print("\n".join(describe(sd, values=a.values)))
    if a.diff:
        x = torch.load(paths[0], map_location="cpu", weights_only=False)
        y = torch.load(a.diff, map_location="cpu", weights_only=False)
        print("\n".join(diff_modules(x.get("module", x), y.get("module", y))) or "identical")


if __name__ == "__main__":
    main()
