"""Module input/output dumps for offline comparison of parallel layouts (reference: savanna/debug.py:16-63):
forward hooks save every leaf module's inputs and outputs under `debug_dir`, tagged with the parallel layout,
so two runs (e.g. tensor-parallel 1 vs 2) can be diffed tensor by tensor."""
from __future__ import annotations

import os

import torch

from ..parallel import state


def layout_tag(cfg) -> str:
    return f"mp{state.get_model_parallel_world_size()}_cp{state.get_context_parallel_world_size()}_" \
           f"mpr{state.get_model_parallel_rank()}_cpr{state.get_context_parallel_rank()}"


def _detach(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu()
    if isinstance(x, (tuple, list)):
        return [_detach(t) for t in x]
    return x


def register_debug_hooks(model: torch.nn.Module, cfg, max_calls: int = 1):
    root = os.path.join(cfg.debug_dir, layout_tag(cfg))
    os.makedirs(root, exist_ok=True)
    counts = {}
    handles = []

    def make(name):
        def hook(mod, inp, out):
            n = counts.get(name, 0)
            if n >= max_calls:
                return
            counts[name] = n + 1
            torch.save({"input": _detach(inp), "output": _detach(out)}, os.path.join(root, f"{name}.call{n}.pt"))
        return hook
    for name, mod in model.named_modules():
        if len(list(mod.children())) == 0:
            handles.append(mod.register_forward_hook(make(name or "root")))
    return handles


def diff_dumps(dir_a: str, dir_b: str, rtol: float = 1e-3, atol: float = 1e-5):
    """Compare two dump directories (one layout tag each, e.g. `<debug_dir>/mp1_cp1_mpr0_cpr0` of two runs) file by
    file: for every module call present in both, the largest absolute difference of the outputs and whether they agree
    within tolerance.  Shapes that differ (a tensor-parallel shard against the whole tensor) are reported as such and
    not compared.  Returns rows (file, max |a - b| or None, status) sorted by file name."""
    rows = []
    names = sorted(set(os.listdir(dir_a)) & set(os.listdir(dir_b)))
    for n in names:
        if not n.endswith(".pt"):
            continue
        a = torch.load(os.path.join(dir_a, n), map_location="cpu", weights_only=False)["output"]
        b = torch.load(os.path.join(dir_b, n), map_location="cpu", weights_only=False)["output"]
        ta = [t for t in (a if isinstance(a, list) else [a]) if isinstance(t, torch.Tensor)]
        tb = [t for t in (b if isinstance(b, list) else [b]) if isinstance(t, torch.Tensor)]
        if len(ta) != len(tb) or any(x.shape != y.shape for x, y in zip(ta, tb)):
            rows.append((n, None, "shape differs"))
            continue
        worst, ok = 0.0, True
        for x, y in zip(ta, tb):
            if x.numel() == 0:
                continue
            x, y = x.float(), y.float()
            worst = max(worst, float((x - y).abs().max()))
            ok = ok and bool(torch.allclose(x, y, rtol=rtol, atol=atol))
        rows.append((n, worst, "equal" if ok else "DIFFERENT"))
    only = sorted(set(os.listdir(dir_a)) ^ set(os.listdir(dir_b)))
    rows += [(n, None, "in one run only") for n in only if n.endswith(".pt")]
    return rows


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="Compare the module dumps of two runs (see register_debug_hooks).")
    ap.add_argument("dir_a")
    ap.add_argument("dir_b")
    ap.add_argument("--rtol", type=float, default=1e-3)
    ap.add_argument("--atol", type=float, default=1e-5)
    a = ap.parse_args(argv)
    bad = 0
    for name, worst, status in diff_dumps(a.dir_a, a.dir_b, a.rtol, a.atol):
        print(f"{status:16s} {'' if worst is None else f'{worst:.3e}':>10s}  {name}")
        bad += status == "DIFFERENT"
    raise SystemExit(1 if bad else 0)


if __name__ == "__main__":
    main()
