"""muP coordinate check: train the same architecture at several widths for a few steps and record the mean absolute
activation of every block, the embedding and the logits at every step.  Under a correct maximal-update
parametrisation the curves stay flat in the width; under standard parametrisation they grow.

Role of the reference's `mup_coord_check` (savanna/training.py:269-302, savanna/mup_substitute.py), which builds the
model at hidden sizes `num_attention_heads * 2^p`, p = 2..8, once with `use_mup` and once without, and plots both
sets.  Here the records are returned and written as CSV (no plotting library is assumed); `summarise` reduces them
to the width-growth exponent of every recorded module, which is what the plot is read for.

    python -m savanna_b200.train.mup_coord_check model.yml [--steps 3] [--powers 2 3 4] [--out coord_check.csv]
"""
from __future__ import annotations

import argparse
import math
from typing import Dict, Iterable, List, Optional


def _records_for_width(paths, over, width: int, use_mup: bool, steps: int, seed: int, base_width: Optional[int] = None) -> List[Dict]:
    import torch
    from ..config import GlobalConfig
    from ..data.synthetic import acgt_batch
    from ..parallel import state
    from .trainer import Trainer
    base = GlobalConfig.from_ymls(paths, dict(over))
    o = dict(over)
    o.update({"hidden_size": width, "use_mup": use_mup, "coord_check": False, "load": None, "save": None,
              "num_groups_hyena": width})
    if base_width:
        # the width multiplier of muP is this model's width over the narrowest one's (the base model of the sweep)
        o["mup_width_scale"] = max(1, width // base_width)
    for k in ("num_groups_hyena_medium", "num_groups_hyena_short"):
        g = getattr(base, k, None)
        if g:
            o[k] = g if width % g == 0 else width
    c = GlobalConfig.from_ymls(paths, o)
    if c.tokenizer is None:
        c.build_tokenizer()
    state.destroy_model_parallel()
    tr = Trainer(c, load=False)
    recs: List[Dict] = []
    cur = {"step": 0}

    def hook(name):
        def fn(_m, _a, out):
            t = out[0] if isinstance(out, (tuple, list)) else out
            if isinstance(t, torch.Tensor) and t.is_floating_point():
                recs.append({"width": width, "mup": int(use_mup), "step": cur["step"], "module": name,
                             "l1": float(t.detach().float().abs().mean())})
        return fn
    handles = [tr.model.embedding.register_forward_hook(hook("embedding"))]
    for i, b in enumerate(tr.model.blocks()):
        handles.append(b.register_forward_hook(hook(f"block{i}")))
    handles.append(tr.model.register_forward_hook(hook("logits")))

    def it():
        i = 0
        while True:
            yield {"text": acgt_batch(c.train_micro_batch_size_per_gpu, c.seq_length, seed=seed + i)}
            i += 1
    d = it()
    for s in range(steps):
        cur["step"] = s
        tr.train_step(d)
    for h in handles:
        h.remove()
    state.destroy_model_parallel()
    return recs


def coord_check(paths, over: Optional[Dict] = None, powers: Iterable[int] = range(2, 9), steps: int = 3,
                seed: int = 0) -> List[Dict]:
    """Records {width, mup, step, module, l1} for widths num_attention_heads * 2^p, with and without muP.  `paths` are
    the YAML files of the model, `over` values that override them (the width-dependent keys are set here)."""
    from ..config import GlobalConfig
    over = dict(over or {})
    over.setdefault("global_num_gpus", 1)
    heads = GlobalConfig.from_ymls(paths, dict(over)).num_attention_heads
    out: List[Dict] = []
    powers = list(powers)
    base_width = heads * (2 ** min(powers))
    for use_mup in (True, False):
        for p in powers:
            out += _records_for_width(list(paths), over, heads * (2 ** p), use_mup, steps, seed, base_width)
    return out


def summarise(records: List[Dict]) -> Dict[str, Dict[str, float]]:
    """Least-squares slope of log(l1) against log(width) at the last recorded step, per module, for muP and standard
    parametrisation: {"mup": {module: slope}, "sp": {module: slope}}."""
    res: Dict[str, Dict[str, float]] = {"mup": {}, "sp": {}}
    last = max(r["step"] for r in records)
    for key, flag in (("mup", 1), ("sp", 0)):
        mods = sorted({r["module"] for r in records})
        for m in mods:
            pts: Dict[int, List[float]] = {}
            for r in records:
                if r["mup"] == flag and r["module"] == m and r["step"] == last and r["l1"] > 0:
                    pts.setdefault(r["width"], []).append(r["l1"])
            if len(pts) < 2:
                continue
            xs = [math.log(w) for w in pts]
            ys = [math.log(sum(v) / len(v)) for v in pts.values()]
            mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
            den = sum((x - mx) ** 2 for x in xs)
            res[key][m] = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den if den else 0.0
    return res


def write_csv(records: List[Dict], path: str) -> None:
    with open(path, "w") as f:
        f.write("width,mup,step,module,l1\n")
        for r in records:
            f.write(f"{r['width']},{r['mup']},{r['step']},{r['module']},{r['l1']:.8e}\n")


def main(argv: Optional[List[str]] = None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("configs", nargs="+")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--powers", type=int, nargs="*", default=list(range(2, 9)))
    ap.add_argument("--out", default="coord_check.csv")
    a = ap.parse_args(argv)
    recs = coord_check(a.configs, {"global_num_gpus": 1}, a.powers, a.steps)
    write_csv(recs, a.out)
    s = summarise(recs)
    for key in ("mup", "sp"):
        print(f"[{key}] width exponent of mean |activation| at step {a.steps - 1}:")
        for m, v in s[key].items():
            print(f"   {m:<12} {v:+.3f}")
    return recs


if __name__ == "__main__":
    main()
