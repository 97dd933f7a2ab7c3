"""Evaluate a checkpoint on every validation set separately and print one loss per data source.

Role of the reference's tools/evaluate_per_ds.py (run through its launcher with a data config and a model config):
build the model from the configs, load the checkpoint named by `load` / `iteration`, build one iterator per file of
`per_ds_valid_data_paths` (or `valid_data_paths`) and report lm loss and perplexity for each.

    python -m savanna_b200.tools.evaluate_per_ds data.yml model.yml [--iters N] [--json out.json] [--override k=v ...]
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Optional


def evaluate_per_dataset(cfg, iters: Optional[int] = None) -> Dict[str, Dict[str, float]]:
    from ..train.trainer import Trainer
    trainer = Trainer(cfg, load=cfg.load is not None)
    return trainer.evaluate_per_dataset(iters)


def format_table(results: Dict[str, Dict[str, float]]) -> str:
    w = max([len(k) for k in results] + [7])
    lines = [f"{'dataset':<{w}}  {'lm_loss':>10}  {'ppl':>12}"]
    for name, r in results.items():
        lines.append(f"{name:<{w}}  {r['lm_loss']:>10.5f}  {r['lm_loss_ppl']:>12.4f}")
    return "\n".join(lines)


def main(argv: Optional[List[str]] = None) -> Dict[str, Dict[str, float]]:
    import yaml
    from ..config import GlobalConfig
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("configs", nargs="+", help="YAML config files (data + model), merged in order")
    ap.add_argument("--iters", type=int, default=None, help="batches per dataset (default eval_per_ds_iters / eval_iters)")
    ap.add_argument("--json", default=None, help="also write the results to this file")
    ap.add_argument("--override", action="append", default=[], metavar="KEY=VALUE")
    a = ap.parse_args(argv)
    over = {}
    for kv in a.override:
        k, v = kv.split("=", 1)
        over[k] = yaml.safe_load(v)
    cfg = GlobalConfig.from_ymls(a.configs, over)
    res = evaluate_per_dataset(cfg, a.iters)
    from .. import print_rank_0
    print_rank_0(format_table(res))
    if a.json and (cfg.rank or 0) == 0:
        with open(a.json, "w") as f:
            json.dump(res, f, indent=1)
    return res


if __name__ == "__main__":
    main()
