"""Expand a search specification into concrete model YAML files (reference: launcher/search_configs.py:58-117).
The specification is a YAML mapping `key: [v1, v2, ...]`; the cartesian product is applied on top of a base
model config, one output file per combination, named after the overridden values."""
from __future__ import annotations

import argparse
import itertools
import os

import yaml


def expand(base: dict, search: dict):
    keys = list(search)
    for combo in itertools.product(*[search[k] for k in keys]):
        cfg = dict(base)
        cfg.update(dict(zip(keys, combo)))
        tag = "_".join(f"{k.replace('_', '').replace('-', '')[:12]}{v}" for k, v in zip(keys, combo))
        yield tag, cfg


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--base", required=True)
    ap.add_argument("--search", required=True)
    ap.add_argument("--output-dir", required=True)
    a = ap.parse_args(argv)
    base = yaml.load(open(a.base), Loader=yaml.FullLoader)
    search = yaml.load(open(a.search), Loader=yaml.FullLoader)
    os.makedirs(a.output_dir, exist_ok=True)
    n = 0
    for tag, cfg in expand(base, search):
        with open(os.path.join(a.output_dir, f"{tag}.yml"), "w") as fh:
            yaml.safe_dump(cfg, fh, sort_keys=False)
        n += 1
    print(f"wrote {n} configs to {a.output_dir}")


if __name__ == "__main__":
    main()
