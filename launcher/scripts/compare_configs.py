"""Diff two configurations key by key.

    python -m launcher.scripts.compare_configs a.yml b.yml            raw YAML documents (nested keys as a/b/c)
    python -m launcher.scripts.compare_configs --resolved a.yml + extra.yml -- b.yml
                                                                       each side merged, validated and derived by the
                                                                       framework's loader; defaults included

Role of the reference's launcher/scripts/compare_configs.py:8-54 (raw diff); the resolved mode is an addition that also
shows differences hidden in defaults and derived values (batch triple, operator expansion, save iterations).
"""
from __future__ import annotations

import argparse
from typing import Any, Dict, List

import yaml


def compare_dicts(a: Dict[str, Any], b: Dict[str, Any], path: str = "") -> List[str]:
    out = []
    for key in sorted(set(a) | set(b), key=str):
        full = f"{path}/{key}" if path else str(key)
        if key not in b:
            out.append(f"{full} only in first")
        elif key not in a:
            out.append(f"{full} only in second")
        elif isinstance(a[key], dict) and isinstance(b[key], dict):
            out.extend(compare_dicts(a[key], b[key], full))
        elif a[key] != b[key]:
            out.append(f"{full} differs: {a[key]!r} != {b[key]!r}")
    return out


def _load_raw(paths: List[str]) -> Dict[str, Any]:
    doc: Dict[str, Any] = {}
    for p in paths:
        with open(p) as fh:
            for k, v in (yaml.load(fh, Loader=yaml.FullLoader) or {}).items():
                doc[str(k).replace("-", "_")] = v
    return doc


def _load_resolved(paths: List[str]) -> Dict[str, Any]:
    from savanna_b200.config import GlobalConfig
    cfg = GlobalConfig.from_ymls(paths, {"global_num_gpus": 1} if not any("global_num_gpus" in open(p).read() for p in paths) else {})
    return {k: v for k, v in vars(cfg).items() if not k.startswith("_") and k != "tokenizer"}


def compare(first: List[str], second: List[str], resolved: bool = False) -> List[str]:
    load = _load_resolved if resolved else _load_raw
    return compare_dicts(load(first), load(second))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--resolved", action="store_true")
    ap.add_argument("files", nargs="+", help="first side [-- second side]; without `--`: exactly two files")
    a = ap.parse_args(argv)
    if "--" in a.files:
        cut = a.files.index("--")
        first, second = a.files[:cut], a.files[cut + 1:]
    elif len(a.files) == 2:
        first, second = [a.files[0]], [a.files[1]]
    else:
        ap.error("give two files, or `first files -- second files`")
    first = [f for f in first if f != "+"]
    second = [f for f in second if f != "+"]
    diffs = compare(first, second, a.resolved)
    for d in diffs:
        print(d)
    print(f"{len(diffs)} differences")
    return diffs


if __name__ == "__main__":
    main()
