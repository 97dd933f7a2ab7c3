"""Context-extension surgery on model states: Hyena-MR stores `filter.h` / `filter.decay` at the full
training sequence length although only the first `hyena_mr_len` taps are used, and Hyena-LI stores a time
index buffer `filter.t`; moving a checkpoint to a longer sequence length needs them re-sized
(reference: tools/7b/conversion/extend_filter.py:20-100).

    python -m savanna_b200.tools.extend_filter --input <file.pt> --output <file.pt> --seq-len 32768 [--taps 128]
"""
from __future__ import annotations

import argparse
import math

import torch


def extend_module(module: dict, new_len: int, taps: int = 128, decay_preset=(-2, 2), mp_rank: int = 0, mp_size: int = 1) -> dict:
    out = dict(module)
    for k, v in module.items():
        if k.endswith("mixer.mixer.filter.h"):
            G, old = v.shape
            h = torch.zeros(G, new_len, dtype=v.dtype)
            n = min(taps, old, new_len)
            h[:, :n] = v[:, :n]
            out[k] = h
        elif k.endswith("mixer.mixer.filter.decay"):
            G, old = v.shape
            # keep the first `taps` values exactly (they are the only ones used) and regenerate the tail on the new grid
            alpha = torch.logspace(decay_preset[0], decay_preset[1], G * mp_size)[mp_rank * G:(mp_rank + 1) * G, None]
            t = torch.linspace(0, 1, new_len)[None]
            d = torch.exp(-alpha * t).to(v.dtype)
            n = min(taps, old, new_len)
            d[:, :n] = v[:, :n]
            out[k] = d
        elif k.endswith("mixer.mixer.filter.t"):
            out[k] = torch.arange(new_len, dtype=torch.float32).view(1, 1, -1)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--seq-len", type=int, required=True)
    ap.add_argument("--taps", type=int, default=128)
    a = ap.parse_args(argv)
    sd = torch.load(a.input, map_location="cpu", weights_only=False)
    sd["module"] = extend_module(sd["module"], a.seq_len, a.taps)
    if sd.get("param_shapes"):
        for grp in sd["param_shapes"]:
            for name in list(grp.keys()):
                if name.endswith("filter.h") and name in sd["module"]:
                    grp[name] = sd["module"][name].shape
    torch.save(sd, a.output)
    print(f"wrote {a.output}")


if __name__ == "__main__":
    main()
