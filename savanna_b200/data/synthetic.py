"""Synthetic byte-level DNA source: tokens drawn uniformly from the ASCII codes of A, C, G, T.

Used by benchmarks, smoke tests and the tiny CPU baseline (no dataset files are needed).  Samples
have `seq_length + 1` tokens, like the packed samples of the indexed dataset.  Deterministic in
(seed, sample index), so resuming at a sample index reproduces the stream.
"""
from __future__ import annotations

import numpy as np
import torch

ACGT = np.array([65, 67, 71, 84], dtype=np.int64)


class SyntheticACGTDataset(torch.utils.data.Dataset):
    def __init__(self, num_samples: int, seq_length: int, seed: int = 0, lowercase_fraction: float = 0.0):
        self.n, self.L, self.seed, self.lower = int(num_samples), int(seq_length), int(seed), lowercase_fraction

    def __len__(self):
        return self.n

    def __getitem__(self, idx: int):
        rng = np.random.default_rng([self.seed, int(idx)])
        toks = ACGT[rng.integers(0, 4, size=self.L + 1)]
        if self.lower > 0:
            toks = np.where(rng.random(self.L + 1) < self.lower, toks + 32, toks)
        return {"text": toks.astype(np.int64)}


def acgt_batch(batch: int, seq_length: int, seed: int, device="cpu", pin: bool = False) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 4, (batch, seq_length + 1), generator=g)
    t = torch.from_numpy(ACGT)[idx]
    if pin and torch.cuda.is_available():
        t = t.pin_memory()
    return t.to(device) if device != "cpu" else t
