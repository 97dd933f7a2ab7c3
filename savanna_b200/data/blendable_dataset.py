"""Weighted mixture of datasets (reference: savanna/data/blendable_dataset.py:9-60): sample i comes from
the dataset whose realised share lags its weight the most (C++ greedy index builder)."""
from __future__ import annotations

import numpy as np
import torch

from . import helpers


class BlendableDataset(torch.utils.data.Dataset):
    def __init__(self, datasets, weights):
        if len(datasets) != len(weights) or not datasets:
            raise ValueError("one weight per dataset is required")
        self.datasets = datasets
        w = np.asarray(weights, dtype=np.float64)
        if w.sum() <= 0:
            raise ValueError("weights must sum to a positive number")
        w = w / w.sum()
        self.size = int(sum(len(d) for d in datasets))
        self.dataset_index, self.dataset_sample_index = helpers.build_blending_indices(w, self.size)

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        d = int(self.dataset_index[idx])
        s = int(self.dataset_sample_index[idx])
        ds = self.datasets[d]
        return ds[s % len(ds)]
