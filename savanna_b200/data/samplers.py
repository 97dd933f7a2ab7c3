"""Batch samplers (reference: savanna/data/samplers.py:6-143).

DistributedBatchSampler wraps a sequential sampler, groups `batch_size` (= micro batch x data-parallel
size) indices and yields this rank's slice — contiguous or interleaved — with `start_iter` fast-forward
for resume.
"""
from __future__ import annotations

import torch
from torch.utils import data


class RandomSampler(data.sampler.Sampler):
    """Seeded random sampler whose order depends on (epoch, seed) only, so every rank agrees."""

    def __init__(self, data_source, replacement=False, num_samples=None, seed: int = 0):
        self.data_source, self.replacement, self._num_samples = data_source, replacement, num_samples
        self.epoch, self.seed = -1, seed

    @property
    def num_samples(self):
        return len(self.data_source) if self._num_samples is None else self._num_samples

    def __iter__(self):
        n = len(self.data_source)
        g = torch.Generator()
        g.manual_seed(self.seed + max(self.epoch, 0))
        if self.replacement:
            return iter(torch.randint(high=n, size=(self.num_samples,), dtype=torch.int64, generator=g).tolist())
        return iter(torch.randperm(n, generator=g).tolist())

    def __len__(self):
        return self.num_samples

    def set_epoch(self, epoch):
        self.epoch = epoch


class DistributedBatchSampler(data.sampler.BatchSampler):
    def __init__(self, sampler, batch_size, drop_last, rank=-1, world_size=2, wrap_last=False, interleave=False):
        super().__init__(sampler, batch_size, drop_last)
        if rank == -1:
            rank = torch.distributed.get_rank()
        self.rank, self.world_size = rank, world_size
        self.sampler.wrap_around = 0
        self.wrap_around = 0
        self.wrap_last = wrap_last
        self.start_iter = 0
        self.interleave = interleave

    def __iter__(self):
        batch = []
        i = 0
        for idx in self.data_iterator(self.sampler, wrap_around=False):
            batch.append(idx)
            if len(batch) == self.batch_size:
                tbatch = self._batch(batch)
                if i >= self.start_iter:
                    yield tbatch
                    self.start_iter = 0
                i += 1
                batch = []
        if len(batch) > 0 and not self.drop_last:
            if self.wrap_last:
                self.sampler.wrap_around -= self.batch_size
                self.wrap_around += len(batch)
                self.wrap_around %= self.batch_size
            yield self._batch(batch)
        if self.wrap_last:
            self.sampler.wrap_around += self.batch_size

    def data_iterator(self, _iter, wrap_around=False):
        for i, idx in enumerate(_iter):
            if i < self.wrap_around % self.batch_size:
                continue
            if wrap_around:
                self.wrap_around += 1
                self.wrap_around %= self.batch_size
            yield idx

    def _batch(self, batch):
        if self.interleave:
            return batch[self.rank:self.batch_size:self.world_size]
        per = self.batch_size // self.world_size
        return batch[self.rank * per:(self.rank + 1) * per]
