"""Batch samplers for data-parallel loading.

`DistributedBatchSampler` cuts an index stream into global batches (micro batch x data-parallel size) and hands
each rank its share of every batch; `start_iter` skips whole global batches so a resumed run continues where the
token cursor of the checkpoint points.  `RandomSampler` is an epoch-seeded permutation every rank agrees on.
Same role as the reference's savanna/data/samplers.py (batch slicing per rank, interleaved or contiguous, resume by
iteration), written as plain index arithmetic: a batch is materialised with `itertools.islice`, the rank's share is
one slice, and nothing is carried between epochs.
"""
from __future__ import annotations

import itertools
from typing import Iterable, Iterator, List, Optional

import torch
from torch.utils.data import Sampler


class RandomSampler(Sampler):
    """Permutation (or draws with replacement) of `range(len(data_source))` that depends only on `seed + epoch`."""

    def __init__(self, data_source, replacement: bool = False, num_samples: Optional[int] = None, seed: int = 0):
        self.data_source = data_source
        self.replacement = replacement
        self.requested = num_samples
        self.seed = seed
        self.epoch = 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = max(0, int(epoch))

    def __len__(self) -> int:
        return len(self.data_source) if self.requested is None else self.requested

    def __iter__(self) -> Iterator[int]:
        gen = torch.Generator().manual_seed(self.seed + self.epoch)
        population = len(self.data_source)
        if self.replacement:
            order = torch.randint(population, (len(self),), generator=gen)
        else:
            order = torch.randperm(population, generator=gen)[: len(self)]
        return iter(order.tolist())


class DistributedBatchSampler(Sampler):
    """Yields, per global batch of `batch_size` indices drawn from `sampler`, the indices of data-parallel rank
    `rank` of `world_size`: a contiguous block (default) or every `world_size`-th index (`interleave`).  The first
    `start_iter` global batches are skipped without being yielded.  A trailing partial batch is dropped when
    `drop_last`, otherwise its share for this rank (possibly shorter, possibly empty) is yielded."""

    def __init__(self, sampler: Iterable[int], batch_size: int, drop_last: bool, rank: int = -1, world_size: int = 1,
                 interleave: bool = False):
        if batch_size % world_size != 0:
            raise ValueError(f"global batch {batch_size} is not divisible by the data-parallel size {world_size}")
        if rank < 0:
            rank = torch.distributed.get_rank()
        if not 0 <= rank < world_size:
            raise ValueError(f"rank {rank} outside the data-parallel group of size {world_size}")
        self.sampler = sampler
        self.batch_size = batch_size
        self.drop_last = drop_last
        self.rank, self.world_size = rank, world_size
        self.interleave = interleave
        self.start_iter = 0

    def share(self, global_batch: List[int]) -> List[int]:
        if self.interleave:
            return global_batch[self.rank::self.world_size]
        per_rank = self.batch_size // self.world_size
        return global_batch[self.rank * per_rank:(self.rank + 1) * per_rank]

    def __len__(self) -> int:
        n = len(self.sampler)                       # type: ignore[arg-type]
        full, rest = divmod(n, self.batch_size)
        total = full + (1 if rest and not self.drop_last else 0)
        return max(0, total - self.start_iter)

    def __iter__(self) -> Iterator[List[int]]:
        stream = iter(self.sampler)
        # resume: consume the indices of the batches that were already trained on
        skipped = self.start_iter * self.batch_size
        self.start_iter = 0                         # the skip applies to the pass that resumes, not to later epochs
        if skipped:
            next(itertools.islice(stream, skipped - 1, skipped), None)
        while True:
            global_batch = list(itertools.islice(stream, self.batch_size))
            if len(global_batch) < self.batch_size:
                if global_batch and not self.drop_last:
                    yield self.share(global_batch)
                return
            yield self.share(global_batch)
