"""GPT-style packed-sequence dataset over an indexed token dataset
(reference: savanna/data/sequence_dataset.py:11-294).

Samples of `seq_length + 1` tokens are cut across document boundaries from the documents visited in a
seeded shuffled order; three index arrays are built once and cached next to the data as
`<prefix>_<name>_indexmap_<ns>ns_<sl>sl_<seed>s_{doc,sample,shuffle}_idx.npy`:
    doc_idx     document order over all epochs
    sample_idx  (position in doc_idx, token offset) of every sample start     [C++ builder]
    shuffle_idx sample permutation
Rank 0 builds the caches; the other ranks wait at a barrier and then memory-map them.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch
import torch.distributed as dist

from .. import print_rank_0
from . import helpers


def _num_tokens(documents, sizes) -> int:
    return int(np.sum(sizes[documents]))


def _num_epochs(tokens_per_epoch: int, seq_length: int, num_samples: int) -> int:
    epochs, total = 0, 0
    while True:
        epochs += 1
        total += tokens_per_epoch
        if (total - 1) // seq_length >= num_samples:
            return epochs


def _build_doc_idx(documents, num_epochs: int, rng: np.random.RandomState) -> np.ndarray:
    doc_idx = np.tile(np.asarray(documents, dtype=np.int32), num_epochs)
    rng.shuffle(doc_idx)
    return doc_idx


def _build_shuffle_idx(size: int, rng: np.random.RandomState) -> np.ndarray:
    dtype = np.uint32 if size < np.iinfo(np.uint32).max - 1 else np.int64
    idx = np.arange(size, dtype=dtype)
    rng.shuffle(idx)
    return idx


def build_index_mappings(name, data_prefix, documents, sizes, num_samples, seq_length, seed, use_shared_fs=True):
    tokens_per_epoch = _num_tokens(documents, sizes)
    num_epochs = _num_epochs(tokens_per_epoch, seq_length, num_samples)
    base = f"{data_prefix}_{name}_indexmap_{num_samples}ns_{seq_length}sl_{seed}s"
    paths = {k: f"{base}_{k}_idx.npy" for k in ("doc", "sample", "shuffle")}
    is_builder = (not dist.is_initialized()) or dist.get_rank() == 0 or \
                 (not use_shared_fs and int(os.environ.get("LOCAL_RANK", "0")) == 0)
    if is_builder and not all(os.path.isfile(p) for p in paths.values()):
        t0 = time.time()
        rng = np.random.RandomState(seed)
        doc_idx = _build_doc_idx(documents, num_epochs, rng)
        np.save(paths["doc"], doc_idx, allow_pickle=True)
        sample_idx = helpers.build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)
        np.save(paths["sample"], sample_idx, allow_pickle=True)
        np.save(paths["shuffle"], _build_shuffle_idx(sample_idx.shape[0] - 1, rng), allow_pickle=True)
        print_rank_0(f" > built index maps for {name} ({sample_idx.shape[0] - 1} samples, {num_epochs} epochs) "
                     f"in {time.time() - t0:.2f}s")
    if dist.is_initialized():
        flag = torch.zeros(1, device="cuda" if dist.get_backend() == "nccl" else "cpu")
        dist.all_reduce(flag)                     # everyone waits for the builder
    return tuple(np.load(paths[k], allow_pickle=True, mmap_mode="r") for k in ("doc", "sample", "shuffle"))


class SequenceDataset(torch.utils.data.Dataset):
    def __init__(self, name, data_prefix, documents, indexed_dataset, num_samples, seq_length, seed,
                 build_index=True, use_shared_fs=True, enforce_sample_length=False, sample_dtype=np.int64):
        self.name, self.ds = name, indexed_dataset
        self.seq_length, self.enforce = seq_length, enforce_sample_length
        self.sample_dtype = sample_dtype        # int64 token ids; float32 for preference rows (tokens + log-probabilities)
        if np.min(documents) < 0 or np.max(documents) >= len(indexed_dataset.sizes):
            raise ValueError("document ids out of range")
        if enforce_sample_length and np.any(np.asarray(indexed_dataset.sizes) != seq_length):
            # fixed-length records (preference rows): every sample is one whole record, so every document must be
            # exactly `seq_length` long (sample i then starts at document i, offset 0)
            raise ValueError(f"enforce_sample_length: {data_prefix} holds documents whose length is not {seq_length}; "
                             "the data needs to be rewritten at that record length")
        if build_index:
            self.doc_idx, self.sample_idx, self.shuffle_idx = build_index_mappings(
                name, data_prefix, documents, indexed_dataset.sizes, num_samples, seq_length, seed, use_shared_fs)
            self.shuffle_idx_len = self.shuffle_idx.shape[0] - 1
            self.sample_idx_len = self.sample_idx.shape[0] - 1
            if self.shuffle_idx_len != self.sample_idx_len:
                print_rank_0(f"WARNING: shuffle index length ({self.shuffle_idx_len}) != sample index length ({self.sample_idx_len})")

    def __len__(self):
        return min(self.shuffle_idx_len, self.sample_idx_len)

    def __getitem__(self, idx):
        idx = int(self.shuffle_idx[idx])
        f_doc, f_off = int(self.sample_idx[idx][0]), int(self.sample_idx[idx][1])
        l_doc, l_off = int(self.sample_idx[idx + 1][0]), int(self.sample_idx[idx + 1][1])
        if f_doc == l_doc:
            sample = self.ds.get(int(self.doc_idx[f_doc]), offset=f_off, length=l_off - f_off + 1)
        else:
            parts = [self.ds.get(int(self.doc_idx[f_doc]), offset=f_off)]
            for i in range(f_doc + 1, l_doc):
                parts.append(self.ds.get(int(self.doc_idx[i])))
            parts.append(self.ds.get(int(self.doc_idx[l_doc]), length=l_off + 1))
            sample = np.concatenate(parts)
        sample = np.asarray(sample, dtype=self.sample_dtype)
        if self.enforce and len(sample) != self.seq_length + 1:
            raise ValueError(f"sample {idx} has {len(sample)} tokens, expected {self.seq_length + 1}")
        return {"text": sample}
