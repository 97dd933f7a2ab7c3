"""Train / validation / test iterators (reference: savanna/data/data_utils.py:336-844).

Only the data-reading ranks (tensor-parallel rank 0 and context-parallel rank 0 of each replica) build
loaders; the batch is broadcast to their peers inside `train.batch.get_batch`.  Sample counts follow the
reference arithmetic (train_iters * global batch, (train_iters // eval_interval + 1) * eval_iters * global
batch, eval_iters * global batch).  Resume: the sampler fast-forwards to the consumed-sample index derived
from `train_data_token_index` (token-based, so a changed batch size resumes at the same token) or from
the iteration.  `synthetic_data: acgt` needs no files.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from .. import print_rank_0
from ..parallel import state
from .blendable_dataset import BlendableDataset
from .indexed_dataset import make_dataset
from .samplers import DistributedBatchSampler
from .sequence_dataset import SequenceDataset
from .synthetic import SyntheticACGTDataset


def _collate(samples):
    return {"text": torch.from_numpy(np.stack([s["text"] for s in samples]))}


def make_data_loader(dataset, cfg, start_sample: int = 0):
    if dataset is None:
        return None
    dp, rank = state.get_data_parallel_world_size(), state.get_data_parallel_rank()
    global_batch = cfg.batch_size * dp
    sampler = torch.utils.data.SequentialSampler(dataset)
    bs = DistributedBatchSampler(sampler, global_batch, drop_last=True, rank=rank, world_size=dp)
    bs.start_iter = start_sample // global_batch
    return torch.utils.data.DataLoader(dataset, batch_sampler=bs, num_workers=cfg.num_workers, pin_memory=True,
                                       collate_fn=_collate, persistent_workers=False)


def get_train_valid_test_split_(splits_string: str, size: int):
    parts = [float(s) for s in splits_string.replace("/", ",").split(",")]
    while len(parts) < 3:
        parts.append(0.0)
    parts = parts[:3]
    total = sum(parts)
    if total <= 0:
        raise ValueError("split must have a positive sum")
    idx = [0]
    for p in parts:
        idx.append(idx[-1] + int(round(p / total * float(size))))
    diff = idx[-1] - size
    for i in range(1, len(idx)):
        idx[i] -= diff
    return idx


def _sample_format(cfg):
    """(sample length, dtype, enforce exact length).  Direct-preference rows are float32 records of
    `dpo_data_seq_length` + 1 values (two texts and their reference log-probabilities, written by
    tools/preprocess_data_dpo.py) and must come back whole; everything else is seq_length + 1 int64 token ids
    (reference: savanna/data/data_utils.py:211-221)."""
    if cfg.alignment_method == "dpo":
        if cfg.dpo_data_seq_length is None:
            raise ValueError("alignment_method dpo: set dpo_data_seq_length (the record length of the preference data)")
        return int(cfg.dpo_data_seq_length), np.float32, True
    return cfg.seq_length, np.int64, bool(cfg.enforce_sample_length)


def build_the_dataset(prefix, name, cfg, num_samples, seed, skip_warmup=True, build_index=True):
    ids = make_dataset(prefix, cfg.data_impl, skip_warmup)
    docs = np.arange(0, ids.sizes.shape[0], dtype=np.int32)
    length, dtype, enforce = _sample_format(cfg)
    return SequenceDataset(name, prefix, docs, ids, num_samples, length, seed, build_index=build_index,
                           use_shared_fs=cfg.use_shared_fs, enforce_sample_length=enforce, sample_dtype=dtype)


def build_train_valid_test_datasets(prefix, cfg, splits_string, nums, seed, skip_warmup=True):
    ids = make_dataset(prefix, cfg.data_impl, skip_warmup)
    total = ids.sizes.shape[0]
    splits = get_train_valid_test_split_(splits_string, total)
    length, dtype, enforce = _sample_format(cfg)
    out = []
    for i, name in enumerate(("train", "valid", "test")):
        if splits[i + 1] > splits[i] and nums[i] > 0:
            docs = np.arange(splits[i], splits[i + 1], dtype=np.int32)
            out.append(SequenceDataset(name, prefix, docs, ids, nums[i], length, seed, use_shared_fs=cfg.use_shared_fs,
                                       enforce_sample_length=enforce, sample_dtype=dtype))
        else:
            out.append(None)
    return out


def get_normalized_weights_and_num_samples(weights, num_samples):
    s = sum(weights)
    w = [x / s for x in weights]
    return w, [int(math.ceil(num_samples * x * 1.005)) for x in w]


def weights_by_num_docs(counts, alpha=0.3):
    """Multinomial re-weighting p_i ~ (n_i / sum n)^alpha, then scaled by 1 - p_i (data_utils.py)."""
    n = np.asarray(counts, dtype=np.float64)
    p = n / n.sum()
    q = p ** alpha
    q = q / q.sum()
    w = (1 - p) * q
    return list(w / w.sum())


def num_samples_triple(cfg):
    train_iters = cfg.train_iters or 0
    eval_iters = ((train_iters // cfg.eval_interval) + 1) * cfg.eval_iters if cfg.eval_interval else 0
    return [train_iters * cfg.train_batch_size, eval_iters * cfg.train_batch_size, cfg.eval_iters * cfg.train_batch_size]


def _cycle(loader):
    if loader is None:
        return None
    def gen():
        while True:
            for b in loader:
                yield b
    return gen()


def build_train_valid_test_data_iterators(cfg, trainer=None):
    """Returns (train, valid, test) iterators; non-reading ranks get iterators that yield None."""
    reader = state.get_model_parallel_rank() == 0 and state.get_context_parallel_rank() == 0
    nums = cfg.train_val_test_num_samples if (cfg.use_checkpoint_num_samples and cfg.train_val_test_num_samples) \
        else num_samples_triple(cfg)
    cfg.train_val_test_num_samples = nums
    print_rank_0(f" > samples: train {nums[0]}, validation {nums[1]}, test {nums[2]}")
    consumed = 0
    if cfg.train_data_token_index:
        consumed = int(cfg.train_data_token_index) // cfg.seq_length
    elif cfg.iteration:
        consumed = cfg.iteration * cfg.train_batch_size
    if not reader:
        def nones():
            while True:
                yield None
        return nones(), nones(), nones()
    train_ds = valid_ds = test_ds = None
    if cfg.synthetic_data:
        if cfg.synthetic_data != "acgt":
            raise ValueError(f"synthetic data source {cfg.synthetic_data!r} unknown")
        train_ds = SyntheticACGTDataset(max(nums[0], 1), cfg.seq_length, cfg.seed)
        valid_ds = SyntheticACGTDataset(max(nums[1], 1), cfg.seq_length, cfg.seed + 1)
        test_ds = SyntheticACGTDataset(max(nums[2], 1), cfg.seq_length, cfg.seed + 2)
    elif cfg.train_data_paths:
        def blend(paths, weights, n, name):
            if not paths:
                return None
            w, per = get_normalized_weights_and_num_samples(weights, n)
            dss = [build_the_dataset(p, f"{name}_{i}", cfg, per[i], cfg.seed, not cfg.mmap_warmup) for i, p in enumerate(paths)]
            if cfg.weight_by_num_documents:
                w = weights_by_num_docs([len(d.ds.doc_idx) - 1 for d in dss], cfg.weighted_sampler_alpha)
            return BlendableDataset(dss, w) if len(dss) > 1 else dss[0]
        train_ds = blend(cfg.train_data_paths, cfg.train_data_weights, nums[0], "train")
        valid_ds = blend(cfg.valid_data_paths, cfg.valid_data_weights, nums[1], "valid")
        test_ds = blend(cfg.test_data_paths, cfg.test_data_weights, nums[2], "test")
    elif cfg.data_path:
        train_ds, valid_ds, test_ds = build_train_valid_test_datasets(cfg.data_path, cfg, cfg.split, nums, cfg.seed,
                                                                      not cfg.mmap_warmup)
    else:
        raise ValueError("no data source: set synthetic_data, data_path or train_data_paths")
    cfg.do_train = int(train_ds is not None and (cfg.train_iters or 0) > 0) if cfg.do_train is None else cfg.do_train
    cfg.do_valid = int(valid_ds is not None and cfg.eval_iters > 0) if cfg.do_valid is None else cfg.do_valid
    cfg.do_test = int(test_ds is not None and cfg.eval_iters > 0) if cfg.do_test is None else cfg.do_test
    train = _cycle(make_data_loader(train_ds, cfg, consumed % max(1, len(train_ds)) if train_ds is not None else 0))
    valid = _cycle(make_data_loader(valid_ds, cfg))
    test = _cycle(make_data_loader(test_ds, cfg))
    return train, valid, test


def dataset_chart_name(path: str) -> str:
    """Short name of a validation set for logs: the reference names a chart after the third-last path component
    (savanna/training.py:1920-1936, `.../<name>/<split>/<file>`); shorter paths fall back to the file stem."""
    parts = [q for q in path.replace("\\", "/").split("/") if q]
    return parts[-3] if len(parts) >= 3 else (parts[-1] if parts else path)


def build_per_dataset_val_iterators(cfg):
    """One validation iterator per file of `per_ds_valid_data_paths` (else `valid_data_paths`), so that the loss of
    every data source is tracked on its own (reference: savanna/data/data_utils.py:732-844).  Returns a list of
    (name, path, iterator); ranks that do not read data get iterators that yield None."""
    paths = cfg.per_ds_valid_data_paths or cfg.valid_data_paths or []
    iters = cfg.eval_per_ds_iters or cfg.eval_iters
    reader = state.get_model_parallel_rank() == 0 and state.get_context_parallel_rank() == 0
    out = []
    for i, path in enumerate(paths):
        name = dataset_chart_name(path)
        if not reader:
            def nones():
                while True:
                    yield None
            out.append((name, path, nones()))
            continue
        n = max(1, iters) * cfg.train_batch_size
        ds = build_the_dataset(path, f"valid_per_ds_{i}", cfg, n, cfg.seed, not cfg.mmap_warmup)
        out.append((name, path, _cycle(make_data_loader(ds, cfg))))
    return out
