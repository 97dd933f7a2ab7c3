import os

import numpy as np
import pytest
import torch

from savanna_b200.data import helpers
from savanna_b200.data.blendable_dataset import BlendableDataset
from savanna_b200.data.indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder
from savanna_b200.data.samplers import DistributedBatchSampler
from savanna_b200.data.sequence_dataset import SequenceDataset
from savanna_b200.data.synthetic import ACGT, SyntheticACGTDataset
from savanna_b200.data.tokenizer import CharLevelTokenizer, pad_vocab_size


def _make_dataset(tmp_path, ndocs=50, seed=0):
    rng = np.random.default_rng(seed)
    prefix = str(tmp_path / "ds")
    b = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    docs = []
    for _ in range(ndocs):
        n = int(rng.integers(5, 200))
        toks = rng.integers(0, 512, size=n)
        docs.append(toks)
        b.add_item(toks)
        b.end_document()
    b.finalize(prefix + ".idx")
    return prefix, docs


def test_indexed_dataset_roundtrip(tmp_path):
    prefix, docs = _make_dataset(tmp_path)
    ds = MMapIndexedDataset(prefix)
    assert len(ds) == len(docs)
    for i in (0, 7, len(docs) - 1):
        assert np.array_equal(ds[i], docs[i])
    assert np.array_equal(ds.get(3, offset=2, length=3), docs[3][2:5])
    assert ds.doc_idx[-1] == len(docs)


def test_sample_idx_native_matches_python():
    rng = np.random.default_rng(1)
    sizes = rng.integers(1, 300, size=400).astype(np.int32)
    doc_idx = np.tile(np.arange(400, dtype=np.int32), 3)
    rng.shuffle(doc_idx)
    tokens = int(sizes.sum())
    a = helpers.build_sample_idx(sizes, doc_idx, 64, 3, tokens, force_python=True)
    if helpers.native_available():
        b = helpers.build_sample_idx(sizes, doc_idx, 64, 3, tokens)
        assert np.array_equal(a, b)
    # every sample spans exactly seq_length + 1 tokens, consecutive samples overlap by one token
    flat_off = np.concatenate([[0], np.cumsum(sizes[doc_idx])])
    starts = flat_off[a[:, 0]] + a[:, 1]
    assert np.all(np.diff(starts) == 64)


def test_blending_indices():
    w = [0.5, 0.3, 0.2]
    ds, dss = helpers.build_blending_indices(w, 1000, force_python=True)
    if helpers.native_available():
        ds2, dss2 = helpers.build_blending_indices(w, 1000)
        assert np.array_equal(ds, ds2) and np.array_equal(dss, dss2)
    counts = np.bincount(ds, minlength=3) / 1000.0
    assert np.allclose(counts, w, atol=0.01)
    for d in range(3):
        assert np.array_equal(dss[ds == d], np.arange((ds == d).sum()))


def test_sequence_dataset_samples(tmp_path):
    prefix, docs = _make_dataset(tmp_path)
    ids = MMapIndexedDataset(prefix)
    sd = SequenceDataset("train", prefix, np.arange(len(docs), dtype=np.int32), ids, num_samples=40, seq_length=32, seed=3)
    assert len(sd) >= 40
    for i in range(0, 40, 7):
        s = sd[i]["text"]
        assert s.shape == (33,) and s.dtype == np.int64
    # the index caches are written once and reused
    files = [f for f in os.listdir(tmp_path) if f.endswith("_idx.npy")]
    assert len(files) == 3
    sd2 = SequenceDataset("train", prefix, np.arange(len(docs), dtype=np.int32), ids, 40, 32, 3)
    assert np.array_equal(sd[5]["text"], sd2[5]["text"])


def test_blendable_dataset():
    a = SyntheticACGTDataset(100, 8, seed=1)
    b = SyntheticACGTDataset(50, 8, seed=2)
    bl = BlendableDataset([a, b], [0.7, 0.3])
    assert len(bl) == 150
    assert set(np.unique(bl[0]["text"])) <= set(ACGT.tolist())


def test_distributed_batch_sampler_partitions():
    data = list(range(64))
    seen = []
    for rank in range(4):
        s = DistributedBatchSampler(torch.utils.data.SequentialSampler(data), 8, True, rank=rank, world_size=4)
        batches = list(s)
        assert all(len(b) == 2 for b in batches)
        seen.append([i for b in batches for i in b])
    assert sorted(i for r in seen for i in r) == data
    s = DistributedBatchSampler(torch.utils.data.SequentialSampler(data), 8, True, rank=1, world_size=4)
    s.start_iter = 3
    assert list(s)[0] == [26, 27]


def test_char_tokenizer_and_padding():
    t = CharLevelTokenizer(512)
    ids = t.tokenize("ACGT")
    assert ids == [65, 67, 71, 84] and t.detokenize(ids) == "ACGT"
    assert pad_vocab_size(512, 8, 2) == 512 and pad_vocab_size(500, 128, 2) == 512


def test_synthetic_is_deterministic():
    a, b = SyntheticACGTDataset(10, 16, seed=5), SyntheticACGTDataset(10, 16, seed=5)
    assert np.array_equal(a[3]["text"], b[3]["text"]) and not np.array_equal(a[3]["text"], a[4]["text"])


def test_dpo_preprocess_and_batch(tmp_path):
    """jsonl preference pairs -> indexed dataset -> batch -> direct-preference loss on the tiny CPU model."""
    import json
    import os
    import torch
    from savanna_b200.config import GlobalConfig
    from savanna_b200.data.indexed_dataset import MMapIndexedDataset
    from savanna_b200.tools import preprocess_data_dpo
    from savanna_b200.train.batch import build_batch_dpo
    from savanna_b200.train.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "pairs.jsonl"
    pairs = [{"text_accept": "ACGTACGTAC", "text_reject": "ACGTTTTT", "ref_logprob_accept": -12.5, "ref_logprob_reject": -9.25},
             {"text_accept": "GGGGCCCC", "text_reject": "GATTACAGATTACA", "ref_logprob_accept": -8.0, "ref_logprob_reject": -20.0}]
    src.write_text("\n".join(json.dumps(p) for p in pairs))
    prefix = str(tmp_path / "pairs")
    preprocess_data_dpo.main(["--input", str(src), "--output-prefix", prefix, "--seq-length", "64"])
    ds = MMapIndexedDataset(prefix + "_text_document")
    assert len(ds) == 2 and ds[0].dtype.name == "float32" and ds[0].shape[0] == 64
    cfg = GlobalConfig.from_ymls([os.path.join(root, "configs", "baseline", "tiny_sh2_cpu.yml")],
                                 {"global_num_gpus": 1, "seq_length": 32, "max_position_embeddings": 32,
                                  "alignment_method": "dpo", "dpo_beta": 0.5, "train_micro_batch_size_per_gpu": 2})
    tr = Trainer(cfg, load=False)
    rows = torch.stack([torch.from_numpy(ds[i].copy()) for i in range(2)])
    b = build_batch_dpo(cfg, rows)
    assert b["tokens"].shape == (4, 32) and b["ref_logps"].tolist() == [-12.5, -8.0, -9.25, -20.0]
    assert b["tokens"][0, :10].tolist() == [ord(c) for c in "ACGTACGTAC"] and b["tokens"][2, :8].tolist() == [ord(c) for c in "ACGTTTTT"]
    # the mask covers the text, not the eod padding
    assert int(b["loss_mask"][0].sum()) in (9, 10) and float(b["loss_mask"][0, 12:].sum()) == 0.0
    loss = tr.forward_step(b)
    assert loss.dim() == 0 and torch.isfinite(loss)
    loss.backward()
    batches = iter([{"text": rows}] * 4)
    l0 = float(tr.train_step(batches))
    assert l0 == l0
    # through the sample index: one record of dpo_data_seq_length float32 values per sample (plus the first value of the
    # next record, which the row parser never reaches), log-probabilities intact
    from savanna_b200.data.loaders import build_the_dataset
    cfg.dpo_data_seq_length = 64
    sd = build_the_dataset(prefix + "_text_document", "train", cfg, num_samples=3, seed=1)
    want = {(-12.5, -9.25), (-8.0, -20.0)}
    for i in range(len(sd)):
        r = sd[i]["text"]
        assert r.dtype.name == "float32" and r.shape == (65,)
        b2 = build_batch_dpo(cfg, torch.from_numpy(r.copy())[None])
        assert tuple(b2["ref_logps"].tolist()) in want
    cfg.dpo_data_seq_length = 48
    with pytest.raises(ValueError):
        build_the_dataset(prefix + "_text_document", "train", cfg, num_samples=3, seed=1)


def test_legacy_indexed_dataset_round_trip(tmp_path):
    """The pre-mmap format: builder -> lazy reader -> cached reader; slices, documents, merge, implementation inferred
    from the index magic."""
    import numpy as np
    from savanna_b200.data import indexed_dataset as ids
    docs = [[np.arange(5), np.arange(3) + 10], [np.arange(7) + 100]]
    prefix = str(tmp_path / "legacy")
    b = ids.make_builder(prefix + ".bin", impl="cached")
    for doc in docs:
        for item in doc:
            b.add_item(item)
        b.end_document()
    b.finalize(prefix + ".idx")
    assert ids.infer_dataset_impl(prefix) == "cached"
    lazy = ids.make_dataset(prefix, "lazy")
    assert len(lazy) == 3 and list(lazy.doc_idx) == [0, 2, 3] and list(lazy.sizes) == [5, 3, 7]
    assert np.array_equal(lazy[1], np.arange(3) + 10)
    parts = lazy[0:3]
    assert [len(p) for p in parts] == [5, 3, 7] and np.array_equal(parts[2], np.arange(7) + 100)
    assert np.array_equal(lazy.get(2, 2, 3), np.arange(7)[2:5] + 100)
    cached = ids.make_dataset(prefix, "infer")
    assert isinstance(cached, ids.IndexedCachedDataset) and cached.supports_prefetch
    cached.prefetch([2, 0])
    assert np.array_equal(cached[2], np.arange(7) + 100) and np.array_equal(cached[1], np.arange(3) + 10)
    # merge a second file behind the first
    p2 = str(tmp_path / "merged")
    b2 = ids.IndexedDatasetBuilder(p2 + ".bin")
    b2.add_item(np.array([1, 2]))
    b2.end_document()
    b2.merge_file_(prefix)
    b2.finalize(p2 + ".idx")
    m = ids.IndexedDataset(p2)
    assert len(m) == 4 and list(m.doc_idx) == [0, 1, 3, 4] and np.array_equal(m[3], np.arange(7) + 100)
    # the mmap format is still told apart
    p3 = str(tmp_path / "mm")
    b3 = ids.make_builder(p3 + ".bin", vocab_size=512)
    b3.add_item([1, 2, 3])
    b3.end_document()
    b3.finalize(p3 + ".idx")
    assert ids.infer_dataset_impl(p3) == "mmap" and isinstance(ids.make_dataset(p3, "infer"), ids.MMapIndexedDataset)


def test_build_blocks_mapping_cuts_documents_into_sentence_blocks():
    """Native block mapping: whole sentences per block, token budget reduced by the title, short and over-long
    documents skipped, rows shuffled reproducibly."""
    docs = np.array([0, 5, 6, 9, 12], dtype=np.int64)               # 4 documents: 5, 1, 3, 3 sentences
    sizes = np.array([4, 4, 4, 4, 4, 7, 3, 3, 3, 5, 600, 5], dtype=np.int32)
    titles = np.array([2, 1, 1, 1], dtype=np.int32)
    m = helpers.build_blocks_mapping(docs, sizes, titles, num_epochs=1, max_num_samples=100, max_seq_length=10, seed=3)
    rows = sorted(map(tuple, m.tolist()))
    # doc 0 (budget 8): sentences 0-1 reach 8 with 3 left -> block; 2-3 would leave one sentence (< 2), so 2-4 is the rest
    # doc 1: one sentence, skipped; doc 2 (budget 9): 3+3+3 = 9 at the last sentence -> one block; doc 3: a 600-token sentence
    assert rows == [(0, 2, 0, 0), (2, 5, 0, 1), (6, 9, 2, 2)]
    again = helpers.build_blocks_mapping(docs, sizes, titles, num_epochs=1, max_num_samples=100, max_seq_length=10, seed=3)
    assert np.array_equal(m, again)
    one = helpers.build_blocks_mapping(docs, sizes, titles, 1, 100, 10, 3, use_one_sent_blocks=True)
    assert (5, 6, 1, 3) in set(map(tuple, one.tolist())) or any(r[2] == 1 for r in one.tolist())
    two_epochs = helpers.build_blocks_mapping(docs, sizes, titles, 2, 100, 10, 3)
    assert len(two_epochs) == 6
    capped = helpers.build_blocks_mapping(docs, sizes, titles, 5, 4, 10, 3)
    assert len(capped) == 4
