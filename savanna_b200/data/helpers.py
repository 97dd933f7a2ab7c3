"""ctypes binding of the C++ index builders (csrc/data_helpers.cpp) with pure-NumPy fallbacks of the
same algorithms (used when the library is not built; reference fallback: sequence_dataset.py:249-294)."""
from __future__ import annotations

import ctypes
import os

import numpy as np

_LIB = None
_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libsavanna_data.so")


def _lib():
    global _LIB
    if _LIB is None and os.path.exists(_PATH):
        _LIB = ctypes.CDLL(_PATH)
        P, I32, I64, D = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_double
        _LIB.sbd_build_sample_idx_int32.argtypes = [P, P, I64, I32, I64, P]
        _LIB.sbd_build_sample_idx_int64.argtypes = [P, P, I64, I32, I64, P]
        _LIB.sbd_build_blending_indices.argtypes = [P, P, P, I32, I64]
        _LIB.sbd_build_mapping.argtypes = [P, I64, P, I32, I64, I32, D, I32, I32, P]
        _LIB.sbd_build_mapping.restype = I64
        _LIB.sbd_build_blocks_mapping.argtypes = [P, I64, P, P, I32, I64, I32, I32, I32, I32, P]
        _LIB.sbd_build_blocks_mapping.restype = I64
    return _LIB


def native_available() -> bool:
    return _lib() is not None


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def build_sample_idx(sizes: np.ndarray, doc_idx: np.ndarray, seq_length: int, num_epochs: int, tokens_per_epoch: int,
                     force_python: bool = False) -> np.ndarray:
    """[(num_samples+1), 2] array of (index into doc_idx, token offset)."""
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    big = num_epochs * tokens_per_epoch >= 2 ** 31 - 1 or len(doc_idx) >= 2 ** 31 - 1
    dtype = np.int64 if big else np.int32
    out = np.zeros((num_samples + 1, 2), dtype=dtype)
    lib = None if force_python else _lib()
    if lib is not None:
        fn = lib.sbd_build_sample_idx_int64 if big else lib.sbd_build_sample_idx_int32
        rc = fn(_ptr(sizes), _ptr(doc_idx), len(doc_idx), seq_length, num_samples, _ptr(out))
        if rc != 0:
            raise RuntimeError("sample index builder ran out of documents")
        return out
    pos, offset = 0, 0
    for s in range(1, num_samples + 1):
        need = seq_length + 1
        while need > 0:
            avail = int(sizes[doc_idx[pos]]) - offset
            if avail >= need:
                offset += need - 1
                need = 0
            else:
                need -= avail
                pos += 1
                offset = 0
        out[s, 0], out[s, 1] = pos, offset
    return out


def build_blending_indices(weights, size: int, force_python: bool = False):
    w = np.ascontiguousarray(weights, dtype=np.float64)
    ds = np.zeros(size, dtype=np.uint8)
    ds_sample = np.zeros(size, dtype=np.int64)
    lib = None if force_python else _lib()
    if lib is not None:
        rc = lib.sbd_build_blending_indices(_ptr(ds), _ptr(ds_sample), _ptr(w), len(w), size)
        if rc != 0:
            raise RuntimeError("blending index builder rejected its arguments")
        return ds, ds_sample
    counts = np.zeros(len(w), dtype=np.int64)
    for i in range(size):
        denom = max(i, 1)
        err = w * denom - counts
        d = int(np.argmax(err))
        ds[i], ds_sample[i] = d, counts[d]
        counts[d] += 1
    return ds, ds_sample


def build_mapping(docs: np.ndarray, sizes: np.ndarray, num_epochs: int, max_num_samples: int, max_seq_length: int,
                  short_seq_prob: float, seed: int, min_num_sent: int = 2) -> np.ndarray:
    lib = _lib()
    if lib is None:
        raise RuntimeError("build_mapping needs the native data library (python -m savanna_b200.csrc.build)")
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    n = lib.sbd_build_mapping(_ptr(docs), len(docs), _ptr(sizes), num_epochs, max_num_samples, max_seq_length,
                              short_seq_prob, seed, min_num_sent, None)
    out = np.zeros((n, 3), dtype=np.int64)
    lib.sbd_build_mapping(_ptr(docs), len(docs), _ptr(sizes), num_epochs, max_num_samples, max_seq_length,
                          short_seq_prob, seed, min_num_sent, _ptr(out))
    return out


def build_blocks_mapping(docs: np.ndarray, sizes: np.ndarray, title_sizes: np.ndarray, num_epochs: int, max_num_samples: int,
                         max_seq_length: int, seed: int, use_one_sent_blocks: bool = False,
                         long_sentence_len: int = 512) -> np.ndarray:
    """Rows (first sentence, one past the last sentence, document, block id), shuffled: the documents' sentences cut
    into blocks of about `max_seq_length - title length` tokens (retrieval-style block datasets).  `docs` holds the
    sentence offset of every document plus the end (len = documents + 1), `sizes` the sentence lengths, `title_sizes`
    one length per document."""
    lib = _lib()
    if lib is None:
        raise RuntimeError("build_blocks_mapping needs the native data library (python -m savanna_b200.csrc.build)")
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    title_sizes = np.ascontiguousarray(title_sizes, dtype=np.int32)
    if len(title_sizes) != len(docs) - 1:
        raise ValueError("one title length per document is needed")
    min_sent = 1 if use_one_sent_blocks else 2
    args = (_ptr(docs), len(docs), _ptr(sizes), _ptr(title_sizes), num_epochs, max_num_samples, max_seq_length, seed,
            min_sent, long_sentence_len)
    n = lib.sbd_build_blocks_mapping(*args, None)
    out = np.zeros((n, 4), dtype=np.int64)
    lib.sbd_build_blocks_mapping(*args, _ptr(out))
    return out
