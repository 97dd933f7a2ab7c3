"""Memory-mapped token datasets in the Megatron `.bin` / `.idx` format
(reference: savanna/data/indexed_dataset.py:336-579).

Index file: magic `MMIDIDX\\x00\\x00`, uint64 version 1, uint8 dtype code, uint64 number of sequences,
uint64 number of documents(+1), int32 sizes[n], int64 byte pointers[n], int64 doc_idx[ndocs].
Data file: the tokens of all sequences back to back.
"""
from __future__ import annotations

import os
import struct
from typing import List, Optional

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


def dtype_code(dtype) -> int:
    for k, v in DTYPES.items():
        if v == dtype:
            return k
    raise ValueError(f"dtype {dtype} has no code in the indexed dataset format")


def best_fitting_dtype(vocab_size: Optional[int]):
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


def index_file_path(prefix: str) -> str:
    return prefix + ".idx"


def data_file_path(prefix: str) -> str:
    return prefix + ".bin"


class _Index:
    def __init__(self, path: str):
        with open(path, "rb") as fh:
            if fh.read(9) != _MAGIC:
                raise ValueError(f"{path} is not an mmap index file (bad magic)")
            (version,) = struct.unpack("<Q", fh.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", fh.read(1))
            self.dtype = DTYPES[code]
            self.itemsize = np.dtype(self.dtype).itemsize
            (self.n,) = struct.unpack("<Q", fh.read(8))
            (self.ndocs,) = struct.unpack("<Q", fh.read(8))
            offset = fh.tell()
        self._mm = np.memmap(path, mode="r", order="C")
        buf = memoryview(self._mm)
        self.sizes = np.frombuffer(buf, dtype=np.int32, count=self.n, offset=offset)
        self.pointers = np.frombuffer(buf, dtype=np.int64, count=self.n, offset=offset + self.sizes.nbytes)
        self.doc_idx = np.frombuffer(buf, dtype=np.int64, count=self.ndocs,
                                     offset=offset + self.sizes.nbytes + self.pointers.nbytes)

    def __len__(self):
        return self.n


class MMapIndexedDataset(torch.utils.data.Dataset):
    def __init__(self, prefix: str, skip_warmup: bool = True):
        self.prefix = prefix
        self._index = _Index(index_file_path(prefix))
        self._bin = np.memmap(data_file_path(prefix), mode="r", order="C")
        self._buf = memoryview(self._bin)
        if not skip_warmup:
            with open(data_file_path(prefix), "rb") as fh:      # touch the pages once
                while fh.read(100 * 1024 * 1024):
                    pass

    def __len__(self):
        return len(self._index)

    @property
    def sizes(self):
        return self._index.sizes

    @property
    def doc_idx(self):
        return self._index.doc_idx

    @property
    def dtype(self):
        return self._index.dtype

    def __getitem__(self, idx):
        if isinstance(idx, (int, np.integer)):
            return self.get(int(idx))
        if isinstance(idx, slice):
            return [self.get(i) for i in range(*idx.indices(len(self)))]
        raise TypeError("index must be an int or a slice")

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        size = int(self._index.sizes[idx])
        if length is None:
            length = size - offset
        ptr = int(self._index.pointers[idx]) + offset * self._index.itemsize
        return np.frombuffer(self._buf, dtype=self._index.dtype, count=length, offset=ptr)

    @staticmethod
    def exists(prefix: str) -> bool:
        return os.path.exists(index_file_path(prefix)) and os.path.exists(data_file_path(prefix))


class MMapIndexedDatasetBuilder:
    def __init__(self, out_bin: str, dtype=np.uint16):
        self._fh = open(out_bin, "wb")
        self.dtype = dtype
        self.sizes: List[int] = []
        self.doc_idx: List[int] = [0]

    def add_item(self, tokens) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        self._fh.write(arr.tobytes(order="C"))
        self.sizes.append(arr.size)

    def end_document(self) -> None:
        self.doc_idx.append(len(self.sizes))

    def merge_file_(self, other_prefix: str) -> None:
        idx = _Index(index_file_path(other_prefix))
        if idx.dtype != self.dtype:
            raise ValueError("cannot merge datasets of different dtypes")
        base = len(self.sizes)
        self.sizes.extend(int(s) for s in idx.sizes)
        self.doc_idx.extend(int(d) + base for d in idx.doc_idx[1:])
        with open(data_file_path(other_prefix), "rb") as fh:
            while True:
                chunk = fh.read(64 << 20)
                if not chunk:
                    break
                self._fh.write(chunk)

    def finalize(self, index_path: str) -> None:
        self._fh.close()
        sizes = np.asarray(self.sizes, dtype=np.int32)
        itemsize = np.dtype(self.dtype).itemsize
        pointers = np.zeros(len(sizes), dtype=np.int64)
        if len(sizes) > 1:
            np.cumsum(sizes[:-1].astype(np.int64) * itemsize, out=pointers[1:])
        with open(index_path, "wb") as fh:
            fh.write(_MAGIC)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<B", dtype_code(self.dtype)))
            fh.write(struct.pack("<Q", len(sizes)))
            fh.write(struct.pack("<Q", len(self.doc_idx)))
            fh.write(sizes.tobytes(order="C"))
            fh.write(pointers.tobytes(order="C"))
            fh.write(np.asarray(self.doc_idx, dtype=np.int64).tobytes(order="C"))


# ------------------------------------------------------------------------------------------------ legacy format
LEGACY_MAGIC = b"TNTIDX\x00\x00"
_LEGACY_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float32, 7: np.float64, 8: np.uint16}


def _legacy_code(dtype) -> int:
    for code, dt in _LEGACY_DTYPES.items():
        if np.dtype(dt) == np.dtype(dtype):
            return code
    raise ValueError(f"dtype {dtype} has no legacy code")


class IndexedDataset(torch.utils.data.Dataset):
    """The older (pre-mmap) fairseq-style format: `.idx` = magic `TNTIDX\\0\\0`, version 1 (u64), dtype code and element
    size (u64 each), number of items and of size entries (u64 each), document count (u64), then int64 arrays
    dim_offsets [n+1], data_offsets [n+1], sizes, doc_idx; `.bin` = the items back to back.  Items are read from the
    file on access (reference: savanna/data/indexed_dataset.py:129-225 `IndexedDataset`)."""

    def __init__(self, prefix: str):
        super().__init__()
        self.prefix = prefix
        self._file = None
        with open(index_file_path(prefix), "rb") as fh:
            if fh.read(8) != LEGACY_MAGIC:
                raise ValueError(f"{index_file_path(prefix)} is not a legacy (TNTIDX) index; is dataset_impl right?")
            (version,) = struct.unpack("<Q", fh.read(8))
            if version != 1:
                raise ValueError(f"unsupported legacy index version {version}")
            code, self.element_size = struct.unpack("<QQ", fh.read(16))
            self._dtype = np.dtype(_LEGACY_DTYPES[code])
            self._len, n_sizes = struct.unpack("<QQ", fh.read(16))
            (n_docs,) = struct.unpack("<Q", fh.read(8))
            rd = lambda n: np.frombuffer(fh.read(8 * n), dtype=np.int64).copy()          # noqa: E731
            self.dim_offsets, self.data_offsets = rd(self._len + 1), rd(self._len + 1)
            self._sizes, self._doc_idx = rd(n_sizes), rd(n_docs)

    def __len__(self):
        return int(self._len)

    @property
    def sizes(self):
        return self._sizes

    @property
    def doc_idx(self):
        return self._doc_idx

    @property
    def dtype(self):
        return self._dtype

    def _read(self, start_elem: int, count: int) -> np.ndarray:
        if self._file is None:
            self._file = open(data_file_path(self.prefix), "rb", buffering=0)
        out = np.empty(count, dtype=self._dtype)
        self._file.seek(int(start_elem) * self.element_size)
        self._file.readinto(out)
        return out

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            start, stop, step = idx.indices(len(self))
            if step != 1:
                raise ValueError("slices into an indexed dataset must be contiguous")
            sizes = self._sizes[self.dim_offsets[start]: self.dim_offsets[stop]]
            flat = self._read(self.data_offsets[start], int(sizes.sum()))
            return np.split(flat, np.cumsum(sizes)[:-1])
        if idx < 0 or idx >= self._len:
            raise IndexError("index out of range")
        shape = self._sizes[self.dim_offsets[idx]: self.dim_offsets[idx + 1]]
        return self._read(self.data_offsets[idx], int(np.prod(shape))).reshape(tuple(int(v) for v in shape))

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        item = self[idx]
        return item[offset: None if length is None else offset + length]

    def __del__(self):
        if getattr(self, "_file", None):
            self._file.close()

    @staticmethod
    def exists(prefix: str) -> bool:
        return os.path.exists(index_file_path(prefix)) and os.path.exists(data_file_path(prefix))

    @property
    def supports_prefetch(self) -> bool:
        return False


class IndexedCachedDataset(IndexedDataset):
    """Legacy format with an in-memory cache: `prefetch(indices)` reads the listed items into one array, `__getitem__`
    then serves them from memory (reference: savanna/data/indexed_dataset.py:228-283)."""

    def __init__(self, prefix: str):
        super().__init__(prefix)
        self.cache, self.cache_index = None, {}

    @property
    def supports_prefetch(self) -> bool:
        return True

    def prefetch(self, indices) -> None:
        indices = sorted(set(int(i) for i in indices))
        if all(i in self.cache_index for i in indices):
            return
        total = sum(int(self.data_offsets[i + 1] - self.data_offsets[i]) for i in indices)
        self.cache = np.empty(total, dtype=self._dtype)
        self.cache_index.clear()
        at = 0
        for i in indices:
            n = int(self.data_offsets[i + 1] - self.data_offsets[i])
            self.cache[at: at + n] = self._read(self.data_offsets[i], n)
            self.cache_index[i] = at
            at += n
        if self._file is not None:                     # the cache now serves the reads
            self._file.close()
            self._file = None

    def __getitem__(self, idx):
        if isinstance(idx, slice) or idx not in self.cache_index:
            return super().__getitem__(idx)
        shape = self._sizes[self.dim_offsets[idx]: self.dim_offsets[idx + 1]]
        n = int(np.prod(shape))
        at = self.cache_index[idx]
        return self.cache[at: at + n].copy().reshape(tuple(int(v) for v in shape))


class IndexedDatasetBuilder:
    """Writer of the legacy format (reference: savanna/data/indexed_dataset.py:286-327)."""

    def __init__(self, out_bin: str, dtype=np.int32):
        self._fh = open(out_bin, "wb")
        self.dtype = np.dtype(dtype)
        self.data_offsets, self.dim_offsets, self.sizes, self.doc_idx = [0], [0], [], [0]

    def add_item(self, tokens) -> None:
        arr = np.asarray(tokens, dtype=self.dtype)
        self._fh.write(arr.tobytes(order="C"))
        self.data_offsets.append(self.data_offsets[-1] + arr.size)
        self.sizes.extend(arr.shape)
        self.dim_offsets.append(self.dim_offsets[-1] + arr.ndim)

    def end_document(self) -> None:
        self.doc_idx.append(len(self.data_offsets) - 1)

    def merge_file_(self, other_prefix: str) -> None:
        other = IndexedDataset(other_prefix)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge datasets of different dtypes")
        begin, dim_begin, n_items = self.data_offsets[-1], self.dim_offsets[-1], len(self.data_offsets) - 1
        self.data_offsets.extend(int(begin + o) for o in other.data_offsets[1:])
        self.dim_offsets.extend(int(dim_begin + o) for o in other.dim_offsets[1:])
        self.sizes.extend(int(v) for v in other.sizes)
        self.doc_idx.extend(int(n_items + d) for d in other.doc_idx[1:])
        with open(data_file_path(other_prefix), "rb") as fh:
            while True:
                chunk = fh.read(1 << 24)
                if not chunk:
                    break
                self._fh.write(chunk)

    def finalize(self, index_path: str) -> None:
        self._fh.close()
        with open(index_path, "wb") as fh:
            fh.write(LEGACY_MAGIC)
            fh.write(struct.pack("<Q", 1))
            fh.write(struct.pack("<QQ", _legacy_code(self.dtype), self.dtype.itemsize))
            fh.write(struct.pack("<QQ", len(self.data_offsets) - 1, len(self.sizes)))
            fh.write(struct.pack("<Q", len(self.doc_idx)))
            for arr in (self.dim_offsets, self.data_offsets, self.sizes, self.doc_idx):
                fh.write(np.asarray(arr, dtype=np.int64).tobytes(order="C"))


def infer_dataset_impl(prefix: str) -> Optional[str]:
    """"cached" for a legacy index, "mmap" for the memory-mapped one, None when the file is neither or missing."""
    path = index_file_path(prefix)
    if not os.path.exists(path):
        return None
    with open(path, "rb") as fh:
        magic = fh.read(9)
    if magic[:8] == LEGACY_MAGIC:
        return "cached"
    if magic == _MAGIC:
        return "mmap"
    return None


def make_dataset(prefix: str, impl: str = "mmap", skip_warmup: bool = True):
    """`impl`: "mmap" (default), "lazy" / "cached" (legacy format, read on access / with a prefetch cache), or "infer"
    (decided by the index file's magic bytes)."""
    if impl == "infer":
        impl = infer_dataset_impl(prefix)
        if impl is None:
            raise FileNotFoundError(f"dataset {prefix}(.bin/.idx) does not exist or has an unknown index format")
    if impl == "mmap":
        if not MMapIndexedDataset.exists(prefix):
            raise FileNotFoundError(f"dataset {prefix}(.bin/.idx) does not exist")
        return MMapIndexedDataset(prefix, skip_warmup)
    if impl in ("lazy", "cached"):
        if not IndexedDataset.exists(prefix):
            raise FileNotFoundError(f"dataset {prefix}(.bin/.idx) does not exist")
        return IndexedDataset(prefix) if impl == "lazy" else IndexedCachedDataset(prefix)
    raise ValueError(f"dataset implementation {impl!r} is not supported (mmap, lazy, cached, infer)")


def make_builder(out_bin: str, impl: str = "mmap", vocab_size: Optional[int] = None):
    if impl == "mmap":
        return MMapIndexedDatasetBuilder(out_bin, dtype=best_fitting_dtype(vocab_size))
    return IndexedDatasetBuilder(out_bin)
