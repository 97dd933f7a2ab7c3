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


def make_dataset(prefix: str, impl: str = "mmap", skip_warmup: bool = True) -> MMapIndexedDataset:
    if not MMapIndexedDataset.exists(prefix):
        raise FileNotFoundError(f"dataset {prefix}(.bin/.idx) does not exist")
    if impl not in ("mmap", "infer"):
        raise ValueError(f"dataset implementation {impl!r} is not supported (only mmap)")
    return MMapIndexedDataset(prefix, skip_warmup)


def make_builder(out_bin: str, impl: str = "mmap", vocab_size: Optional[int] = None) -> MMapIndexedDatasetBuilder:
    return MMapIndexedDatasetBuilder(out_bin, dtype=best_fitting_dtype(vocab_size))
