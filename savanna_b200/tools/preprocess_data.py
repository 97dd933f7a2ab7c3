"""jsonl -> `.bin` / `.idx` indexed dataset (reference: tools/preprocess_data.py).  Each input line is a JSON
object; the text under --jsonl-keys is tokenized (optionally with an end-of-document token appended) and stored
as one document.  Tokenization runs in a process pool.

    python -m savanna_b200.tools.preprocess_data --input data.jsonl --output-prefix out/mydata \
        --tokenizer-type CharLevelTokenizer --append-eod [--workers 8]
"""
from __future__ import annotations

import argparse
import json
import multiprocessing
import os
import time

import numpy as np

from ..data.indexed_dataset import MMapIndexedDatasetBuilder, best_fitting_dtype

_TOK = None


class _Cfg:
    def __init__(self, a):
        self.tokenizer_type, self.vocab_file, self.merge_file = a.tokenizer_type, a.vocab_file, a.merge_file
        self.make_vocab_size_divisible_by, self.model_parallel_size, self.padded_vocab_size = 8, 1, None


def _init(args):
    global _TOK
    from ..data.tokenizer import build_tokenizer
    _TOK = build_tokenizer(_Cfg(args))


def _encode(payload):
    line, keys, append_eod, enforce_len = payload
    line = line.strip()
    if not line:
        return None, 0
    doc = json.loads(line)
    out = {}
    for k in keys:
        ids = list(_TOK.tokenize(doc[k]))
        if append_eod:
            ids.append(_TOK.eod)
        if enforce_len and len(ids) != enforce_len:
            continue
        out[k] = ids
    return out, len(line)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True, help="jsonl file, or comma-separated list")
    ap.add_argument("--jsonl-keys", nargs="+", default=["text"])
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--tokenizer-type", default="CharLevelTokenizer")
    ap.add_argument("--vocab-file", default=None)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--append-eod", action="store_true")
    ap.add_argument("--enforce-sample-length", type=int, default=None)
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--log-interval", type=int, default=10000)
    a = ap.parse_args(argv)
    _init(a)
    vocab = _TOK.vocab_size
    os.makedirs(os.path.dirname(os.path.abspath(a.output_prefix)), exist_ok=True)
    builders = {k: MMapIndexedDatasetBuilder(f"{a.output_prefix}_{k}_document.bin", dtype=best_fitting_dtype(vocab))
                for k in a.jsonl_keys}

    def lines():
        for path in a.input.split(","):
            with open(path) as fh:
                for ln in fh:
                    yield (ln, a.jsonl_keys, a.append_eod, a.enforce_sample_length)
    t0, n, nbytes = time.time(), 0, 0
    if a.workers > 1:
        pool = multiprocessing.Pool(a.workers, initializer=_init, initargs=(a,))
        it = pool.imap(_encode, lines(), 25)
    else:
        pool, it = None, map(_encode, lines())
    for doc, nb in it:
        if not doc:
            continue
        for k, ids in doc.items():
            builders[k].add_item(np.asarray(ids))
            builders[k].end_document()
        n += 1
        nbytes += nb
        if n % a.log_interval == 0:
            dt = time.time() - t0
            print(f"processed {n} documents ({n / dt:.1f} docs/s, {nbytes / dt / 1e6:.2f} MB/s)", flush=True)
    if pool is not None:
        pool.close()
    for k, b in builders.items():
        b.finalize(f"{a.output_prefix}_{k}_document.idx")
    print(f"wrote {n} documents to {a.output_prefix}_*_document.(bin|idx)")


if __name__ == "__main__":
    main()
