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

from ..data.indexed_dataset import make_builder

_TOK = None


class _Cfg:
    def __init__(self, a):
        self.tokenizer_type, self.vocab_file, self.merge_file = a.tokenizer_type, a.vocab_file, a.merge_file
        self.make_vocab_size_divisible_by, self.model_parallel_size, self.padded_vocab_size = 8, 1, None


_FIX = None


def _init(args):
    global _TOK, _FIX
    from ..data.tokenizer import build_tokenizer
    _TOK = build_tokenizer(_Cfg(args))
    if getattr(args, "ftfy", False):
        try:
            import ftfy
        except ImportError as exc:
            raise SystemExit("--ftfy needs the ftfy package, which is not installed") from exc
        _FIX = ftfy.fix_text


def _encode(payload):
    line, keys, append_eod, enforce_len = payload
    line = line.strip()
    if not line:
        return None, 0
    doc = json.loads(line)
    out = {}
    for k in keys:
        ids = list(_TOK.tokenize(_FIX(doc[k]) if _FIX is not None else doc[k]))
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
    ap.add_argument("--num-docs", type=int, default=None, help="number of input documents, if known: progress is then "
                    "reported as a share of it")
    ap.add_argument("--ftfy", action="store_true", help="repair mis-decoded text with ftfy before tokenizing")
    ap.add_argument("--dataset-impl", default="mmap", choices=["mmap", "lazy", "cached"],
                    help="on-disk format: memory-mapped (default) or the older index format read lazily / cached")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--log-interval", type=int, default=10000)
    a = ap.parse_args(argv)
    _init(a)
    vocab = _TOK.vocab_size
    os.makedirs(os.path.dirname(os.path.abspath(a.output_prefix)), exist_ok=True)
    builders = {k: make_builder(f"{a.output_prefix}_{k}_document.bin", impl=a.dataset_impl, vocab_size=vocab)
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
            share = f" = {100.0 * n / a.num_docs:.1f} %" if a.num_docs else ""
            print(f"processed {n} documents{share} ({n / dt:.1f} docs/s, {nbytes / dt / 1e6:.2f} MB/s)", flush=True)
    if pool is not None:
        pool.close()
    for k, b in builders.items():
        b.finalize(f"{a.output_prefix}_{k}_document.idx")
    print(f"wrote {n} documents to {a.output_prefix}_*_document.(bin|idx)")


if __name__ == "__main__":
    main()
