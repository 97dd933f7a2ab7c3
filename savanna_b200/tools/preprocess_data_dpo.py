"""jsonl of preference pairs -> `.bin` / `.idx` dataset for direct-preference training (reference:
tools/preprocess_data_dpo.py).  Every input line holds `text_accept`, `text_reject` and the two log-probabilities of a
frozen reference model, `ref_logprob_accept`, `ref_logprob_reject`.  A document is the float32 row

    accept tokens, pad, reject tokens, pad, ref_logprob_accept, pad, ref_logprob_reject [, pad ... up to --seq-length]

which `train/batch.py:build_batch_dpo` splits again.  Training reads one record per sample, so every row has to have
the same length: give `--seq-length` and set the run's `dpo_data_seq_length` to the same number.  The pad token must not occur inside the texts (the byte-level
tokenizer's pad id 1 never does for printable text).

    python -m savanna_b200.tools.preprocess_data_dpo --input pairs.jsonl --output-prefix out/pairs --seq-length 1024
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from ..data.indexed_dataset import MMapIndexedDatasetBuilder


def encode_pair(doc: dict, tok, seq_length: int | None = None) -> np.ndarray:
    pad = float(tok.pad)
    a = [float(t) for t in tok.tokenize(doc["text_accept"])]
    r = [float(t) for t in tok.tokenize(doc["text_reject"])]
    row = a + [pad] + r + [pad, float(doc["ref_logprob_accept"]), pad, float(doc["ref_logprob_reject"])]
    if seq_length is not None:
        if len(row) > seq_length:
            raise ValueError(f"pair of {len(row)} entries does not fit --seq-length {seq_length}")
        row = row + [pad] * (seq_length - len(row))
    return np.asarray(row, dtype=np.float32)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True, help="jsonl file, or comma-separated list")
    ap.add_argument("--output-prefix", required=True)
    ap.add_argument("--tokenizer-type", default="CharLevelTokenizer")
    ap.add_argument("--vocab-file", default=None)
    ap.add_argument("--merge-file", default=None)
    ap.add_argument("--seq-length", "--enforce-sample-length", dest="seq_length", type=int, default=None,
                    help="pad every row to this many entries (set the run's dpo_data_seq_length to the same number)")
    ap.add_argument("--ftfy", action="store_true", help="repair mis-decoded text with ftfy before tokenizing")
    a = ap.parse_args(argv)
    fix = None
    if a.ftfy:
        try:
            import ftfy
        except ImportError as exc:
            raise SystemExit("--ftfy needs the ftfy package, which is not installed") from exc
        fix = ftfy.fix_text
    from ..data.tokenizer import build_tokenizer
    from .preprocess_data import _Cfg
    tok = build_tokenizer(_Cfg(a))
    if getattr(tok, "pad", None) is None:
        raise SystemExit("the DPO row format needs a tokenizer with a pad token (CharLevelTokenizer)")
    builder = MMapIndexedDatasetBuilder(a.output_prefix + "_text_document.bin", dtype=np.float32)
    n = 0
    for path in a.input.split(","):
        with open(path) as fh:
            for line in fh:
                line = line.strip()
                if not line:
                    continue
                doc = json.loads(line)
                if fix is not None:
                    doc = dict(doc, text_accept=fix(doc["text_accept"]), text_reject=fix(doc["text_reject"]))
                builder.add_item(encode_pair(doc, tok, a.seq_length))
                builder.end_document()
                n += 1
    builder.finalize(a.output_prefix + "_text_document.idx")
    print(f"wrote {n} preference pairs to {a.output_prefix}_text_document.{{bin,idx}}")


if __name__ == "__main__":
    main()
