"""Download (or take from disk) and tokenise a named dataset.

    python -m savanna_b200.tools.prepare_data enwik8 -t CharLevelTokenizer -d ./data
    python -m savanna_b200.tools.prepare_data mygenomes -t CharLevelTokenizer -d ./data --files a.jsonl b.jsonl

Role of the reference's tools/prepare_data.py:1-60 over tools/corpora.py.
"""
from __future__ import annotations

import argparse

from .corpora import DATA_DOWNLOADERS, prepare_dataset

TOKENIZER_CHOICES = ["HFGPT2Tokenizer", "HFTokenizer", "GPT2BPETokenizer", "CharLevelTokenizer", "TiktokenTokenizer"]


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("dataset", nargs="?", default="enwik8",
                    help=f"one of {sorted(k for k in DATA_DOWNLOADERS if k != 'pass')}, or any name together with --files")
    ap.add_argument("-t", "--tokenizer", default="GPT2BPETokenizer", choices=TOKENIZER_CHOICES)
    ap.add_argument("-d", "--data-dir", default=None, help="where raw and tokenised files go (default ./data or $DATA_DIR)")
    ap.add_argument("-v", "--vocab-file", default=None)
    ap.add_argument("-m", "--merge-file", default=None)
    ap.add_argument("-f", "--force-redownload", action="store_true")
    ap.add_argument("--files", nargs="*", default=None, help="jsonl files already on disk (no download)")
    ap.add_argument("--workers", type=int, default=None)
    a = ap.parse_args(argv)
    prefix = prepare_dataset(a.dataset, a.tokenizer, a.data_dir, a.vocab_file, a.merge_file, a.force_redownload, a.workers, a.files)
    print(f"dataset prefix: {prefix}")
    return prefix


if __name__ == "__main__":
    main()
