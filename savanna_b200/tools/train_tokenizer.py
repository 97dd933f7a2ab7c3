"""Train a byte-level BPE tokenizer on jsonl documents and save it in the Hugging Face `tokenizers` JSON format, which
`data/tokenizer.py:HFTokenizer` loads (`tokenizer_type: HFTokenizer`, `vocab_file: <the saved file>`).

    python -m savanna_b200.tools.train_tokenizer --json_input_dir data/ --tokenizer_output_path tok.json -v 52000

Input: every `*.jsonl` / `*.json` file of the directory, one JSON object per line, text under `--text_key`.  Documents
are streamed (never all in memory).  Special tokens `<|endoftext|>` (id 0) and `<|padding|>` (id 1).  Role of the
reference's savanna/tokenizer/train_tokenizer.py:38-106.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
from typing import Iterator

SPECIAL_TOKENS = ["<|endoftext|>", "<|padding|>"]


def iter_texts(input_dir: str, text_key: str = "text") -> Iterator[str]:
    files = sorted(glob.glob(os.path.join(input_dir, "*.jsonl")) + glob.glob(os.path.join(input_dir, "*.json")))
    if not files:
        raise FileNotFoundError(f"no .jsonl / .json files in {input_dir}")
    for path in files:
        with open(path, encoding="utf-8") as fh:
            for line in fh:
                line = line.strip()
                if line:
                    yield json.loads(line)[text_key]


def train_tokenizer(input_dir: str, save_path: str, tokenizer_type: str = "BPE", vocab_size: int = 52000,
                    text_key: str = "text"):
    if tokenizer_type != "BPE":
        raise NotImplementedError(f"tokenizer type {tokenizer_type!r} is not implemented (BPE only)")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, processors, trainers
    from tokenizers.normalizers import NFKC
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=True)
    tok.decoder = decoders.ByteLevel()
    tok.post_processor = processors.ByteLevel(trim_offsets=True)
    tok.normalizer = NFKC()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=SPECIAL_TOKENS, show_progress=False)
    tok.train_from_iterator(iter_texts(input_dir, text_key), trainer)
    os.makedirs(os.path.dirname(os.path.abspath(save_path)), exist_ok=True)
    tok.save(save_path, pretty=True)
    print(f"tokenizer with {tok.get_vocab_size()} entries saved at {save_path}")
    return tok


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--json_input_dir", required=True)
    ap.add_argument("--tokenizer_output_path", required=True, help="should end in .json")
    ap.add_argument("--tokenizer_type", choices=["BPE"], default="BPE")
    ap.add_argument("-v", "--vocab_size", type=int, default=52000)
    ap.add_argument("--text_key", default="text")
    a = ap.parse_args(argv)
    train_tokenizer(a.json_input_dir, a.tokenizer_output_path, a.tokenizer_type, a.vocab_size, a.text_key)


if __name__ == "__main__":
    main()
