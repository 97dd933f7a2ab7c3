"""Tokenizers (reference: savanna/tokenizer/tokenizer.py:14-323).

`CharLevelTokenizer` is the Evo 2 tokenizer: raw bytes, vocabulary 512, eod 0, pad 1.  The others
wrap optional third-party packages and raise a clear error when those are missing.  The vocabulary is
padded to a multiple of `make_vocab_size_divisible_by * model_parallel_size`.
"""
from __future__ import annotations

from typing import List

import numpy as np


class AbstractTokenizer:
    name = "abstract"
    vocab_size: int = 0
    eod: int = 0

    def tokenize(self, text):
        raise NotImplementedError

    def detokenize(self, ids):
        raise NotImplementedError

    def tokenize_batch(self, texts):
        return [self.tokenize(t) for t in texts]


class CharLevelTokenizer(AbstractTokenizer):
    name = "CharLevelTokenizer"

    def __init__(self, vocab_size: int = 512):
        self.vocab_size = vocab_size
        self.eod_id, self.pad_id = 0, 1
        self.eos_id = 0

    @property
    def eod(self):
        return self.eod_id

    @property
    def pad(self):
        return self.pad_id

    def clamp(self, n: int) -> int:
        return max(32, min(self.vocab_size, n))

    def tokenize(self, text) -> List[int]:
        if isinstance(text, str):
            text = text.encode("utf-8")
        return list(np.frombuffer(text, dtype=np.uint8))

    def tokenize_batch(self, text_batch):
        """A list of strings -> a list of id lists; a single string is tokenized as such."""
        if isinstance(text_batch, list):
            return [self.tokenize(s) for s in text_batch]
        return self.tokenize(text_batch)

    def decode_token(self, token: int) -> str:
        return chr(self.clamp(int(token)))

    def detokenize(self, ids) -> str:
        return "".join(self.decode_token(t) for t in ids)

    def detokenize_batch(self, batch):
        return [self.detokenize(row) for row in batch]


class GPT2BPETokenizer(AbstractTokenizer):
    name = "GPT2BPETokenizer"

    def __init__(self, vocab_file, merge_file):
        try:
            from transformers import GPT2TokenizerFast
        except Exception as exc:
            raise ImportError("GPT2BPETokenizer needs the `transformers` package") from exc
        self.tk = GPT2TokenizerFast(vocab_file=vocab_file, merges_file=merge_file)
        self.vocab_size = len(self.tk)
        self.eod_id = self.tk.convert_tokens_to_ids("<|endoftext|>")

    @property
    def eod(self):
        return self.eod_id

    def tokenize(self, text):
        return self.tk.encode(text)

    def detokenize(self, ids):
        return self.tk.decode(ids)


class HFTokenizer(AbstractTokenizer):
    name = "HFTokenizer"

    def __init__(self, vocab_file):
        try:
            from tokenizers import Tokenizer
        except Exception as exc:
            raise ImportError("HFTokenizer needs the `tokenizers` package") from exc
        self.tk = Tokenizer.from_file(vocab_file)
        self.vocab_size = self.tk.get_vocab_size()
        self.eod_id = self.tk.token_to_id("<|endoftext|>") or 0
        self.pad_id = self.tk.token_to_id("<|padding|>") or 1

    @property
    def eod(self):
        return self.eod_id

    def tokenize(self, text):
        return self.tk.encode(text).ids

    def detokenize(self, ids):
        return self.tk.decode(list(ids))


class SentencePieceTokenizer(AbstractTokenizer):
    name = "SPMTokenizer"

    def __init__(self, vocab_file):
        import sentencepiece as spm

        self.tk = spm.SentencePieceProcessor(model_file=vocab_file)
        self.vocab_size = self.tk.get_piece_size()
        self.eod_id = self.tk.piece_to_id("<|endoftext|>")

    @property
    def eod(self):
        return self.eod_id

    def tokenize(self, text):
        return self.tk.encode(text)

    def detokenize(self, ids):
        return self.tk.decode(list(ids))


class TiktokenTokenizer(AbstractTokenizer):
    name = "TiktokenTokenizer"

    def __init__(self, vocab_file):
        try:
            import tiktoken
        except Exception as exc:
            raise ImportError("TiktokenTokenizer needs the `tiktoken` package") from exc
        self.tk = tiktoken.get_encoding(vocab_file)
        self.vocab_size = self.tk.n_vocab
        self.eod_id = self.tk.eot_token

    @property
    def eod(self):
        return self.eod_id

    def tokenize(self, text):
        return self.tk.encode(text, allowed_special="all")

    def detokenize(self, ids):
        return self.tk.decode(list(ids))


def pad_vocab_size(n: int, divisible_by: int, tp: int) -> int:
    m = divisible_by * tp
    return m * ((n + m - 1) // m)


def build_tokenizer(cfg):
    t = str(cfg.tokenizer_type).lower()                 # names compare without case, as in the reference
    if t == "charleveltokenizer":
        tok = CharLevelTokenizer(512)
    elif t == "gpt2bpetokenizer":
        tok = GPT2BPETokenizer(cfg.vocab_file, cfg.merge_file)
    elif t in ("hftokenizer", "hfgpt2tokenizer"):
        tok = HFTokenizer(cfg.vocab_file)
    elif t == "spmtokenizer":
        tok = SentencePieceTokenizer(cfg.vocab_file)
    elif t == "tiktokentokenizer":
        tok = TiktokenTokenizer(cfg.vocab_file)
    else:
        raise NotImplementedError(f"tokenizer {cfg.tokenizer_type!r} not implemented")
    cfg.padded_vocab_size = pad_vocab_size(tok.vocab_size, cfg.make_vocab_size_divisible_by, cfg.model_parallel_size)
    return tok
