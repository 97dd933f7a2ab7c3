"""Named corpora: fetch the raw files of a dataset, then tokenise them into the `.bin/.idx` training format.

    DATA_DOWNLOADERS           name -> DataDownloader subclass (public text corpora, plus `local` for files already on disk)
    prepare_dataset(name, ...) fetch (unless present) and run tools/preprocess_data.py over the fetched files

A downloader lists `urls`; `download()` fetches each into `<data_dir>/<name>/` with the Python standard library
(`http(s)://` and `file://` URLs; a machine without network access gets a clear error naming the URL, and files placed
there by hand are used as they are); `tokenize()` calls the preprocessing tool in-process.  Role of the reference's
tools/corpora.py:38-412 (which shells out to `wget` and `python tools/preprocess_data.py`).
"""
from __future__ import annotations

import os
import shutil
import urllib.error
import urllib.request
from multiprocessing import cpu_count
from typing import Dict, List, Optional, Type

GPT2_VOCAB_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-vocab.json"
GPT2_MERGE_URL = "https://s3.amazonaws.com/models.huggingface.co/bert/gpt2-merges.txt"


def fetch(url: str, dest: str) -> str:
    """Copy `url` to `dest` (atomic rename at the end)."""
    os.makedirs(os.path.dirname(os.path.abspath(dest)), exist_ok=True)
    tmp = dest + ".part"
    try:
        with urllib.request.urlopen(url, timeout=60) as src, open(tmp, "wb") as out:
            shutil.copyfileobj(src, out, 1 << 22)
    except (urllib.error.URLError, OSError) as exc:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise RuntimeError(f"cannot download {url}: {exc} (no network? place the file at {dest} by hand)") from exc
    os.replace(tmp, dest)
    return dest


class DataDownloader:
    name: str = ""
    urls: List[str] = []
    num_docs: Optional[int] = None

    def __init__(self, tokenizer_type: Optional[str] = None, merge_file: Optional[str] = None, vocab_file: Optional[str] = None,
                 data_dir: Optional[str] = None, force_redownload: bool = False, num_workers: Optional[int] = None):
        self.tokenizer_type = tokenizer_type or "GPT2BPETokenizer"
        self.data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
        self.merge_file = merge_file or os.path.join(self.data_dir, "gpt2-merges.txt")
        if vocab_file is None:
            if self.tokenizer_type == "GPT2BPETokenizer":
                vocab_file = os.path.join(self.data_dir, "gpt2-vocab.json")
            elif self.tokenizer_type == "HFGPT2Tokenizer":
                vocab_file = "gpt2"
            elif self.tokenizer_type != "CharLevelTokenizer":
                raise ValueError(f"tokenizer {self.tokenizer_type} needs a vocab file")
        self.vocab_file = vocab_file
        self.force_redownload = bool(force_redownload)
        self.num_workers = num_workers or cpu_count()

    @property
    def folder(self) -> str:
        return os.path.join(self.data_dir, self.name)

    def local_files(self) -> List[str]:
        return [os.path.join(self.folder, os.path.basename(u)) for u in self.urls]

    def exists(self) -> bool:
        return all(os.path.isfile(p) for p in self.local_files()) and bool(self.urls)

    def download(self) -> None:
        for url, dest in zip(self.urls, self.local_files()):
            if self.force_redownload or not os.path.isfile(dest):
                fetch(url, dest)

    def tokenize(self) -> str:
        from . import preprocess_data
        prefix = os.path.join(self.folder, self.name)
        argv = ["--input", ",".join(self.local_files()), "--output-prefix", prefix, "--tokenizer-type", self.tokenizer_type,
                "--append-eod", "--workers", str(self.num_workers)]
        if self.vocab_file:
            argv += ["--vocab-file", self.vocab_file]
        if self.tokenizer_type == "GPT2BPETokenizer":
            argv += ["--merge-file", self.merge_file]
        preprocess_data.main(argv)
        return prefix

    def prepare(self) -> str:
        if self.force_redownload or not self.exists():
            self.download()
        return self.tokenize()


def _make(name_: str, urls_: List[str], num_docs_: Optional[int] = None) -> Type[DataDownloader]:
    return type(name_.title().replace("_", ""), (DataDownloader,), {"name": name_, "urls": list(urls_), "num_docs": num_docs_})


_PILE = "https://the-eye.eu/public/AI/pile_preliminary_components"
DATA_DOWNLOADERS: Dict[str, object] = {
    "pass": "pass",
    "enron": _make("enron", ["http://eaidata.bmk.sh/data/enron_emails.jsonl.zst"]),
    "pile_subset": _make("pile_00", ["https://the-eye.eu/public/AI/pile/train/00.jsonl.zst"]),
    "pile": _make("pile", [f"https://the-eye.eu/public/AI/pile/train/{i:02}.jsonl.zst" for i in range(30)]),
    "pile_validation": _make("pile_validation", ["https://the-eye.eu/public/AI/pile/val.jsonl.zst"]),
    "pile_test": _make("pile_test", ["https://the-eye.eu/public/AI/pile/test.jsonl.zst"]),
    "github": _make("github", [f"{_PILE}/github.tar"]),
    "arxiv": _make("arxiv", [f"{_PILE}/2020-09-08-arxiv-extracts-nofallback-until-2007-068.tar.gz"]),
    "europarl": _make("europarl", [f"{_PILE}/EuroParliamentProceedings_1996_2011.jsonl.zst"]),
    "freelaw": _make("freelaw", [f"{_PILE}/FreeLaw_Opinions.jsonl.zst"]),
    "nih": _make("nih", [f"{_PILE}/NIH_ExPORTER_awarded_grant_text.jsonl.zst"]),
    "pubmed": _make("pubmed", [f"{_PILE}/PMC_extracts.tar.gz"]),
    "books1": _make("books1", [f"{_PILE}/books1.tar.gz"]),
    "books3": _make("books3", [f"{_PILE}/books3.tar.gz"]),
    "hackernews": _make("hackernews", [f"{_PILE}/hn.tar.gz"], 373000),
    "openwebtext2": _make("openwebtext2", [f"{_PILE}/openwebtext2.jsonl.zst.tar"], 17103000),
    "stackexchange": _make("stackexchange", [f"{_PILE}/stackexchange_dataset.tar"]),
    "ubuntu_irc": _make("ubuntu_irc", [f"{_PILE}/ubuntu_irc_until_2020_9_1.jsonl.zst"]),
    "youtube_subtitles": _make("youtube_subtitles", [f"{_PILE}/yt_subs.jsonl.zst"]),
    "enwik8": _make("enwik8", ["https://data.deepai.org/enwik8.zip"]),
}


class Local(DataDownloader):
    """Files that are already on disk: `urls` are their paths (given as `file://` URLs or plain paths)."""
    name = "local"

    def __init__(self, files: List[str], name: str = "local", **kw):
        super().__init__(**kw)
        self.name = name
        self.urls = [f if "://" in f else "file://" + os.path.abspath(f) for f in files]


def maybe_download_gpt2_tokenizer_data(tokenizer_type: Optional[str], data_dir: str) -> None:
    if tokenizer_type is None or tokenizer_type == "GPT2BPETokenizer":
        for url, fname in ((GPT2_VOCAB_URL, "gpt2-vocab.json"), (GPT2_MERGE_URL, "gpt2-merges.txt")):
            dest = os.path.join(data_dir, fname)
            if not os.path.isfile(dest):
                fetch(url, dest)


def prepare_dataset(dataset_name: str, tokenizer_type: Optional[str] = None, data_dir: Optional[str] = None,
                    vocab_file: Optional[str] = None, merge_file: Optional[str] = None, force_redownload: bool = False,
                    num_workers: Optional[int] = None, files: Optional[List[str]] = None) -> Optional[str]:
    """Returns the output prefix of the tokenised dataset (None for the `pass` placeholder)."""
    data_dir = data_dir or os.environ.get("DATA_DIR", "./data")
    os.makedirs(data_dir, exist_ok=True)
    kw = dict(tokenizer_type=tokenizer_type, vocab_file=vocab_file, merge_file=merge_file, data_dir=data_dir,
              force_redownload=force_redownload, num_workers=1 if dataset_name == "enwik8" else num_workers)
    if files:
        return Local(files, dataset_name, **kw).prepare()
    cls = DATA_DOWNLOADERS.get(dataset_name.lower())
    if cls is None:
        raise NotImplementedError(f"dataset {dataset_name!r} not recognised; choose from {sorted(DATA_DOWNLOADERS)}")
    if cls == "pass":
        return None
    maybe_download_gpt2_tokenizer_data(tokenizer_type, data_dir)
    return cls(**kw).prepare()
