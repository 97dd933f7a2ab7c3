"""Secondary checkpoint stores: after a checkpoint is complete it is copied to every configured store.

Configuration (`checkpoint_stores`, a list of dicts as in the reference, savanna/checkpointing.py:187-291):
    {"storage_type": "posix", "location": <directory>, "num_checkpoints": <keep last N, optional>}
    {"storage_type": "s3", "bucket": ..., "location": <key prefix>, "access_id": ..., "secret": ..., "max_retries": 3}

A checkpoint directory carries a `.uploading` marker while any store is still being written and `.uploaded` once all
succeeded; pruning (`ckpt/io.py:_delete_old`) never removes a directory that has `.uploading`.  The S3 store needs
`boto3`; when it is not installed the store reports that once and is skipped (the posix store needs nothing).  Every
file transfer is retried with a growing delay; a checkpoint whose upload failed keeps its `.uploading` marker, so it is
neither pruned nor mistaken for safely stored.
"""
from __future__ import annotations

import glob
import os
import re
import shutil
import time
from typing import Callable, Dict, Iterable, List, Optional

from .. import print_rank_0

MARKERS = (".uploading", ".uploaded")


def _files(ckpt_dir: str) -> Iterable[str]:
    for root, _, names in os.walk(ckpt_dir):
        for n in names:
            if n not in MARKERS:
                yield os.path.join(root, n)


def _retry(fn: Callable[[], None], what: str, retries: int, base_delay: float, sleep=time.sleep) -> bool:
    for attempt in range(1, retries + 2):
        try:
            fn()
            return True
        except Exception as exc:  # noqa: BLE001
            if attempt > retries:
                print_rank_0(f"  {what}: giving up after {retries} retries ({exc})")
                return False
            print_rank_0(f"  {what}: attempt {attempt} failed ({exc}); retrying")
            sleep(base_delay * attempt)
    return False


class PosixStore:
    def __init__(self, cfg: Dict):
        self.location = cfg["location"]
        self.keep = cfg.get("num_checkpoints")
        self.retries = int(cfg.get("max_retries", 3))

    def upload(self, ckpt_dir: str, tag: str, sleep=time.sleep) -> bool:
        dst = os.path.join(self.location, tag)
        ok = _retry(lambda: shutil.copytree(ckpt_dir, dst, dirs_exist_ok=True, ignore=shutil.ignore_patterns(*MARKERS)),
                    f"copy {tag} -> {dst}", self.retries, 1.0, sleep)
        if ok and self.keep and self.keep > 0:
            steps = sorted((int(m.group(1)), p) for p in glob.glob(os.path.join(self.location, "global_step*"))
                           if (m := re.match(r"global_step(\d+)$", os.path.basename(p))))
            for _, p in steps[:-self.keep]:
                shutil.rmtree(p, ignore_errors=True)
        return ok


class S3Store:
    def __init__(self, cfg: Dict, client=None):
        self.bucket, self.prefix = cfg["bucket"], cfg.get("location", "").strip("/")
        self.retries = int(cfg.get("max_retries", 3))
        if client is None:
            import boto3                                   # raises ImportError when the SDK is not installed
            client = boto3.client("s3", aws_access_key_id=cfg.get("access_id"), aws_secret_access_key=cfg.get("secret"))
        self.client = client

    def upload(self, ckpt_dir: str, tag: str, sleep=time.sleep) -> bool:
        ok = True
        for path in sorted(_files(ckpt_dir)):
            rel = os.path.relpath(path, ckpt_dir).replace(os.sep, "/")
            key = "/".join(x for x in (self.prefix, tag, rel) if x)
            ok &= _retry(lambda p=path, k=key: self.client.upload_file(p, self.bucket, k), f"upload {rel} -> s3://{self.bucket}/{key}",
                         self.retries, 10.0, sleep)
            if not ok:
                return False                               # a partial checkpoint in the bucket is of no use: stop here
        return ok


def build_stores(configs: Optional[List[Dict]]) -> List:
    stores = []
    for c in configs or []:
        kind = c.get("storage_type", "posix")
        if kind == "posix":
            stores.append(PosixStore(c))
        elif kind == "s3":
            try:
                stores.append(S3Store(c))
            except ImportError:
                print_rank_0("  checkpoint store 's3' needs boto3, which is not installed; this store is skipped")
        else:
            raise ValueError(f"unknown checkpoint store type {kind!r}")
    return stores


def upload_checkpoint(ckpt_dir: str, stores: List, sleep=time.sleep) -> bool:
    """Copy a finished checkpoint to every store.  `.uploading` exists for the duration and is replaced by `.uploaded`
    only when all stores succeeded."""
    if not stores:
        return True
    tag = os.path.basename(os.path.normpath(ckpt_dir))
    marker = os.path.join(ckpt_dir, ".uploading")
    open(marker, "w").close()
    ok = all([s.upload(ckpt_dir, tag, sleep) for s in stores])
    if ok:
        os.replace(marker, os.path.join(ckpt_dir, ".uploaded"))
    return ok
