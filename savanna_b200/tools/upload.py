"""Upload checkpoints or exported models: to a checkpoint store (posix directory or S3 bucket) or to the Hugging Face hub.

    python -m savanna_b200.tools.upload store <local dir> --store s3 --bucket my-bucket --prefix runs/x   [--store posix --root /archive]
    python -m savanna_b200.tools.upload hf <local dir> --repo-id org/name [--private] [--token ...]

`store` goes through the same code as the trainer's background uploads (`ckpt/stores.py`: `.uploading` / `.uploaded`
markers, retries with back-off).  `hf` needs the `huggingface_hub` package and network access.  Role of the reference's
tools/upload.py and tools/upload_model_to_hf.py.
"""
from __future__ import annotations

import argparse
import os


def upload_to_store(local_dir: str, kind: str, bucket: str = None, prefix: str = "", root: str = None, retries: int = 3) -> bool:
    from ..ckpt.stores import PosixStore, S3Store, upload_checkpoint
    if kind == "s3":
        if not bucket:
            raise ValueError("--bucket is required for the s3 store")
        store = S3Store({"bucket": bucket, "location": prefix, "max_retries": retries})
    elif kind == "posix":
        if not root:
            raise ValueError("--root is required for the posix store")
        store = PosixStore({"location": root, "max_retries": retries})
    else:
        raise ValueError(f"unknown store {kind!r}")
    return upload_checkpoint(local_dir, [store])


def upload_to_hf(local_dir: str, repo_id: str, private: bool = False, token: str = None, commit_message: str = "upload"):
    try:
        from huggingface_hub import HfApi
    except Exception as exc:  # noqa: BLE001
        raise ImportError("uploading to the Hugging Face hub needs the `huggingface_hub` package") from exc
    api = HfApi(token=token or os.environ.get("HF_TOKEN"))
    api.create_repo(repo_id, private=private, exist_ok=True)
    return api.upload_folder(folder_path=local_dir, repo_id=repo_id, commit_message=commit_message)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    st = sub.add_parser("store")
    st.add_argument("local_dir")
    st.add_argument("--store", choices=["s3", "posix"], default="s3")
    st.add_argument("--bucket", default=None)
    st.add_argument("--prefix", default="")
    st.add_argument("--root", default=None)
    st.add_argument("--retries", type=int, default=3)
    hf = sub.add_parser("hf")
    hf.add_argument("local_dir")
    hf.add_argument("--repo-id", required=True)
    hf.add_argument("--private", action="store_true")
    hf.add_argument("--token", default=None)
    a = ap.parse_args(argv)
    if a.cmd == "store":
        ok = upload_to_store(a.local_dir, a.store, a.bucket, a.prefix, a.root, a.retries)
        print("uploaded" if ok else "upload FAILED")
        return ok
    return upload_to_hf(a.local_dir, a.repo_id, a.private, a.token)


if __name__ == "__main__":
    main()
