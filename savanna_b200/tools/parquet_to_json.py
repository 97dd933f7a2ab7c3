"""Convert a parquet file of documents into the JSON-lines form that `preprocess_data` reads (role of the reference's
tools/parquet_to_json.py).

    python -m savanna_b200.tools.parquet_to_json in.parquet out.jsonl [--columns text ...]
"""
from __future__ import annotations

import argparse
import json
from typing import List, Optional


def convert(src: str, dst: str, columns: Optional[List[str]] = None, batch_rows: int = 65536) -> int:
    import pyarrow.parquet as pq
    pf = pq.ParquetFile(src)
    n = 0
    with open(dst, "w") as out:
        for batch in pf.iter_batches(batch_size=batch_rows, columns=columns):
            for row in batch.to_pylist():
                out.write(json.dumps(row, ensure_ascii=False, default=str) + "\n")
                n += 1
    return n


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("src")
    ap.add_argument("dst")
    ap.add_argument("--columns", nargs="*", default=None)
    a = ap.parse_args(argv)
    n = convert(a.src, a.dst, a.columns)
    print(f"wrote {n} rows to {a.dst}")
    return n


if __name__ == "__main__":
    main()
