"""Builds the in-tree native libraries.

    python -m savanna_b200.csrc.build [--force]

  savanna_b200/libsavanna_b200.so    every CUDA kernel, compiled for sm_100a only
                                     (nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo), C ABI
  savanna_b200/libsavanna_data.so    C++ dataset index builders, C ABI

The libraries expose plain C symbols and are loaded with ctypes (ops/cuda_ops.py, data/helpers.py), so
no PyTorch headers are compiled and a rebuild takes seconds.  A content hash of the sources is stored
next to each library; an up-to-date library is not rebuilt.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "build")
CUDA_LIB = os.path.join(PKG, "libsavanna_b200.so")
DATA_LIB = os.path.join(PKG, "libsavanna_data.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources(ext):
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(ext))


def _digest(files, extra=""):
    h = hashlib.sha256(extra.encode())
    for f in sorted(files):
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _stamp(lib):
    return lib + ".hash"


def _fresh(lib, digest):
    try:
        return os.path.exists(lib) and open(_stamp(lib)).read().strip() == digest
    except OSError:
        return False


def _run(cmd, log):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError("command failed:\n" + " ".join(cmd) + "\n" + r.stdout)


def build_cuda(force=False, verbose=False):
    cus = _sources(".cu")
    headers = _sources(".cuh") + _sources(".h")
    digest = _digest(cus + headers, " ".join(NVCC_FLAGS))
    if not force and _fresh(CUDA_LIB, digest):
        return CUDA_LIB
    os.makedirs(BUILD, exist_ok=True)
    nvcc = _nvcc()
    log = []
    objs = [os.path.join(BUILD, os.path.basename(c)[:-3] + ".o") for c in cus]
    with cf.ThreadPoolExecutor(max_workers=min(8, len(cus))) as ex:
        futs = [ex.submit(_run, [nvcc] + NVCC_FLAGS + ["-c", c, "-o", o], log) for c, o in zip(cus, objs)]
        for f in futs:
            f.result()
    _run([nvcc, "-shared", "-o", CUDA_LIB] + objs + ["-lcudart"], log)
    with open(_stamp(CUDA_LIB), "w") as fh:
        fh.write(digest)
    with open(os.path.join(BUILD, "build.log"), "w") as fh:
        fh.write("\n".join(log))
    if verbose:
        print("\n".join(log))
    return CUDA_LIB


def build_data(force=False):
    cpps = _sources(".cpp")
    digest = _digest(cpps)
    if not force and _fresh(DATA_LIB, digest):
        return DATA_LIB
    cxx = shutil.which("g++") or "g++"
    log = []
    _run([cxx, "-O3", "-std=c++17", "-shared", "-fPIC", "-o", DATA_LIB] + cpps, log)
    with open(_stamp(DATA_LIB), "w") as fh:
        fh.write(digest)
    return DATA_LIB


def build_all(force=False, verbose=False):
    return build_cuda(force, verbose), build_data(force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    libs = build_all(a.force, a.verbose)
    print("built:", *libs)
