"""Builds the CUDA sources in this directory into ``axlearn_b200/lib/libaxb200.so``.

Every ``*.cu`` file is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``)
and linked into one shared library that exposes plain C entry points; Python reaches them with
``ctypes`` (see ``axlearn_b200/ops/cuda_ops.py``).  Objects are rebuilt only when their source
or one of the headers is newer.  ``nvcc`` cross-compiles, so no GPU is needed to build.

Usage: ``python -m axlearn_b200.csrc.build [--force] [--verbose]``.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(os.path.dirname(HERE), "lib")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(LIB_DIR, "libaxb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def sources() -> list[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers_mtime() -> float:
    hs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    return max((os.path.getmtime(h) for h in hs), default=0.0)


def _compile(src: str, force: bool, verbose: bool) -> tuple[str, str]:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    newest = max(os.path.getmtime(src), _headers_mtime())
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{proc.stdout}\n{proc.stderr}")
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles what is stale and links; returns the library path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    srcs = sources()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    # The list of linked objects is recorded beside the library: a source that was removed (or
    # added) changes the list and forces a new link even when no object is newer than the library.
    manifest = LIB_PATH + ".objects"
    listing = "\n".join(os.path.basename(o) for o in objs)
    previous = open(manifest, encoding="utf-8").read() if os.path.exists(manifest) else None
    stale = force or not os.path.exists(LIB_PATH) or previous != listing or any(
        os.path.getmtime(o) > os.path.getmtime(LIB_PATH) for o in objs)
    if stale:
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "shared"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
        with open(manifest, "w", encoding="utf-8") as f:
            f.write(listing)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
