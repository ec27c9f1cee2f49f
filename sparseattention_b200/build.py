"""Compile the CUDA sources in csrc/ into libhsa_b200.so (in-tree, next to this file).

    python -m sparseattention_b200.build [--force] [--verbose]

nvcc cross-compiles for sm_100a without a GPU.  The library links the static CUDA runtime, so it
loads on a machine without a driver (where only its host-side entry points are usable).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libhsa_b200.so")
STAMP = os.path.join(HERE, "libhsa_b200.stamp")

NVCC_FLAGS = [
    "-std=c++20", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-DHSA_TARGET_ARCH=100",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    files = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC))]
    files += [os.path.join(INCLUDE, f) for f in sorted(os.listdir(INCLUDE))]
    for f in files:
        with open(f, "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as fh:
        return fh.read().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Build the shared library if sources changed; returns its path."""
    if not force and is_current():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libhsa_b200.so")
    # one nvcc per source file, in parallel, then one link step
    with tempfile.TemporaryDirectory(prefix="hsa_b200_build_") as tmp:
        def compile_one(src: str):
            obj = os.path.join(tmp, os.path.basename(src)[:-3] + ".o")
            cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", "-o", obj, src]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            return obj, subprocess.run(cmd, capture_output=True, text=True)

        with ThreadPoolExecutor(max_workers=min(len(sources()), os.cpu_count() or 1)) as pool:
            results = list(pool.map(compile_one, sources()))
        failed = [r for _, r in results if r.returncode != 0]
        if failed:
            raise RuntimeError("nvcc failed:\n" + "\n".join(r.stdout + r.stderr for r in failed))
        if verbose:
            for _, r in results:
                print(r.stderr, file=sys.stderr)
        link = subprocess.run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB,
                               *[o for o, _ in results]], capture_output=True, text=True)
        if link.returncode != 0:
            raise RuntimeError("link failed:\n" + link.stdout + link.stderr)
    with open(STAMP, "w") as fh:
        fh.write(_digest())
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))
