"""Builds ``libigs_b200.so`` (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m igs_b200.build            # build if stale
    python -m igs_b200.build --force

The shared object sits beside this file so that it travels with the source tree; it
links only against the CUDA runtime (no torch, no Python).
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB_PATH = os.path.join(HERE, "libigs_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xptxas=-v",
    "-Xcompiler", "-fPIC", "-shared",
    "-Xlinker", "--no-undefined",  # a function that lost its definition fails the build, not the first load
    "--threads", "0",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the igs_b200 kernels cannot be built")
    return cand


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


STAMP_PATH = LIB_PATH + ".srchash"


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    out += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return sorted(out)


def source_hash() -> str:
    """Hash of everything the shared object is built from (sources, headers, flags).  The
    contents, not the time stamps: a copied tree keeps no usable mtimes."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for path in _deps():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the shared object is missing or was built from other sources than the tree
    holds now (its stamp file records the hash of the sources it was built from)."""
    if not os.path.exists(LIB_PATH) or not os.path.exists(STAMP_PATH):
        return True
    with open(STAMP_PATH) as f:
        return f.read().strip() != source_hash()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    # one builder at a time (several ranks may import the package at once)
    with open(LIB_PATH + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not is_stale():
            return LIB_PATH
        return _build_locked(verbose)


def _build_locked(verbose: bool) -> str:
    env = dict(os.environ)
    digest = source_hash()
    # the image exports CC/CXX pointing at a wrapper; nvcc must use the system host compiler
    cmd = [_nvcc(), *NVCC_FLAGS, "-ccbin", "/usr/bin/g++", "-I", INCLUDE, "-o", LIB_PATH, *sources()]
    if not os.path.exists("/usr/bin/g++"):
        cmd = [c for c in cmd if c not in ("-ccbin", "/usr/bin/g++")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    log = res.stdout + res.stderr
    with open(os.path.join(HERE, "build.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + log)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + log[-4000:])
    with open(STAMP_PATH, "w") as f:
        f.write(digest + "\n")
    if verbose:
        print(log)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
