"""Builds ``libigs_b200.so`` (the CUDA kernels + C ABI) in-tree with nvcc for sm_100a.

    python -m igs_b200.build            # build if stale
    python -m igs_b200.build --force

The shared object sits beside this file so that it travels with the source tree; it
links only against the CUDA runtime (no torch, no Python).
"""
from __future__ import annotations

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
    "--threads", "0",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the igs_b200 kernels cannot be built")
    return cand


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    out = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    out += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    out.append(os.path.abspath(__file__))
    return out


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > t for d in _deps())


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    env = dict(os.environ)
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
    if verbose:
        print(log)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
