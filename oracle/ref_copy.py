"""The reference's own Python package as the timed CPU arm.

TEST / MEASUREMENT INFRASTRUCTURE ONLY (like everything under ``oracle/``): used by the
CPU legs of ``bench.py``; never by the product package.

The reference (KohakuBlueleaf/IGS) is pure Python, so there is nothing to compile: this
recipe copies its package directory ``src/igs/`` unchanged into ``oracle/_ref/igs/``
(git-ignored, never committed; it travels with the working tree to wherever the benchmark
runs) where the reference tree is present, and ``load()`` imports it from there with the
two settings its CPU path needs:

* ``TORCHDYNAMO_DISABLE=1`` -- ``render`` is wrapped in ``torch.compile``
  (src/igs/gs2d.py:525), which does not compile on CPU here;
* ``GaussianSplatting2DKernel`` rebound to ``GaussianSplatting2DChunkedKernel``
  (src/igs/gs2d.py:265-465) -- the module's default binding is the Triton class
  (:471-476), which needs a GPU.

    python -m oracle.ref_copy [/path/to/reference]     # make the copy

Without an argument the reference tree is looked up under the ``reference_path`` that
``BASELINE.json`` at the repository root names.
"""
from __future__ import annotations

import importlib
import json
import os
import shutil
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")


def default_reference() -> str | None:
    """Where the reference tree lives according to BASELINE.json beside the package, or None."""
    try:
        with open(os.path.join(os.path.dirname(_HERE), "BASELINE.json")) as f:
            return json.load(f).get("reference_path")
    except (OSError, ValueError):
        return None


def make(reference_root: str | None = None) -> str | None:
    """Copies <reference_root>/src/igs to oracle/_ref/igs; returns the copy's path, or None
    when the reference tree is not there (then an existing copy is left as it is)."""
    reference_root = reference_root or default_reference()
    if not reference_root:
        return None
    src = os.path.join(reference_root, "src", "igs")
    if not os.path.isdir(src):
        return None
    dst = os.path.join(REF_DIR, "igs")
    os.makedirs(REF_DIR, exist_ok=True)
    if os.path.isdir(dst):
        _make_writable(dst)
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
    _make_writable(dst)  # (a read-only reference tree hands its modes to the copy)
    return dst


def _make_writable(root: str) -> None:
    for base, dirs, files in os.walk(root):
        for name in dirs + files:
            path = os.path.join(base, name)
            os.chmod(path, os.stat(path).st_mode | 0o200)
    os.chmod(root, os.stat(root).st_mode | 0o200)


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "igs", "gs2d.py"))


def load():
    """The reference's ``igs.gs2d`` module from the copy, bound to its chunked torch
    Function; raises ImportError when there is no copy."""
    if not available():
        raise ImportError("no copy of the reference under oracle/_ref (python -m oracle.ref_copy makes one)")
    os.environ["TORCHDYNAMO_DISABLE"] = "1"
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    mod = importlib.import_module("igs.gs2d")
    if os.path.dirname(os.path.abspath(mod.__file__)) != os.path.join(REF_DIR, "igs"):
        raise ImportError(f"`igs` resolved to {mod.__file__}, not to the copy under oracle/_ref")
    mod.GaussianSplatting2DKernel = mod.GaussianSplatting2DChunkedKernel
    return mod


def render_fwd_bwd(mod, positions, colors, scales, rotations, alphas, x, y, gout_fn, eps=1e-6):
    """One forward + backward of the reference's ``gaussian_splatting_2d`` on CPU tensors:
    (out, grads for positions, colors, scales, rotations, alphas)."""
    names = ("positions", "colors", "scales", "rotations", "alphas")
    leaves = [t.detach().clone().requires_grad_() for t in (positions, colors, scales, rotations, alphas)]
    out = mod.gaussian_splatting_2d(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], x, y, eps)
    # the reference's backward divides the upstream gradient in place (src/igs/gs2d.py:371)
    out.backward(gout_fn(out.detach()).clone())
    return out.detach(), {k: t.grad for k, t in zip(names, leaves)}


if __name__ == "__main__":
    path = make(sys.argv[1] if len(sys.argv) > 1 else None)
    print(path or "reference tree not found; nothing copied")
