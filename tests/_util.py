"""Shared helpers for the tests: fixture loading and the two error norms used everywhere.

Element-wise relative error is meaningless for these tensors (gradients span many
decades and cross zero), so parity is stated as
    max_err = max|a-b| / max|b|      and      l2_err = ||a-b||_2 / ||b||_2 .
"""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def load_golden(name):
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        return {k: z[k] for k in z.files}


def max_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    den = np.abs(b).max() if b.size else 0.0
    num = np.abs(a - b).max() if b.size else 0.0
    return float(num / den) if den > 0 else float(num)


def l2_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    den = np.sqrt((b * b).sum())
    num = np.sqrt(((a - b) ** 2).sum())
    return float(num / den) if den > 0 else float(num)


def assert_close(a, b, tol, what=""):
    assert np.asarray(a).shape == np.asarray(b).shape, f"{what}: shape {np.asarray(a).shape} vs {np.asarray(b).shape}"
    assert np.isfinite(np.asarray(a, np.float64)).all(), f"{what}: non-finite values"
    me, le = max_err(a, b), l2_err(a, b)
    assert me <= tol and le <= tol, f"{what}: max_err={me:.3e} l2_err={le:.3e} > tol={tol:.1e}"


def xy_grid_np(H, W, B):
    """numpy restatement of the reference's pixel grid (src/igs/gs2d.py:503-522):
    linspace(-wr, wr, W) along width, linspace(-hr, hr, H) along height,
    hr = sqrt(H/W), wr = 1/hr; float32 like torch.linspace's default."""
    import torch  # torch.linspace is what the reference calls; keep its exact rounding

    hr = (H / W) ** 0.5
    wr = 1 / hr
    xs = torch.linspace(-wr, wr, W).numpy()
    ys = torch.linspace(-hr, hr, H).numpy()
    x = np.broadcast_to(xs[None, None, :], (B, H, W)).copy()
    y = np.broadcast_to(ys[None, :, None], (B, H, W)).copy()
    return x, y
