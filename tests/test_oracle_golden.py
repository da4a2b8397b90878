"""Pins the CPU oracle against fixtures produced by running the reference itself
(tests/golden/make_golden.py).  No GPU needed."""
import numpy as np
import pytest

from oracle import splat_oracle as so
from tests._util import assert_close, load_golden, xy_grid_np

RENDER_CASES = ["render_small_c3", "render_narrow_c3", "render_c1", "render_c4", "render_c16",
                "render_c17", "render_n1", "render_tall"]

# fp32 oracle vs fp32 reference: both carry fp32 rounding (the reference's own noise
# floor against fp64 is ~2e-6, up to 4e-5 on rotations with narrow scales)
TOL32 = 1e-4
# fp64 oracle vs fp32 reference: the difference is the reference's fp32 rounding alone
TOL64 = 1e-4


def _render_grads(g, dtype, mode=so.MODE_REFERENCE):
    return so.render_with_grads(g["positions"], g["colors"], g["scales"], g["rotations"], g["alphas"],
                                g["x"][:, 0], g["y"][:, 0], lambda out: g["gout"], float(g["eps"]),
                                mode=mode, dtype=dtype)


@pytest.mark.parametrize("name", RENDER_CASES)
@pytest.mark.parametrize("dtype,tol", [(np.float32, TOL32), (np.float64, TOL64)])
def test_render_matches_reference(name, dtype, tol):
    g = load_golden(name)
    out, _, grads = _render_grads(g, dtype)
    assert_close(out, g["out"], tol, f"{name} image")
    for k in ("positions", "colors", "scales", "rotations", "alphas"):
        assert_close(grads[k], g["g_" + k], tol, f"{name} d_{k}")


def test_xy_grid_restatement():
    g = load_golden("render_small_c3")
    B, _, H, W = g["x"].shape
    x, y = xy_grid_np(H, W, B)
    assert np.array_equal(x, g["x"][:, 0]) and np.array_equal(y, g["y"][:, 0])
    g = load_golden("render_tall")
    B, _, H, W = g["x"].shape
    x, y = xy_grid_np(H, W, B)
    assert np.array_equal(x, g["x"][:, 0]) and np.array_equal(y, g["y"][:, 0])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_kernel_level_entry_both_gradient_modes(dtype):
    """cov_inv-level entry, arbitrary sample coordinates, indefinite cov_inv; checks the
    reference-mode backward (src/igs/gs2d.py:339-465) and the exact one (autograd of
    src/igs/gs2d.py:24-44), including d/dx and d/dy."""
    g = load_golden("kernel_xy_c3")
    eps = float(g["eps"])
    args = (g["x"][:, 0], g["y"][:, 0], g["positions"], g["c00"], g["c01"], g["c11"], g["alphas"], g["colors"])
    out, wsum = so.forward(*args, eps, dtype)
    assert_close(out, g["out"], 2e-5, "image")
    assert_close(out, g["out_dense"], 2e-5, "image vs dense formula")
    for mode, tag in ((so.MODE_REFERENCE, "ref"), (so.MODE_EXACT, "exact")):
        gr = so.backward(*args, wsum, out, g["gout"], eps, mode, True, dtype)
        for k in ("x", "y", "positions", "c00", "c01", "c11", "alphas", "colors"):
            want = g[f"g_{tag}_{k}"]
            assert_close(np.asarray(gr[k]).reshape(want.shape), want, 1e-4, f"{tag} d_{k}")


def test_cfg0_full_size():
    """Benchmark configuration 0 (B=1, N=2048, 256x256, C=3) against the reference's output."""
    g = load_golden("cfg0_full")
    B, C, H, W = g["out"].shape
    x, y = xy_grid_np(H, W, B)
    out, _, grads = so.render_with_grads(g["positions"], g["colors"], g["scales"], g["rotations"],
                                         g["alphas"], x, y, lambda o: 2 * (o - g["target"]),
                                         float(g["eps"]), dtype=np.float32)
    assert_close(out, g["out"], 1e-5, "image")
    for k in ("positions", "colors", "scales", "rotations", "alphas"):
        assert_close(grads[k], g["g_" + k], 1e-4, f"d_{k}")
    loss = float(((out.astype(np.float64) - g["target"]) ** 2).sum())
    assert abs(loss - float(g["loss"])) <= 1e-5 * abs(float(g["loss"]))


def test_empty_inputs():
    """No gaussians: the reference's loop body never runs and the image is 0/(0+eps)."""
    x, y = xy_grid_np(4, 6, 1)
    out, wsum = so.forward(x, y, np.zeros((1, 0, 2)), np.zeros((1, 0)), np.zeros((1, 0)), np.zeros((1, 0)),
                           np.zeros((1, 0)), np.zeros((1, 0, 3)), 1e-6, np.float32)
    assert out.shape == (1, 3, 4, 6) and not out.any() and not wsum.any()


@pytest.mark.parametrize("name", ["render_small_c3", "render_narrow_c3", "render_c17", "render_n1"])
def test_chunked_torch_port_matches_reference(name):
    """The torch restatement that is timed as the CPU baseline gives the reference's numbers."""
    import torch

    from oracle import chunked_port as cp

    g = load_golden(name)
    t = {k: torch.from_numpy(g[k]) for k in ("positions", "colors", "scales", "rotations", "alphas", "x", "y", "gout")}
    out, grads = cp.render_fwd_bwd(t["positions"], t["colors"], t["scales"], t["rotations"], t["alphas"], t["x"],
                                   t["y"], lambda o: t["gout"], float(g["eps"]))
    assert_close(out.numpy(), g["out"], 1e-5, f"{name} image")
    for k, v in grads.items():
        assert_close(v.numpy(), g["g_" + k], 2e-5, f"{name} d_{k}")
