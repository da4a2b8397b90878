"""The dense debugging path: ``naive_gaussian_2d`` and ``render(..., fused=False)``
(reference src/igs/gs2d.py:24-44, :598-609).  Plain torch ops, differentiable by autograd,
so it gives the TRUE gradient of the forward; the reference's fixture holds the image and
the autograd gradients of its own dense function on the same inputs.

The CPU test holds the function to the fixture; the GPU tests run it on CUDA tensors and set
the fused kernels' "exact" gradient mode against it.
"""
import numpy as np
import pytest
import torch

from tests._util import assert_close, load_golden

TOL = 1e-4
NAMES = ("x", "y", "positions", "c00", "c01", "c11", "alphas", "colors")


def _dense_on(device):
    from igs_b200.gs2d import naive_gaussian_2d

    g = load_golden("kernel_xy_c3")
    leaves = [torch.from_numpy(g[k]).to(device).requires_grad_() for k in NAMES]
    out = naive_gaussian_2d(*leaves, float(g["eps"]))
    out.backward(torch.from_numpy(g["gout"]).to(device))
    return g, out, leaves


def test_naive_gaussian_2d_matches_the_reference_dense_fixture_on_cpu():
    g, out, leaves = _dense_on("cpu")
    assert_close(out.detach().numpy(), g["out_dense"], 1e-5, "dense image")
    for k, t in zip(NAMES, leaves):
        assert_close(t.grad.numpy(), g[f"g_exact_{k}"], TOL, f"autograd d_{k}")


@pytest.mark.gpu
def test_naive_gaussian_2d_matches_the_reference_dense_fixture_on_gpu():
    g, out, leaves = _dense_on(torch.device("cuda", 0))
    assert_close(out.detach().cpu().numpy(), g["out_dense"], 1e-5, "dense image")
    for k, t in zip(NAMES, leaves):
        assert_close(t.grad.cpu().numpy(), g[f"g_exact_{k}"], TOL, f"autograd d_{k}")


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["render_small_c3", "render_c4"])
def test_render_unfused_against_fixture_oracle_and_exact_mode(name):
    """render(fused=False): the image equals the reference's fused image (same formula); its
    autograd gradients equal the fp64 oracle's exact-mode gradients and the fused CUDA path in
    exact mode."""
    from igs_b200 import gs2d
    from oracle import splat_oracle as so

    dev = torch.device("cuda", 0)
    g = load_golden(name)
    names = ("positions", "colors", "scales", "rotations", "alphas")
    eps = float(g["eps"])

    def run(fused):
        leaves = {k: torch.from_numpy(g[k]).to(dev).requires_grad_() for k in names}
        out = gs2d.gaussian_splatting_2d(*[leaves[k] for k in names], torch.from_numpy(g["x"]).to(dev),
                                         torch.from_numpy(g["y"]).to(dev), eps, fused)
        out.backward(torch.from_numpy(g["gout"]).to(dev))
        return out.detach().cpu().numpy(), {k: v.grad.cpu().numpy() for k, v in leaves.items()}

    out_dense, g_dense = run(False)
    with gs2d.grad_mode("exact"):
        out_fused, g_fused = run(True)
    assert_close(out_dense, g["out"], TOL, "dense image vs the reference's fused image")
    assert_close(out_fused, out_dense, 1e-5, "fused image vs dense image")
    _, _, o_grads = so.render_with_grads(g["positions"], g["colors"], g["scales"], g["rotations"], g["alphas"],
                                         g["x"][:, 0], g["y"][:, 0], lambda o: g["gout"], eps, mode=so.MODE_EXACT,
                                         dtype=np.float64)
    for k in names:
        assert_close(g_dense[k], o_grads[k], TOL, f"dense autograd d_{k} vs fp64 oracle (exact mode)")
        assert_close(g_fused[k], g_dense[k], TOL, f"fused exact-mode d_{k} vs dense autograd")
