"""Lossless culling: with narrow gaussians the kernels skip (gaussian, pixel tile)
combinations whose weights are exactly zero.  Skipping must not change one bit, so every
case is run with the switch on and off and compared with torch.equal; one case is also
held to the oracle."""
import numpy as np
import pytest
import torch

from tests._util import assert_close, xy_grid_np

pytestmark = pytest.mark.gpu


def _case(B, N, H, W, C, lo, hi, seed, dev):
    gen = torch.Generator().manual_seed(seed)
    d = {
        "positions": torch.rand(B, N, 2, generator=gen) * 2 - 1,
        "colors": torch.rand(B, N, C, generator=gen),
        "scales": torch.rand(B, N, 2, generator=gen) * (hi - lo) + lo,
        "rotations": torch.rand(B, N, generator=gen) * 6.2831853,
        "alphas": torch.rand(B, N, generator=gen) + 0.1,
    }
    gout = torch.randn(B, C, H, W, generator=gen)
    x, y = xy_grid_np(H, W, B)
    return {k: v.to(dev) for k, v in d.items()}, gout.to(dev), torch.from_numpy(x[:, None]).to(dev), \
        torch.from_numpy(y[:, None]).to(dev)


def _run(d, gout, x, y, culling):
    from igs_b200 import _lib
    from igs_b200.gs2d import gaussian_splatting_2d

    _lib.set_culling(culling)
    try:
        leaves = {k: v.clone().requires_grad_() for k, v in d.items()}
        out = gaussian_splatting_2d(leaves["positions"], leaves["colors"], leaves["scales"], leaves["rotations"],
                                    leaves["alphas"], x, y)
        out.backward(gout)
        torch.cuda.synchronize()
        return out.detach(), {k: v.grad for k, v in leaves.items()}
    finally:
        _lib.set_culling(True)


def _narrow_count(d, x, y):
    from igs_b200 import _lib

    _, _, ws = _lib.forward("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"],
                            x[:, 0], y[:, 0], 1e-6, keep_workspace=True)
    torch.cuda.synchronize()
    return int(ws[:16].view(torch.int32)[2])


@pytest.mark.parametrize("materialised", [True, False], ids=["checked-on-device", "stride-0"])
def test_culling_changes_no_bit(materialised):
    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 3000, 96, 160
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=7, dev=dev)
    if not materialised:
        x = x[:, :, :1, :].expand(B, 1, H, W)
        y = y[:, :, :, :1].expand(B, 1, H, W)
    assert _narrow_count(d, x, y) * 8 >= B * N, "the case must be narrow enough to switch culling on"
    o_on, g_on = _run(d, gout, x, y, True)
    o_off, g_off = _run(d, gout, x, y, False)
    assert torch.equal(o_on, o_off)
    for k in g_on:
        assert torch.equal(g_on[k], g_off[k]), k


def test_culled_result_matches_oracle():
    from oracle import splat_oracle as so

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 1200, 64, 96
    d, gout, x, y = _case(B, N, H, W, 3, 0.005, 0.04, seed=9, dev=dev)
    out, grads = _run(d, gout, x, y, True)
    P = {k: v.cpu().numpy() for k, v in d.items()}
    o_out, _, o_grads = so.render_with_grads(P["positions"], P["colors"], P["scales"], P["rotations"], P["alphas"],
                                             x[:, 0].cpu().numpy(), y[:, 0].cpu().numpy(), lambda o: gout.cpu().numpy(),
                                             1e-6, dtype=np.float64)
    assert_close(out.cpu().numpy(), o_out, 1e-4, "image")
    for k, v in grads.items():
        assert_close(v.cpu().numpy(), o_grads[k], 1e-4, f"d_{k}")


def test_culling_with_reversed_axes_and_wide_gaussians_mixed():
    """x decreasing along the row (separable but not monotone increasing): the backward must
    not take a run's ends as its range; plus a few image-wide gaussians among the narrow."""
    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 2000, 64, 128
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=11, dev=dev)
    d["scales"][:, ::97] = 0.8
    x = x.flip(-1).contiguous()
    o_on, g_on = _run(d, gout, x, y, True)
    o_off, g_off = _run(d, gout, x, y, False)
    assert torch.equal(o_on, o_off)
    for k in g_on:
        assert torch.equal(g_on[k], g_off[k]), k
