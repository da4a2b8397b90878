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
    _lib.set_backward_sort("off")  # one partition of the rows throughout: bits are comparable
    try:
        leaves = {k: v.clone().requires_grad_() for k, v in d.items()}
        out = gaussian_splatting_2d(leaves["positions"], leaves["colors"], leaves["scales"], leaves["rotations"],
                                    leaves["alphas"], x, y)
        out.backward(gout)
        torch.cuda.synchronize()
        return out.detach(), {k: v.grad for k, v in leaves.items()}
    finally:
        _lib.set_culling(True)
        _lib.set_backward_sort("auto")


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


@pytest.mark.parametrize("level", ["scales", "cov_inv"])
def test_culling_with_strongly_anisotropic_rotated_gaussians(level):
    """Long thin gaussians at random angles (axis ratios 1000:1 and 2000:1): the zero-weight
    box must come out conservative although the determinant of the inverse covariance cancels
    almost completely in fp32.  Culling on and off: the same bits, from the scale / rotation
    entry and from the inverse-covariance entry."""
    from igs_b200 import _lib, gs2d

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 2048, 96, 128
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=13, dev=dev)
    d["scales"][:, ::2, 0] = 0.4
    d["scales"][:, ::2, 1] = 0.0004
    d["scales"][:, 1::4, 0] = 0.0002
    d["scales"][:, 1::4, 1] = 0.4
    if level == "scales":
        o_on, g_on = _run(d, gout, x, y, True)
        o_off, g_off = _run(d, gout, x, y, False)
    else:
        c00, c01, c11 = gs2d._cov_inv_torch(d["scales"], d["rotations"], 1e-6)

        def run(culling):
            _lib.set_culling(culling)
            _lib.set_backward_sort("off")
            try:
                leaves = [t.clone().requires_grad_() for t in (d["positions"], c00, c01, c11, d["alphas"], d["colors"])]
                out = gs2d.GaussianSplatting2DKernel.apply(x, y, *leaves)
                out.backward(gout)
                torch.cuda.synchronize()
                return out.detach(), {i: t.grad for i, t in enumerate(leaves)}
            finally:
                _lib.set_culling(True)
                _lib.set_backward_sort("auto")

        o_on, g_on = run(True)
        o_off, g_off = run(False)
    assert torch.equal(o_on, o_off)
    for k in g_on:
        assert torch.equal(g_on[k], g_off[k]), k


@pytest.mark.parametrize("C", [5, 8, 12, 16, 17])
def test_many_channels_culling_changes_no_bit_and_matches_the_oracle(C):
    """5 to 8 and 9 to 16 channels run the row-streaming separable backward (two gaussians per
    packed operand; instantiated for 8 and 16, zero-padded in between) and its skipping
    instantiation; 17 channels are a chunk of 16 plus one and take the general kernels.  Odd image sizes, a ragged gaussian count, a few image-wide gaussians
    among the narrow ones.  Culling on / off: the same bits; and the culled result against the
    fp64 oracle."""
    from oracle import splat_oracle as so

    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 1501, 71, 150
    d, gout, x, y = _case(B, N, H, W, C, 0.004, 0.03, seed=50 + C, dev=dev)
    d["scales"][:, ::131] = 0.7
    assert _narrow_count(d, x, y) * 8 >= B * N
    o_on, g_on = _run(d, gout, x, y, True)
    o_off, g_off = _run(d, gout, x, y, False)
    assert torch.equal(o_on, o_off)
    for k in g_on:
        assert torch.equal(g_on[k], g_off[k]), k
    P = {k: v.cpu().numpy() for k, v in d.items()}
    o_out, _, o_grads = so.render_with_grads(P["positions"], P["colors"], P["scales"], P["rotations"], P["alphas"],
                                             x[:, 0].cpu().numpy(), y[:, 0].cpu().numpy(), lambda o: gout.cpu().numpy(),
                                             1e-6, dtype=np.float64)
    assert_close(o_on.cpu().numpy(), o_out, 1e-4, "image")
    for k, v in g_on.items():
        assert_close(v.cpu().numpy(), o_grads[k], 1e-4, f"d_{k}")


@pytest.mark.parametrize("C", [8, 16])
def test_many_channels_gradients_do_not_depend_on_the_processing_order(C):
    """The row-streaming backward with an explicit order (wide and narrow gaussians): every
    gaussian's sums run over the same pixels in the same sequence whichever thread owns it."""
    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 900, 64, 96
    gen = torch.Generator().manual_seed(8)
    for lo, hi in ((0.004, 0.03), (0.2, 0.5)):
        d, gout, x, y = _case(B, N, H, W, C, lo, hi, seed=60 + C, dev=dev)
        orders = [torch.randperm(N, generator=gen).to(torch.int32).to(dev)[None].contiguous() for _ in range(2)]
        orders.append(torch.arange(N - 1, -1, -1, dtype=torch.int32, device=dev)[None].contiguous())
        res = [_backward_with(d, gout, x, y, o) for o in orders]
        for r in res[1:]:
            for k in res[0]:
                assert torch.equal(r[k], res[0][k]), (k, lo)


@pytest.mark.parametrize("C,warp", [(3, True), (17, False), (17, True)])
def test_general_kernels_take_an_order_too(C, warp):
    """The general backward (sample points off a grid; more than 16 channels in two chunks)
    with an explicit order: the partial sums are laid out by processing slot and mapped back
    through the order, so every permutation gives the same bits, and the result agrees with
    an order-less call to rounding."""
    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 777, 40, 72
    gen = torch.Generator().manual_seed(90 + C)
    d, gout, x, y = _case(B, N, H, W, C, 0.02, 0.3, seed=80 + C, dev=dev)
    if warp:
        x = (x + 0.03 * torch.sin(4 * y)).contiguous()
    orders = [torch.stack([torch.randperm(N, generator=gen) for _ in range(B)]).to(torch.int32).to(dev).contiguous()
              for _ in range(2)]
    orders.append(torch.arange(N - 1, -1, -1, dtype=torch.int32, device=dev).expand(B, N).contiguous())
    res = [_backward_with(d, gout, x, y, o) for o in orders]
    plain = _backward_with(d, gout, x, y, None)
    for k in plain:
        for r in res[1:]:
            assert torch.equal(r[k], res[0][k]), k
        assert _rel(res[0][k], plain[k]) < 2e-5, (k, _rel(res[0][k], plain[k]))


def _backward_with(d, gout, x, y, order):
    """Gradients through the library call itself, with an explicit processing order."""
    from igs_b200 import _lib

    x3, y3 = x[:, 0], y[:, 0]
    out, wsum = _lib.forward("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"], x3, y3,
                             1e-6)
    res = _lib.backward("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"], x3, y3,
                        wsum, out, gout, 1e-6, 0, False, order=order)
    torch.cuda.synchronize()
    return res


def test_box_order_sorts_by_the_clipped_box_centre():
    """igs_spatial_order_boxes against igs_spatial_order on the key it documents: per axis the
    centre of the zero-weight box clipped to the sampled extent.  Hand-made gaussians whose
    keys are known, then random ones with the key recomputed by torch (also from a
    feature-layout tensor read in place, with logarithmic scales and a position offset)."""
    import math

    from igs_b200 import _lib
    from igs_b200.gs2d import GaussianSplatting2D

    dev = torch.device("cuda", 0)
    R = 13.43  # box half-width in standard deviations of the axis
    xg, yg = GaussianSplatting2D.xy_grid((16, 16), dev)
    x3, y3 = xg, yg  # [1,16,16] views; the extent is [-1,1] x [-1,1]
    pos = torch.tensor([[[0.3, -0.2], [0.3, -0.2], [-0.9, 0.1], [0.5, 0.5], [0.1, 0.9]]], device=dev)
    sc = torch.tensor([[[0.01, 0.01],     # narrow: keeps its centre
                        [0.5, 0.5],       # covers the whole extent: the image's centre
                        [0.04, 0.01],     # sticks out on the left: placed by how far it reaches in
                        [0.01, 0.5],      # a vertical strip (rotation 0): x kept, y = centre line
                        [0.01, 0.5]]], device=dev)  # the same shape turned by 90 degrees: a horizontal strip
    rot = torch.tensor([[0.0, 0.0, 0.0, 0.0, math.pi / 2]], device=dev)
    key = torch.tensor([[[0.3, -0.2], [0.0, 0.0], [0.5 * (-1.0 + (-0.9 + R * 0.04)), 0.1], [0.5, 0.0],
                         [0.0, 0.5 * ((0.9 - R * 0.01) + 1.0)]]], device=dev)
    assert torch.equal(_lib.spatial_order_boxes(pos, x3, y3, sc, False, rot), _lib.spatial_order(key, x3, y3))
    # without rotations the larger scale stands in for both axes: the strips become image-wide
    key2 = key.clone()
    key2[0, 3] = 0.0
    key2[0, 4] = 0.0
    assert torch.equal(_lib.spatial_order_boxes(pos, x3, y3, sc), _lib.spatial_order(key2, x3, y3))
    # without scales: the centres
    assert torch.equal(_lib.spatial_order_boxes(pos, x3, y3), _lib.spatial_order(pos, x3, y3))

    # random gaussians; the lattice has 64 cells per axis, so keys are kept away from cell
    # boundaries (where one rounding decides the cell) by drawing until they are
    gen = torch.Generator().manual_seed(33)
    B, N, K = 2, 3000, 9
    xg, yg = GaussianSplatting2D.xy_grid((48, 80), dev)
    x3, y3 = xg.expand(B, -1, -1), yg.expand(B, -1, -1)
    feat = torch.zeros(B, N, K)
    feat[..., :2] = torch.rand(B, N, 2, generator=gen) * 2.4 - 1.2
    feat[..., 2:4] = torch.rand(B, N, 2, generator=gen) * 4.0 - 5.0  # log scales: e^-5 .. e^-1
    feat[..., 4] = torch.rand(B, N, generator=gen) * 6.28
    off = (torch.rand(B, N, 2, generator=gen) - 0.5) * 0.1
    lo = torch.tensor([float(xg.min()), float(yg.min())])
    hi = torch.tensor([float(xg.max()), float(yg.max())])

    def keys(f):
        p, s, r = f[..., :2].double() + off.double(), torch.exp(f[..., 2:4].double()), f[..., 4].double()
        c2 = (torch.cos(r) ** 2)[..., None]
        half = R * torch.sqrt(c2 * s * s + (1 - c2) * (s * s).flip(-1))
        return 0.5 * (torch.maximum(p - half, lo.double()) + torch.minimum(p + half, hi.double()))

    mid = 0.5 * (lo.double() + hi.double())
    for _ in range(20):
        k = keys(feat)
        cell = (k - lo) / (hi - lo) * 64.0
        # (a box that covers an axis sits exactly on the centre line in either computation)
        near = (((cell - cell.round()).abs() < 1e-3) & (k != mid)).any(-1)
        if not bool(near.any()):
            break
        feat[..., :2][near] += 0.01
    assert not bool(near.any())
    feat_d, off_d = feat.to(dev), off.to(dev)
    want = _lib.spatial_order(keys(feat).float().to(dev), x3, y3)
    got = _lib.spatial_order_boxes(feat_d[..., :2], x3, y3, feat_d[..., 2:4], True, feat_d[..., 4], off_d)
    assert torch.equal(got, want)
    # the same parameters as separate contiguous tensors with plain scales
    got2 = _lib.spatial_order_boxes((feat_d[..., :2] + off_d).contiguous(), x3, y3,
                                    torch.exp(feat_d[..., 2:4]).contiguous(), False, feat_d[..., 4].contiguous())
    assert torch.equal(got2, want)


def test_spatial_order_is_a_permutation_with_neighbours_adjacent():
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 3, 5000, 64, 96
    d, _, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=21, dev=dev)
    order = _lib.spatial_order(d["positions"], x[:, 0], y[:, 0])
    assert order.dtype == torch.int32 and order.shape == (B, N)
    assert torch.equal(order.long().sort(dim=1).values, torch.arange(N, device=dev).expand(B, N))
    for _ in range(3):  # a stable sort: the same permutation on every run
        assert torch.equal(_lib.spatial_order(d["positions"], x[:, 0], y[:, 0]), order)
    # gaussians at one and the same place share a cell and must keep their index order
    same = d["positions"].clone()
    same[:] = same[:, :1]
    assert torch.equal(_lib.spatial_order(same, x[:, 0], y[:, 0]).long(), torch.arange(N, device=dev).expand(B, N))
    # a run of 64 consecutive slots (two warps' gaussians) spans a small patch, not the image
    p = torch.gather(d["positions"], 1, order.long()[..., None].expand(B, N, 2))
    runs = p[:, : N // 64 * 64].reshape(B, -1, 64, 2)
    span = (runs.amax(2) - runs.amin(2)).amax(-1)  # [B, runs]: larger side of the run's box
    assert float(span.median()) < 0.5, float(span.median())  # the image spans 2


def _identity(B, N, dev):
    return torch.arange(N, dtype=torch.int32, device=dev).expand(B, N).contiguous()


def _rel(a, b):
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("kind", ["spatial", "random", "reversed"])
def test_processing_order_changes_no_bit(kind):
    """Whatever permutation is passed, the gradients are the same bits (each gaussian's sums
    run over the same pixels in the same sequence, whichever thread owns it).  Passing an
    order at all selects a finer partition of the rows, so against a call without one the
    sums associate differently: equal to rounding, not to the bit."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 3001, 96, 160  # N odd: the last thread's second slot is empty
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=23, dev=dev)
    d["scales"][:, ::89] = 0.7
    if kind == "spatial":
        order = _lib.spatial_order(d["positions"], x[:, 0], y[:, 0])
    elif kind == "random":
        gen = torch.Generator().manual_seed(5)
        order = torch.stack([torch.randperm(N, generator=gen) for _ in range(B)]).to(torch.int32).to(dev)
    else:
        order = torch.arange(N - 1, -1, -1, dtype=torch.int32, device=dev).expand(B, N).contiguous()
    want = _backward_with(d, gout, x, y, _identity(B, N, dev))
    got = _backward_with(d, gout, x, y, order)
    for k in want:
        assert torch.equal(got[k], want[k]), k
    _lib.set_backward_sort("off")
    try:
        plain = _backward_with(d, gout, x, y, None)
    finally:
        _lib.set_backward_sort("auto")
    for k in want:
        assert _rel(got[k], plain[k]) < 2e-6, (k, _rel(got[k], plain[k]))


@pytest.mark.parametrize("C", [1, 2, 3, 4])
def test_culling_changes_no_bit_with_an_order(C):
    """With an order the skipping is done warp by warp (each warp follows the reach of its
    own 32 gaussians); against the dense kernel on the same row partition: same bits.  A
    few image-wide and one indefinite gaussian (infinite box) are mixed in."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 4000, 200, 264
    d, gout, x, y = _case(B, N, H, W, C, 0.004, 0.03, seed=27 + C, dev=dev)
    d["scales"][:, ::211] = 0.9
    order = _lib.spatial_order(d["positions"], x[:, 0], y[:, 0])
    on = _backward_with(d, gout, x, y, order)
    _lib.set_culling(False)
    try:
        off = _backward_with(d, gout, x, y, order)
    finally:
        _lib.set_culling(True)
    for k in on:
        assert torch.equal(on[k], off[k]), k


def test_processing_order_on_general_grid_and_wide_channels():
    """The general kernels (warped grid) and a 16-channel chunk honour the order too."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 777, 48, 80
    d, gout, x, y = _case(B, N, H, W, 16, 0.01, 0.2, seed=29, dev=dev)
    x = (x + 0.01 * torch.sin(7 * y)).contiguous()
    gen = torch.Generator().manual_seed(6)
    order = torch.randperm(N, generator=gen).to(torch.int32).to(dev)[None].contiguous()
    # on a general grid and with more than 4 channels there is one partition only
    _lib.set_backward_sort("off")
    try:
        want = _backward_with(d, gout, x, y, None)
    finally:
        _lib.set_backward_sort("auto")
    got = _backward_with(d, gout, x, y, order)
    for k in want:
        assert torch.equal(got[k], want[k]), k


def _grads_via_api(d, gout, x, y):
    """Gradients through the public function (the autograd Functions are where the policy
    lives); synchronises, so a status read queued by the call has landed afterwards."""
    from igs_b200.gs2d import gaussian_splatting_2d

    leaves = {k: v.clone().requires_grad_() for k, v in d.items()}
    out = gaussian_splatting_2d(leaves["positions"], leaves["colors"], leaves["scales"], leaves["rotations"],
                                leaves["alphas"], x, y)
    out.backward(gout)
    torch.cuda.synchronize()
    return {k: v.grad for k, v in leaves.items()}


def test_auto_policy_learns_that_gaussians_are_narrow(monkeypatch):
    """'auto' starts unsorted, waits for the device's narrow count once (the first call on
    gaussians nothing is known about; every later look is read back without blocking), and
    sorts from the next call on; from then on the gradients are the same bits call after call,
    and equal to the first call's to rounding."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 4096, 128, 128
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.02, seed=31, dev=dev)
    monkeypatch.setattr(_lib, "AUTO_ORDER_MIN_EVALS", 0)  # small case: lift the size threshold of "auto"
    _lib.set_backward_sort("auto")  # forgets what earlier tests taught it
    first = _grads_via_api(d, gout, x, y)
    memo = _lib._shape_memos[(dev.index, B, N, H, W)]
    assert memo.calls == 2 and memo.narrow is True  # forward + backward; the forward's answer was waited for
    for _ in range(3):
        again = _grads_via_api(d, gout, x, y)
    assert memo.narrow is True
    once_more = _grads_via_api(d, gout, x, y)
    for k in first:
        assert torch.equal(once_more[k], again[k]), k
        assert _rel(again[k], first[k]) < 2e-6, k
    # wide gaussians never switch it on, and are remembered as wide (later calls pass the hint)
    # (forgetting first: a new image size would otherwise start from what this many gaussians
    # showed last, narrow, and be corrected a call later, with another partition of the sums)
    _lib.forget_what_calls_learnt()
    d2, gout2, x2, y2 = _case(B, N, 100, W, 3, 0.3, 0.6, seed=32, dev=dev)
    wide_first = _grads_via_api(d2, gout2, x2, y2)
    for _ in range(3):
        wide_again = _grads_via_api(d2, gout2, x2, y2)
    assert _lib._shape_memos[(dev.index, B, N, 100, W)].narrow is False
    for k in wide_first:  # with and without the hint: the same kernels do the work, the same bits
        assert torch.equal(wide_again[k], wide_first[k]), k
    # below the size threshold "auto" still learns, but orders only inside a graph capture
    monkeypatch.setattr(_lib, "AUTO_ORDER_MIN_EVALS", 5e8)
    _lib.set_backward_sort("auto")
    for _ in range(4):
        _grads_via_api(d, gout, x, y)
    memo = _lib._shape_memos[(dev.index, B, N, H, W)]
    assert memo.narrow is True
    assert _lib.order_by_policy(memo, d["positions"], None, None, x[:, 0], y[:, 0]) is None


def test_materialised_grid_is_remembered_as_separable():
    """A materialised xy_grid is checked on the device by the first call; later calls with the
    very same (unmodified) tensors pass stride-0 views and skip the check -- same bits.  An
    in-place change of the grid tensor makes the next call look again."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 600, 40, 48
    d, gout, x, y = _case(B, N, H, W, 3, 0.1, 0.4, seed=33, dev=dev)
    _lib.forget_what_calls_learnt()
    first = _grads_via_api(d, gout, x, y)
    entry = _lib._grid_memos[(id(x), id(y))]
    n0 = _lib.launch_count()
    second = _grads_via_api(d, gout, x, y)   # the answer of the first call's check is picked up here
    n1 = _lib.launch_count()
    assert entry.kind == "separable"
    third = _grads_via_api(d, gout, x, y)
    assert _lib.launch_count() - n1 <= n1 - n0
    for k in first:
        assert torch.equal(second[k], first[k]) and torch.equal(third[k], first[k]), k
    # a warped grid in the same storage: the version counter moved, so the entry no longer applies
    x.add_(0.01 * torch.sin(7 * y))
    _lib.set_backward_sort("off")
    try:
        warped = _grads_via_api(d, gout, x, y)  # checked on the device again: not separable
        hinted = _grads_via_api(d, gout, x, y)  # picks the answer up: IGS_HINT_GENERAL_GRID
        assert _lib._grid_memos[(id(x), id(y))].kind == "general"
    finally:
        _lib.set_backward_sort("auto")
    for k in warped:
        assert torch.equal(hinted[k], warped[k]), k


@pytest.mark.parametrize("C", [1, 3, 4])
def test_ordered_forward_skips_stages_without_changing_a_bit(C):
    """With an order the forward records are written in that order and a CTA lists the stages
    (128 consecutive gaussians) whose box meets its pixels.  Same order, culling on / off:
    the same bits.  Against the order-less forward: equal to rounding (another sequence of
    additions).  A few image-wide and one NaN-positioned gaussian are mixed in."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 2, 5000, 136, 200
    d, _, x, y = _case(B, N, H, W, C, 0.004, 0.03, seed=41 + C, dev=dev)
    d["scales"][:, ::173] = 0.9
    x3, y3 = x[:, 0], y[:, 0]
    order = _lib.spatial_order(d["positions"], x3, y3)
    args = ("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"], x3, y3, 1e-6)
    on, wsum_on, ws = _lib.forward(*args, order=order, keep_workspace=True)
    executed = _lib.read_executed(ws)
    _lib.set_culling(False)
    try:
        off, wsum_off = _lib.forward(*args, order=order)
    finally:
        _lib.set_culling(True)
    plain, wsum_plain = _lib.forward(*args)
    torch.cuda.synchronize()
    assert torch.equal(on, off) and torch.equal(wsum_on, wsum_off)
    assert 0 < executed < 0.5 * B * N * H * W, executed
    assert _rel(on, plain) < 2e-6 and _rel(wsum_on, wsum_plain) < 2e-6
    # the same call again: the same bits (the order is deterministic, and so are the sums)
    again, _ = _lib.forward(*args, order=_lib.spatial_order(d["positions"], x3, y3))
    assert torch.equal(again, on)


def test_ordered_forward_keeps_nan_where_the_reference_has_it():
    """A NaN position poisons every pixel in the reference (NaN weight); stage boxes must not
    cull such a gaussian away."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 1000, 64, 96
    d, _, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=51, dev=dev)
    d["positions"][0, 123, 0] = float("nan")
    x3, y3 = x[:, 0], y[:, 0]
    order = _lib.spatial_order(d["positions"], x3, y3)
    args = ("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"], x3, y3, 1e-6)
    with_order, _ = _lib.forward(*args, order=order)
    without, _ = _lib.forward(*args)
    assert torch.equal(torch.isnan(with_order), torch.isnan(without))
    assert bool(torch.isnan(without).all())


def _same_with_nans(a, b):
    return torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(torch.nan_to_num(a), torch.nan_to_num(b))


@pytest.mark.parametrize("what", ["position", "color", "alpha", "gout"])
def test_non_finite_values_propagate_as_without_culling(what):
    """0 * NaN is NaN: skipping a zero weight is only lossless while what it multiplies is
    finite.  A gaussian with a non-finite parameter therefore reaches every pixel, and a
    non-finite upstream gradient switches the backward to its dense kernel; either way the
    NaNs land where the dense kernels (and the reference) put them."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 3000, 96, 160
    d, gout, x, y = _case(B, N, H, W, 3, 0.004, 0.03, seed=61, dev=dev)
    if what == "position":
        d["positions"][0, 77, 1] = float("nan")
    elif what == "color":
        d["colors"][0, 78, 2] = float("inf")
    elif what == "alpha":
        d["alphas"][0, 79] = float("nan")
    else:
        gout[0, 1, 40, 50] = float("nan")
    res = {}
    for sort in ("off", "on"):
        for culling in (True, False):
            _lib.set_backward_sort(sort)
            _lib.set_culling(culling)
            try:
                leaves = {k: v.clone().requires_grad_() for k, v in d.items()}
                from igs_b200.gs2d import gaussian_splatting_2d
                out = gaussian_splatting_2d(leaves["positions"], leaves["colors"], leaves["scales"],
                                            leaves["rotations"], leaves["alphas"], x, y)
                out.backward(gout)
                torch.cuda.synchronize()
                res[(sort, culling)] = (out.detach(), {k: v.grad for k, v in leaves.items()})
            finally:
                _lib.set_culling(True)
                _lib.set_backward_sort("auto")
    for sort in ("off", "on"):
        o_on, g_on = res[(sort, True)]
        o_off, g_off = res[(sort, False)]
        assert _same_with_nans(o_on, o_off), (what, sort, "image")
        for k in g_on:
            assert _same_with_nans(g_on[k], g_off[k]), (what, sort, k)
    if what in ("position", "alpha"):
        assert bool(torch.isnan(res[("off", True)][0]).all())  # the reference's image is all NaN here
    elif what == "color":
        assert not bool(torch.isfinite(res[("off", True)][0][:, 2]).any())  # ... in the channel that has the inf
    else:
        assert bool(torch.isnan(res[("off", True)][1]["positions"]).all())


def test_entries_of_an_order_that_are_no_index_are_not_followed():
    """A malformed order (entries outside 0..N-1) must not send a kernel outside its arrays:
    those slots stay empty, every gaussian that is listed still gets its gradient."""
    from igs_b200 import _lib

    dev = torch.device("cuda", 0)
    B, N, H, W = 1, 500, 48, 64
    d, gout, x, y = _case(B, N, H, W, 3, 0.01, 0.2, seed=71, dev=dev)
    good = _backward_with(d, gout, x, y, _identity(B, N, dev))
    bad = _identity(B, N, dev).clone()
    bad[0, 10] = -5
    bad[0, 20] = N + 3
    got = _backward_with(d, gout, x, y, bad)
    keep = torch.ones(N, dtype=torch.bool, device=dev)
    keep[10] = keep[20] = False
    for k in good:
        assert torch.equal(got[k][:, keep], good[k][:, keep]), k
    out, _, ws = _lib.forward("sr", d["positions"], d["scales"], d["rotations"], None, d["alphas"], d["colors"],
                              x[:, 0], y[:, 0], 1e-6, order=bad, keep_workspace=True)
    assert _lib.read_status(ws) == 0 and bool(torch.isfinite(out).all())
