"""The benchmark configurations other than the headline one, at their full sizes (config 4
on one of its 64 batch elements), each checked against the fp64 oracle on random subsets:
the image at sampled pixels, the per-gaussian gradients (sums over ALL pixels) for sampled
gaussians.  The oracle accepts any set of sample points and any subset of gaussians, given
the device's own per-pixel weight sums, so these checks cost seconds whatever the size.
"""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-4


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda", 0)


def _np(t):
    return t.detach().cpu().numpy()


def subset_check(d, out, gout, grads, n_pix=192, n_gauss=24, seed=0, eps=1e-6, tol=TOL):
    """d: dict of device tensors (positions, colors, scales, rotations, alphas, x, y);
    out, gout: [B,C,H,W]; grads: dict of device gradients shaped like the parameters."""
    from igs_b200 import _lib
    from oracle import splat_oracle as so

    B, C, H, W = out.shape
    N = d["positions"].shape[1]
    rng = np.random.default_rng(seed)
    P = {k: _np(d[k]) for k in ("positions", "colors", "scales", "rotations", "alphas")}
    x, y = _np(d["x"].expand(B, 1, H, W))[:, 0], _np(d["y"].expand(B, 1, H, W))[:, 0]

    # image at sampled pixels: an H=1, W=K "image" for the oracle
    idx = rng.choice(H * W, size=min(n_pix, H * W), replace=False)
    xs, ys = x.reshape(B, -1)[:, idx][:, None, :], y.reshape(B, -1)[:, idx][:, None, :]
    o_out, _ = so.render(P["positions"], P["colors"], P["scales"], P["rotations"], P["alphas"], xs, ys, eps,
                         dtype=np.float64)
    got = _np(out).reshape(B, C, -1)[:, :, idx][:, :, None, :]
    err = np.abs(got - o_out).max() / max(np.abs(_np(out)).max(), 1e-30)
    assert err <= tol, f"image at sampled pixels: {err:.3e}"

    # gradients of sampled gaussians, from the device's weight sums (ones-colour forward)
    sel = np.sort(rng.choice(N, size=min(n_gauss, N), replace=False))
    _, wsum = _lib.forward("sr", d["positions"].contiguous(), d["scales"].contiguous(), d["rotations"].contiguous(),
                           None, d["alphas"].contiguous(), torch.ones_like(d["colors"]).contiguous(),
                           d["x"].expand(B, 1, H, W)[:, 0], d["y"].expand(B, 1, H, W)[:, 0], eps)
    S = {k: v[:, sel] for k, v in P.items()}
    c00, c01, c11 = so.cov_inv(S["scales"], S["rotations"], eps, np.float64)
    gr = so.backward(x, y, S["positions"], c00, c01, c11, S["alphas"], S["colors"], _np(wsum), _np(out), _np(gout),
                     eps, so.MODE_REFERENCE, False, np.float64)
    gs, grot = so.cov_inv_backward(S["scales"], S["rotations"], gr["c00"], gr["c01"], gr["c11"], eps, np.float64)
    want = {"positions": gr["positions"], "colors": gr["colors"], "scales": gs, "rotations": grot,
            "alphas": gr["alphas"]}
    errs = {}
    for k, w in want.items():
        if k not in grads or grads[k] is None:
            continue
        full = _np(grads[k])
        errs[k] = float(np.abs(full[:, sel] - w).max() / max(np.abs(full).max(), 1e-30))
        assert errs[k] <= tol, f"d_{k} on sampled gaussians: {errs[k]:.3e}"
    return errs


def _render_and_backward(d, loss_fn):
    from igs_b200.gs2d import gaussian_splatting_2d

    names = ("positions", "colors", "scales", "rotations", "alphas")
    leaves = {k: d[k].clone().requires_grad_() for k in names}
    out = gaussian_splatting_2d(*[leaves[k] for k in names], d["x"], d["y"])
    out.retain_grad()
    loss = loss_fn(out)
    loss.backward()
    return out.detach(), out.grad.detach(), {k: v.grad for k, v in leaves.items()}, float(loss.detach())


def test_cfg3_single_image_fit_shape(dev):
    """B=1, N=16384, 512x512, C=3, scales U[0.05,0.3]: one forward + backward."""
    from igs_b200 import workloads

    cfg = workloads.CONFIGS["cfg3"]
    d = workloads.draw(cfg, device=dev)
    out, gout, grads, _ = _render_and_backward(d, lambda o: torch.nn.functional.mse_loss(o, d["target"]))
    subset_check(d, out, gout, grads, seed=3)


def _sinusoid_target(x, y, seed=33):
    """The fit protocol's target: per channel a sum of 64 random sinusoids over the sample
    grid (x, y: [H,W] CPU tensors), min-max normalised; [1,3,H,W]."""
    gen = torch.Generator().manual_seed(seed)
    a = torch.rand(3, 64, generator=gen)
    f = torch.rand(3, 64, 2, generator=gen) * 16 - 8
    ph = torch.rand(3, 64, generator=gen) * 2 * math.pi
    tgt = (a[:, :, None, None] * torch.sin(math.pi * (f[:, :, 0, None, None] * x + f[:, :, 1, None, None] * y)
                                           + ph[:, :, None, None])).sum(1)
    tgt = (tgt - tgt.amin((1, 2), keepdim=True)) / (tgt.amax((1, 2), keepdim=True) - tgt.amin((1, 2), keepdim=True))
    return tgt[None].contiguous()


def test_cfg3_adam_steps_reduce_the_loss(dev):
    """The fit protocol: Adam (lr 1e-2) on the five parameter tensors against a smooth
    target (sum of 64 random sinusoids per channel, min-max normalised); the loss must go
    down, and nothing may turn non-finite when scales drift through zero."""
    from igs_b200 import workloads
    from igs_b200.gs2d import gaussian_splatting_2d

    cfg = workloads.CONFIGS["cfg3"]
    d = workloads.draw(cfg, device=dev, with_target=False)
    tgt = _sinusoid_target(d["x"][0, 0].cpu(), d["y"][0, 0].cpu()).to(dev)
    names = ("positions", "colors", "scales", "rotations", "alphas")
    params = [d[k].clone().requires_grad_() for k in names]
    opt = torch.optim.Adam(params, lr=1e-2)
    losses = []
    for _ in range(60):
        opt.zero_grad(set_to_none=True)
        out = gaussian_splatting_2d(*params, d["x"], d["y"])
        loss = torch.nn.functional.mse_loss(out, tgt)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert all(math.isfinite(v) for v in losses)
    assert losses[-1] < 0.5 * losses[0], (losses[0], losses[-1])
    assert all(bool(torch.isfinite(p).all()) for p in params)


NAMES = ("positions", "colors", "scales", "rotations", "alphas")


def _oracle_loss_and_grads(P, x, y, tgt):
    """MSE loss and its gradients from the fp64 oracle alone; P: dict of numpy parameters."""
    from oracle import splat_oracle as so

    out, _, grads = so.render_with_grads(P["positions"], P["colors"], P["scales"], P["rotations"], P["alphas"], x, y,
                                         lambda o: 2 * (o - tgt) / o.size, 1e-6, dtype=np.float64)
    return float(((out - tgt) ** 2).mean()), out, grads


class _NumpyAdam:
    """torch.optim.Adam's update (no weight decay, no amsgrad) in float64 on float32 parameters."""

    def __init__(self, params, lr=1e-2, b1=0.9, b2=0.999, eps=1e-8):
        self.lr, self.b1, self.b2, self.eps, self.t = lr, b1, b2, eps, 0
        self.m = {k: np.zeros(v.shape) for k, v in params.items()}
        self.v = {k: np.zeros(v.shape) for k, v in params.items()}

    def step(self, params, grads):
        self.t += 1
        for k in params:
            g = np.asarray(grads[k], np.float64)
            self.m[k] = self.b1 * self.m[k] + (1 - self.b1) * g
            self.v[k] = self.b2 * self.v[k] + (1 - self.b2) * g * g
            denom = np.sqrt(self.v[k]) / math.sqrt(1 - self.b2 ** self.t) + self.eps
            params[k] = (params[k].astype(np.float64) - self.lr / (1 - self.b1 ** self.t) * self.m[k] / denom
                         ).astype(np.float32)


def _assert_grads(got, want, what):
    from tests._util import assert_close

    ref_scale = max(float(np.abs(w).max()) for w in want.values())
    for k, w in want.items():
        if float(np.abs(w).max()) < 1e-9 * ref_scale:  # a gradient that is zero but for rounding
            assert float(np.abs(got[k]).max()) <= 1e-6 * ref_scale, f"{what} d_{k}"
        else:
            assert_close(got[k], w, TOL, f"{what} d_{k}")


def test_fit_protocol_first_adam_steps_against_an_oracle_driven_adam(dev):
    """The single-image fit protocol at a reduced size (N=1024, 64x64; same distributions,
    target and optimiser as the full one): three Adam steps of gaussian_splatting_2d on the
    device against Adam driven by the CPU oracle alone.  At every step the loss and all five
    gradients are compared at the device's current parameters, and the independent oracle
    trajectory's losses and parameters must stay with the device's."""
    from igs_b200 import workloads
    from igs_b200.gs2d import gaussian_splatting_2d

    cfg = workloads.SplatConfig("cfg3_small", 1, 1024, 64, 64, 3, 0.05, 0.30, seed=3)
    d = workloads.draw(cfg, device="cpu", with_target=False)
    tgt = _sinusoid_target(d["x"][0, 0], d["y"][0, 0])
    x, y, tgt_np = _np(d["x"])[:, 0], _np(d["y"])[:, 0], _np(tgt)
    params = [d[k].to(dev).clone().requires_grad_() for k in NAMES]
    opt = torch.optim.Adam(params, lr=1e-2)
    oracle_params = {k: _np(d[k]).copy() for k in NAMES}
    oracle_adam = _NumpyAdam(oracle_params)
    xd, yd, tgt_d = d["x"].to(dev), d["y"].to(dev), tgt.to(dev)
    for step in range(3):
        opt.zero_grad(set_to_none=True)
        out = gaussian_splatting_2d(*params, xd, yd)
        loss = torch.nn.functional.mse_loss(out, tgt_d)
        loss.backward()
        here = {k: _np(p) for k, p in zip(NAMES, params)}
        o_loss, o_out, o_grads = _oracle_loss_and_grads(here, x, y, tgt_np)
        assert abs(float(loss) - o_loss) <= 1e-5 * o_loss, (step, float(loss), o_loss)
        _assert_grads({k: _np(p.grad) for k, p in zip(NAMES, params)}, o_grads, f"step {step}")
        # the oracle's own trajectory: its gradients at ITS parameters, its Adam
        t_loss, _, t_grads = _oracle_loss_and_grads(oracle_params, x, y, tgt_np)
        assert abs(float(loss) - t_loss) <= 1e-4 * t_loss, (step, float(loss), t_loss)
        oracle_adam.step(oracle_params, t_grads)
        opt.step()
    for k, p in zip(NAMES, params):
        diff = np.abs(_np(p) - oracle_params[k])
        # Adam divides by |g|: the few parameters whose gradient is ~1e-8 may step differently
        assert float(np.percentile(diff, 99)) <= 1e-5, (k, float(np.percentile(diff, 99)), float(diff.max()))


@pytest.mark.parametrize("fused", [True, False], ids=["fused-call", "autograd-route"])
def test_image_fitter_steps_against_an_oracle_driven_adam(fused, dev):
    """igs_b200.fit: three steps of ImageFitter + Adam (the loop fit() runs, eager; through
    the fused render + MSE + gradient call and through autograd) against
    the oracle-driven Adam in the fitter's own parametrisation (scales = exp(log_scale) + eps,
    opacities one): per-step loss and the gradients of position, log-scale, rotation, colour."""
    from igs_b200 import fit

    N, H, W = 1024, 64, 64
    gen = torch.Generator().manual_seed(5)
    model = fit.ImageFitter(N, 3, init_log_scale=-3.0)
    with torch.no_grad():  # generic starting values: no two gaussians alike, none isotropic
        model.position.add_(torch.randn(1, N, 2, generator=gen) * 0.02)
        model.log_scale.add_(torch.rand(1, N, 2, generator=gen) * 0.7)
        model.rotation.copy_(torch.rand(1, N, generator=gen) * 2 * math.pi)
        model.color.copy_(torch.rand(1, N, 3, generator=gen))
    start = {k: v.detach().clone().numpy() for k, v in model.named_parameters()}
    model.to(dev)
    xg, yg = model.grids((H, W))
    x, y = _np(xg.expand(1, 1, H, W))[:, 0], _np(yg.expand(1, 1, H, W))[:, 0]
    tgt = _sinusoid_target(torch.from_numpy(x[0]), torch.from_numpy(y[0]))
    tgt_np, tgt_d = _np(tgt), tgt.to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    oracle_params = {k: v.copy() for k, v in start.items()}
    oracle_adam = _NumpyAdam(oracle_params)
    alphas = np.ones((1, N), np.float32)

    def oracle_at(p):
        scales = np.exp(p["log_scale"].astype(np.float64)) + fit.EPS
        P = {"positions": p["position"], "colors": p["color"], "scales": scales, "rotations": p["rotation"],
             "alphas": alphas}
        loss, _, g = _oracle_loss_and_grads(P, x, y, tgt_np)
        return loss, {"position": g["positions"], "color": g["colors"], "rotation": g["rotations"],
                      "log_scale": g["scales"] * np.exp(p["log_scale"].astype(np.float64))}

    for step in range(3):
        here = {k: _np(v) for k, v in model.named_parameters()}
        loss = fit._eager_step(model, opt, tgt_d, fused=fused)  # render, MSE, backward, Adam step
        o_loss, o_grads = oracle_at(here)
        assert abs(float(loss) - o_loss) <= 1e-5 * o_loss, (step, float(loss), o_loss)
        _assert_grads({k: _np(v.grad) for k, v in model.named_parameters()}, o_grads, f"step {step}")
        t_loss, t_grads = oracle_at(oracle_params)
        assert abs(float(loss) - t_loss) <= 1e-4 * t_loss, (step, float(loss), t_loss)
        oracle_adam.step(oracle_params, t_grads)
    for k, v in model.named_parameters():
        diff = np.abs(_np(v) - oracle_params[k])
        assert float(np.percentile(diff, 99)) <= 1e-5, (k, float(np.percentile(diff, 99)), float(diff.max()))


def test_cfg3_one_full_size_step_against_the_oracle_alone(dev):
    """One step of the single-image fit at its full size (B=1, N=16384, 512x512): loss, image
    and every gradient of every gaussian against the fp64 oracle's own forward and backward
    (nothing taken from the device)."""
    from igs_b200 import workloads
    from igs_b200.gs2d import gaussian_splatting_2d
    from tests._util import assert_close

    cfg = workloads.CONFIGS["cfg3"]
    d = workloads.draw(cfg, device="cpu", with_target=False)
    tgt = _sinusoid_target(d["x"][0, 0], d["y"][0, 0])
    params = [d[k].to(dev).clone().requires_grad_() for k in NAMES]
    out = gaussian_splatting_2d(*params, d["x"].to(dev), d["y"].to(dev))
    loss = torch.nn.functional.mse_loss(out, tgt.to(dev))
    loss.backward()
    o_loss, o_out, o_grads = _oracle_loss_and_grads({k: _np(d[k]) for k in NAMES}, _np(d["x"])[:, 0],
                                                    _np(d["y"])[:, 0], _np(tgt))
    assert abs(float(loss) - o_loss) <= 1e-5 * o_loss
    assert_close(_np(out), o_out, 1e-5, "image")
    _assert_grads({k: _np(p.grad) for k, p in zip(NAMES, params)}, o_grads, "cfg3")


def test_cfg4_feature_map_regime_one_batch_element(dev):
    """C=16 colours ~ N(0,1), N=65536, 512x512, scales U[0.02,0.2] (config 4, one of its 64
    independent batch elements)."""
    from igs_b200 import workloads

    cfg = workloads.CONFIGS["cfg4"]
    d = workloads.draw(cfg, B=1, device=dev)
    out, gout, grads, _ = _render_and_backward(d, lambda o: torch.nn.functional.mse_loss(o, d["target"]))
    subset_check(d, out, gout, grads, n_pix=96, n_gauss=8, seed=4)


def test_cfg1_module_at_init(dev):
    """GaussianSplatting2D(32 per feature, 1024) with random-init weights on x ~ N(0,1)
    [1,128,1024]: N=4096 narrow gaussians (scale ~ e^-4) at 256x256, where about one pixel
    in a hundred has a weight sum near zero.  The splat inside the module is checked on
    subsets; the projection in front of it is plain torch."""
    from igs_b200 import GaussianSplatting2D

    torch.manual_seed(1)
    m = GaussianSplatting2D(32, 1024).to(dev)
    feat = torch.randn(1, 128, 1024, device=dev, requires_grad=True)
    out, gs_feature = m(feat, size=(256, 256))
    gs_feature.retain_grad()
    out.retain_grad()
    tgt = torch.rand(1, 3, 256, 256, device=dev)
    torch.nn.functional.mse_loss(out, tgt).backward()
    assert out.shape == (1, 3, 256, 256) and gs_feature.shape == (1, 4096, 9)
    assert bool(torch.isfinite(m.proj.weight.grad).all()) and bool(torch.isfinite(feat.grad).all())

    pos, log_sc, rot, _, col = gs_feature.detach().split([2, 2, 1, 1, 3], dim=-1)
    xg, yg = GaussianSplatting2D.xy_grid((256, 256), dev)
    d = {"positions": pos.contiguous(), "colors": col.contiguous(), "scales": torch.exp(log_sc) + 1e-6,
         "rotations": rot[..., 0].contiguous(), "alphas": torch.ones(1, 4096, device=dev), "x": xg[None], "y": yg[None]}
    g = gs_feature.grad
    sc = d["scales"]
    grads = {"positions": g[..., 0:2], "colors": g[..., 6:9], "rotations": g[..., 4],
             # d/d log_scale = d/d scale * exp(log_scale); undo it to compare scale gradients
             "scales": g[..., 2:4] / (sc - 1e-6)}
    subset_check(d, out.detach(), out.grad.detach(), grads, n_pix=256, n_gauss=32, seed=1)


@pytest.mark.parametrize("tag", ["grid", "posmap"])
def test_module_optional_inputs_match_reference_fixture(tag, dev):
    """The module with a caller-supplied warped sampling grid (general kernels) and with
    pos_map_offset=True plus a scale factor, against outputs of the reference module."""
    from igs_b200 import GaussianSplatting2D
    from tests._util import assert_close, load_golden

    g = load_golden("module_variants")
    t = lambda k: torch.from_numpy(g[k]).to(dev)
    m = GaussianSplatting2D(int(g["n_per"]), int(g["emb"]), 3, pos_map_offset=(tag == "posmap")).to(dev)
    with torch.no_grad():
        m.proj.weight.copy_(t(f"{tag}_weight"))
        m.proj.bias.copy_(t(f"{tag}_bias"))
    feat = t(f"{tag}_feature").requires_grad_()
    if tag == "grid":
        out, _ = m(feat, grid=t("grid"))
    else:
        out, _ = m(feat, size=(int(g["H"]), int(g["W"])), scale=int(g["scale"]))
    torch.nn.functional.mse_loss(out, t("target")).backward()
    assert_close(_np(out), g[f"{tag}_out"], TOL, f"{tag} image")
    assert_close(_np(m.proj.weight.grad), g[f"{tag}_g_weight"], TOL, f"{tag} d_weight")
    assert_close(_np(m.proj.bias.grad), g[f"{tag}_g_bias"], TOL, f"{tag} d_bias")
    assert_close(_np(feat.grad), g[f"{tag}_g_feature"], TOL, f"{tag} d_feature")


@pytest.mark.parametrize("name", ["narrow", "narrow64k"])
def test_narrow_workloads_ordered_culling_path_against_the_oracle(name, dev):
    """The image-compression regime at full size (16384 / 65536 narrow gaussians on a
    1024x1024 grid), forward and backward taking the gaussians in a spatial order: stage
    lists in the forward, the task queue in the backward, 97-99 % of the pairs skipped.
    Image at sampled pixels and gradients of sampled gaussians against the fp64 oracle,
    which skips nothing."""
    from igs_b200 import _lib, workloads

    cfg = workloads.CONFIGS[name]
    d = workloads.draw(cfg, device=dev)
    _lib.set_backward_sort("on")
    try:
        out, gout, grads, _ = _render_and_backward(d, lambda o: torch.nn.functional.mse_loss(o, d["target"]))
    finally:
        _lib.set_backward_sort("auto")
    subset_check(d, out, gout, grads, n_pix=128, n_gauss=16, seed=7)
