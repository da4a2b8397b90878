"""Generate the golden fixtures in this folder by RUNNING THE REFERENCE ITSELF on CPU.

Usage (only where the reference tree is present; it does not travel with the repo):

    TORCHDYNAMO_DISABLE=1 python tests/golden/make_golden.py /path/to/reference

What is executed is the reference's own code, unmodified:
``igs.gs2d.gaussian_splatting_2d`` (src/igs/gs2d.py:692) with the module-global
``GaussianSplatting2DKernel`` bound to ``GaussianSplatting2DChunkedKernel``
(src/igs/gs2d.py:265-465; the default binding, :471-476, is the Triton class, which
needs a GPU), ``GaussianSplatting2DChunkedKernel.apply`` directly for the
cov_inv-level entry, ``naive_gaussian_2d`` (:24-44) under autograd for the exact
gradient, and ``GaussianSplatting2D`` (:479-689) for the module case.
``TORCHDYNAMO_DISABLE=1`` is required because ``render`` is wrapped in
``torch.compile`` (:525), which does not build on CPU.

Each ``<case>.npz`` stores the inputs, the image, the upstream gradient that was fed
to backward and every gradient autograd returned, all float32.
"""
from __future__ import annotations

import math
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    sys.path.insert(0, os.path.join(root, "src"))
    import igs.gs2d as ref

    ref.GaussianSplatting2DKernel = ref.GaussianSplatting2DChunkedKernel
    return ref


def grids(ref, B, H, W):
    xg, yg = ref.GaussianSplatting2D.xy_grid((H, W), "cpu")
    return xg[None].repeat(B, 1, 1, 1).contiguous(), yg[None].repeat(B, 1, 1, 1).contiguous()


def draw_params(gen, B, N, C, scale_lo, scale_hi, normal_colors=False):
    pos = torch.rand(B, N, 2, generator=gen) * 2 - 1
    col = torch.randn(B, N, C, generator=gen) if normal_colors else torch.rand(B, N, C, generator=gen)
    sc = torch.rand(B, N, 2, generator=gen) * (scale_hi - scale_lo) + scale_lo
    rot = torch.rand(B, N, generator=gen) * 2 * math.pi
    al = torch.rand(B, N, generator=gen)
    return pos, col, sc, rot, al


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = np.asarray(v)
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def render_case(ref, name, seed, B, N, H, W, C, lo, hi, loss="sse", normal_colors=False, slim=False):
    """Function-level API: gaussian_splatting_2d + a dense-gradient loss.

    ``slim`` leaves out what a test can rebuild exactly (the xy_grid planes and the
    upstream gradient 2*(out-target)) to keep a full-size fixture small."""
    gen = torch.Generator().manual_seed(seed)
    pos, col, sc, rot, al = draw_params(gen, B, N, C, lo, hi, normal_colors)
    tgt = torch.rand(B, C, H, W, generator=gen)
    xg, yg = grids(ref, B, H, W)
    leaves = [t.requires_grad_() for t in (pos, col, sc, rot, al)]
    out = ref.gaussian_splatting_2d(pos, col, sc, rot, al, xg, yg)
    out.retain_grad()
    if loss == "sse":
        val = ((out - tgt) ** 2).sum()
    else:
        val = torch.nn.functional.mse_loss(out, tgt)
    # the reference's backward divides the upstream gradient in place (:371), so the
    # value fed to it is re-derived from the loss definition rather than read back
    gout = (2 * (out.detach() - tgt)) if loss == "sse" else (2 * (out.detach() - tgt) / out.numel())
    val.backward()
    extra = {} if slim else dict(x=xg, y=yg, gout=gout)
    save(name, positions=pos, colors=col, scales=sc, rotations=rot, alphas=al,
         target=tgt, out=out, loss=val.detach(), eps=np.float32(1e-6), **extra,
         g_positions=pos.grad, g_colors=col.grad, g_scales=sc.grad, g_rotations=rot.grad,
         g_alphas=al.grad)
    return leaves


def kernel_case(ref, name, seed, B, N, H, W, C):
    """cov_inv-level entry with arbitrary (non-grid) sample coordinates and
    indefinite cov_inv, as the reference's own self-checks call it
    (src/igs/gs2d.py:717-762, scripts/profiling.py:53-66); gradients of x and y
    included.  Stores the custom backward (reference mode) and autograd of the dense
    formula (exact mode) for the same inputs and upstream gradient."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.rand(B, 1, H, W, generator=gen) * 2 - 1
    y = torch.rand(B, 1, H, W, generator=gen) * 2 - 1
    pos = torch.rand(B, N, 2, generator=gen) * 2 - 1
    c00 = torch.randn(B, N, 1, 1, generator=gen) * 0.5 + 1.0
    c01 = torch.randn(B, N, 1, 1, generator=gen) * 0.5
    c11 = torch.randn(B, N, 1, 1, generator=gen) * 0.5 + 1.0
    al = torch.rand(B, N, generator=gen)
    col = torch.rand(B, N, C, generator=gen)
    tgt = torch.rand(B, C, H, W, generator=gen)
    res = {}
    for mode, fn in (("ref", ref.GaussianSplatting2DChunkedKernel.apply), ("exact", ref.naive_gaussian_2d)):
        leaves = [t.clone().requires_grad_() for t in (x, y, pos, c00, c01, c11, al, col)]
        out = fn(*leaves)
        gout = 2 * (out.detach() - tgt)
        ((out - tgt) ** 2).sum().backward()
        res[mode] = (out.detach(), gout, [t.grad for t in leaves])
    names = ("x", "y", "positions", "c00", "c01", "c11", "alphas", "colors")
    arrs = dict(x=x, y=y, positions=pos, c00=c00, c01=c01, c11=c11, alphas=al, colors=col,
                target=tgt, out=res["ref"][0], gout=res["ref"][1], out_dense=res["exact"][0],
                eps=np.float32(1e-6))
    for mode in ("ref", "exact"):
        for k, g in zip(names, res[mode][2]):
            arrs[f"g_{mode}_{k}"] = g
    save(name, **arrs)


def per_gaussian_cross_check(ref):
    """The reference's two torch Functions agree (same formulas); assert it here so the
    fixture set stands for both (src/igs/gs2d.py:47-262 vs :265-465)."""
    gen = torch.Generator().manual_seed(99)
    B, N, H, W, C = 2, 40, 12, 12, 3
    args = [torch.rand(B, 1, H, W, generator=gen), torch.rand(B, 1, H, W, generator=gen),
            torch.rand(B, N, 2, generator=gen), torch.rand(B, N, 1, 1, generator=gen) + 0.5,
            torch.rand(B, N, 1, 1, generator=gen) * 0.2, torch.rand(B, N, 1, 1, generator=gen) + 0.5,
            torch.rand(B, N, generator=gen), torch.rand(B, N, C, generator=gen)]
    outs = []
    for fn in (ref.TorchGaussianSplatting2DKernel, ref.TorchGaussianSplatting2DChunked):
        leaves = [a.clone().requires_grad_() for a in args]
        o = fn.apply(*leaves)
        (o ** 2).sum().backward()
        outs.append([o.detach()] + [t.grad for t in leaves])
    for a, b in zip(*outs):
        assert (a - b).abs().max() <= 2e-5 * b.abs().max().clamp_min(1e-30), "reference Functions disagree"
    print("per-gaussian vs chunked reference Functions: agree")


def module_case(ref, name, seed, n_per, emb, feats, H, W, out_dim=3, B=1):
    """nn.Module entry (src/igs/gs2d.py:479-689) with random-init weights."""
    torch.manual_seed(seed)
    m = ref.GaussianSplatting2D(n_per, emb, out_dim)
    feat = torch.randn(B, feats, emb).requires_grad_()
    tgt = torch.rand(B, out_dim, H, W)
    out, gs_feature = m(feat, size=(H, W))
    loss = torch.nn.functional.mse_loss(out, tgt)
    loss.backward()
    save(name, weight=m.proj.weight, bias=m.proj.bias, feature=feat, target=tgt, out=out,
         gs_feature=gs_feature, loss=loss.detach(), g_weight=m.proj.weight.grad,
         g_bias=m.proj.bias.grad, g_feature=feat.grad,
         n_per=np.int64(n_per), emb=np.int64(emb), H=np.int64(H), W=np.int64(W))


def module_variants_case(ref, name, seed):
    """The module's two optional inputs: a caller-supplied (here warped) sampling grid
    [B,2,H,W] with the row coordinate first (src/igs/gs2d.py:650-653), and
    pos_map_offset=True with a scale factor (:654-667), where every feature's gaussians
    are offset by the grid position of that feature."""
    torch.manual_seed(seed)
    B, n_per, emb, H, W, scale = 2, 4, 32, 32, 32, 8
    feats = (H // scale) * (W // scale)
    tgt = torch.rand(B, 3, H, W)
    xg, yg = ref.GaussianSplatting2D.xy_grid((H, W), "cpu")
    warp = 0.05 * torch.sin(3 * xg) * torch.cos(2 * yg)
    grid = torch.stack([(yg + warp).expand(B, H, W), (xg - warp).expand(B, H, W)], dim=1).contiguous()
    out = {}
    for tag, kwargs, pmo in (("grid", dict(grid=grid), False), ("posmap", dict(size=(H, W), scale=scale), True)):
        m = ref.GaussianSplatting2D(n_per, emb, 3, pos_map_offset=pmo)
        feat = torch.randn(B, feats, emb).requires_grad_()
        img, gs_feature = m(feat, **kwargs)
        loss = torch.nn.functional.mse_loss(img, tgt)
        loss.backward()
        out.update({f"{tag}_weight": m.proj.weight, f"{tag}_bias": m.proj.bias, f"{tag}_feature": feat,
                    f"{tag}_out": img, f"{tag}_g_weight": m.proj.weight.grad, f"{tag}_g_bias": m.proj.bias.grad,
                    f"{tag}_g_feature": feat.grad})
    save(name, target=tgt, grid=grid, n_per=np.int64(n_per), emb=np.int64(emb), H=np.int64(H), W=np.int64(W),
         scale=np.int64(scale), **out)


def koleo_case(name, seed):
    """The diversity regulariser used beside the module (src/igs/reg.py:5-40)."""
    import igs.reg as ref_reg

    gen = torch.Generator().manual_seed(seed)
    f = torch.randn(3, 17, 8, generator=gen, requires_grad=True)
    loss = ref_reg.koleo_diversity_loss(f)
    loss.backward()
    save(name, features=f, loss=loss.detach(), g_features=f.grad)


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py /path/to/reference   (the reference's source tree)")
    ref = load_reference(sys.argv[1])
    torch.set_num_threads(os.cpu_count() or 1)
    per_gaussian_cross_check(ref)
    render_case(ref, "render_small_c3", 11, 2, 70, 20, 28, 3, 0.25, 0.75)
    render_case(ref, "render_narrow_c3", 12, 1, 96, 32, 32, 3, 0.02, 0.2, loss="mse")
    render_case(ref, "render_c1", 13, 1, 33, 16, 16, 1, 0.25, 0.75)
    render_case(ref, "render_c4", 14, 2, 64, 16, 24, 4, 0.1, 0.5)
    render_case(ref, "render_c16", 15, 1, 48, 24, 24, 16, 0.05, 0.3, normal_colors=True)
    render_case(ref, "render_c17", 16, 1, 40, 24, 16, 17, 0.1, 0.5, normal_colors=True)
    render_case(ref, "render_n1", 17, 3, 1, 8, 8, 3, 0.25, 0.75)
    render_case(ref, "render_tall", 18, 1, 130, 48, 12, 3, 0.1, 0.4)
    kernel_case(ref, "kernel_xy_c3", 21, 2, 45, 12, 20, 3)
    module_case(ref, "module_small", 31, 4, 64, 16, 32, 32)
    module_variants_case(ref, "module_variants", 32)
    koleo_case("koleo", 5)
    # benchmark configuration 0 at full size (B=1, N=2048, 256x256, C=3), seed 0
    render_case(ref, "cfg0_full", 0, 1, 2048, 256, 256, 3, 0.25, 0.75, slim=True)


if __name__ == "__main__":
    main()
