"""Per-image fit: free gaussian parameters optimised against one target image.

This is the reference's realistic caller of the function API
(``scripts/2dgs_img_comp.py``: the ``ProgressiveGaussianSplatter`` model :28-126 renders
``GaussianSplatting2D.render(position, color, exp(log_scale)+eps, rotation, ones, grids)``
and an Adam-family optimiser steps the four parameter tensors, :149-252), reduced to what
the splat path needs: MSE loss, Adam, an optional resolution schedule.  Perceptual losses,
image files and video dumps of that script are not part of it.

One fit step is a dozen small launches; for small problems the host cost of issuing them
dominates, so ``fit(..., graph=True)`` captures forward + loss + backward + optimiser step
once in a CUDA graph per resolution and replays it.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .gs2d import GaussianSplatting2D, gaussian_splatting_2d

EPS = 1e-6


class ImageFitter(nn.Module):
    """``num_gaussians`` free gaussians for one image of ``channels`` channels.

    Parameters as in the reference's model (scripts/2dgs_img_comp.py:95-102): ``position``
    [1,N,2] on a regular lattice over the image extent, ``log_scale`` [1,N,2] (constant
    start), ``rotation`` [1,N] (zero) and ``color`` [1,N,C] (sampled from ``image`` when
    given, else 0.5); opacities are fixed to one.
    """

    def __init__(self, num_gaussians, channels=3, image=None, init_log_scale=-3.0, aspect=1.0):
        super().__init__()
        self.num_gaussians = int(num_gaussians)
        if image is not None:
            aspect = image.shape[-2] / image.shape[-1]
            channels = image.shape[1]
        hr, wr = aspect ** 0.5, 1 / aspect ** 0.5  # same extents as xy_grid
        side = max(1, int(math.sqrt(num_gaussians)))
        ys = torch.linspace(-hr, hr, side + 2)[1:-1]
        xs = torch.linspace(-wr, wr, side + 2)[1:-1]
        lattice = torch.stack(torch.meshgrid(xs, ys, indexing="xy"), dim=-1).reshape(-1, 2)
        rest = num_gaussians - lattice.shape[0]
        if rest > 0:  # gaussians beyond the square lattice start at seeded random places
            gen = torch.Generator().manual_seed(0)
            extra = (torch.rand(rest, 2, generator=gen) * 2 - 1) * torch.tensor([wr, hr])
            lattice = torch.cat([lattice, extra], 0)
        if image is not None:
            grid = (lattice / torch.tensor([wr, hr])).view(1, -1, 1, 2).to(image)
            color = F.grid_sample(image, grid, mode="bilinear", align_corners=True)[..., 0].permute(0, 2, 1)
            color = color.detach().cpu().float()
        else:
            color = torch.full((1, num_gaussians, channels), 0.5)
        self.position = nn.Parameter(lattice[None].contiguous())
        self.log_scale = nn.Parameter(torch.full((1, num_gaussians, 2), float(init_log_scale)))
        self.rotation = nn.Parameter(torch.zeros(1, num_gaussians))
        self.color = nn.Parameter(color.contiguous())
        self.register_buffer("alphas", torch.ones(1, num_gaussians))
        self._grids = {}
        # The spatial processing order of the gaussians (narrow gaussians only, see
        # igs_b200.set_backward_sort) is kept for this many fused steps before it is computed
        # again: the gaussians move a little per step, any permutation gives the same gradients,
        # and an eager step is bound by host time that the ordering adds to.
        self.order_every = 8
        self._kept_order = None  # (steps since it was computed, (image size, policy), order or None)

    def grids(self, size):
        """[1,1,H,W] sample coordinates of ``xy_grid`` on the parameters' device, built once
        per size (they are made on the host, which a graph capture cannot do)."""
        key = (int(size[0]), int(size[1]), str(self.position.device))
        if key not in self._grids:
            x_grid, y_grid = GaussianSplatting2D.xy_grid(size, self.position.device)
            self._grids[key] = (x_grid[None], y_grid[None])  # stride-0 views: known separable
        return self._grids[key]

    def forward(self, size):
        x_grid, y_grid = self.grids(size)
        return gaussian_splatting_2d(self.position, self.color, torch.exp(self.log_scale) + EPS, self.rotation,
                                     self.alphas, x_grid, y_grid)

    def mse_loss_and_backward(self, target):
        """mean((render - target)^2) with the gradients of all four parameter tensors written
        to their ``.grad`` (replacing what was there), through ONE library call
        (igs_render_mse_sr): what ``mse_loss(self(size), target).backward()`` computes, without
        the image, the upstream gradient or the weight sums ever going to memory.  Returns the
        loss as a device scalar."""
        from . import gs2d

        x_grid, y_grid = self.grids(target.shape[-2:])
        pos, ls, rot, col = (p.detach() for p in (self.position, self.log_scale, self.rotation, self.color))
        size = (tuple(target.shape[-2:]), _lib._BACKWARD_SORT)  # (an order is only good for one image size and policy)
        kept = self._kept_order
        if (kept is not None and kept[1] == size and kept[0] < self.order_every
                and not torch.cuda.is_current_stream_capturing()):
            # (a captured graph computes the order in every replay: that costs no host time)
            info = _lib.prepare_call(x_grid, y_grid, pos, order=(_lib.KEEP_ORDER, kept[2]))
            self._kept_order = (kept[0] + 1, size, kept[2])
        else:
            info = _lib.prepare_call(x_grid, y_grid, pos, scales=ls, log_scales=True, rotations=rot)
            # (only an actual order is kept: while the policy wants none, asking again costs nothing)
            self._kept_order = (1, size, info.order) if info.order is not None else None
        loss, g, _ = _lib.render_mse(pos, ls, rot, None, col, info.x3, info.y3, target, EPS,
                                     gs2d._GRAD_MODES[gs2d.get_grad_mode()], log_scales=True, order=info.order,
                                     hints=info.hints, info=info)
        self.position.grad, self.log_scale.grad = g["positions"], g["scales"]
        self.rotation.grad, self.color.grad = g["rotations"], g["colors"]
        return loss


class ShardedImageFitter(ImageFitter):
    """An ``ImageFitter`` whose gaussians are spread over the ranks of a process group: the
    one-image case on several GPUs (one process per GPU).

    Every rank builds the same initial gaussians and keeps the contiguous range
    ``igs_b200.dist.gaussian_range`` gives it; ``forward`` renders through
    ``sharded_gaussian_splatting_2d`` (one all-reduce of the [1,C+1,H,W] sums, every rank gets
    the whole image), the loss is computed from the whole image on every rank, and backward
    and the optimiser touch the rank's own gaussians only: no gradient or parameter ever
    crosses ranks.  ``gathered()`` collects the parameters of all ranks, e.g. for saving.
    ``backend``: the three device calls (default: the CUDA library).
    """

    def __init__(self, num_gaussians, channels=3, image=None, init_log_scale=-3.0, aspect=1.0, group=None,
                 backend=None):
        import torch.distributed as tdist

        from .dist import gaussian_range

        super().__init__(num_gaussians, channels, image, init_log_scale, aspect)
        if not tdist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised (launch with torchrun)")
        self.group, self.backend = group, backend
        lo, hi = gaussian_range(self.num_gaussians, tdist.get_world_size(group), tdist.get_rank(group))
        self.range = (lo, hi)
        for name in ("position", "log_scale", "rotation", "color"):
            setattr(self, name, nn.Parameter(getattr(self, name).detach()[:, lo:hi].clone()))
        self.alphas = self.alphas[:, lo:hi].clone()

    def forward(self, size):
        from .dist import sharded_gaussian_splatting_2d

        x_grid, y_grid = self.grids(size)
        return sharded_gaussian_splatting_2d(self.position, self.color, torch.exp(self.log_scale) + EPS,
                                             self.rotation, self.alphas, x_grid, y_grid, group=self.group,
                                             backend=self.backend)

    def mse_loss_and_backward(self, target):
        raise NotImplementedError("the one-call step renders all gaussians on one GPU; the sharded fitter "
                                  "goes through forward() and autograd")

    @torch.no_grad()
    def gathered(self):
        """{name: [1,N,...]} of position, log_scale, rotation and color over all ranks (a
        collective: every rank must call it)."""
        import torch.distributed as tdist

        from .dist import gaussian_range

        world = tdist.get_world_size(self.group)
        ranges = [gaussian_range(self.num_gaussians, world, r) for r in range(world)]
        longest = max(hi - lo for lo, hi in ranges)
        res = {}
        for name in ("position", "log_scale", "rotation", "color"):
            mine = getattr(self, name).detach()
            padded = mine.new_zeros((1, longest) + tuple(mine.shape[2:]))  # ranges differ by at most one
            padded[:, : mine.shape[1]] = mine
            parts = [torch.empty_like(padded) for _ in range(world)]
            tdist.all_gather(parts, padded, group=self.group)
            res[name] = torch.cat([part[:, : hi - lo] for part, (lo, hi) in zip(parts, ranges)], 1)
        return res


class _MSELoss(torch.autograd.Function):
    """F.mse_loss(out, target) for contiguous fp32 CUDA tensors through the library's two
    loss kernels (three launches forward + backward where the torch ops take about eight)."""

    @staticmethod
    def forward(ctx, out, target):
        ctx.save_for_backward(out, target)
        return _lib.mse_loss(out, target)

    @staticmethod
    def backward(ctx, grad_loss):
        out, target = ctx.saved_tensors
        return _lib.mse_grad(out, target, grad_loss.contiguous().float()), None


def mse_loss(out, target):
    """Mean squared error; the library's kernels when both tensors are contiguous fp32 CUDA
    tensors of one shape and only ``out`` needs a gradient, torch's otherwise."""
    if (out.is_cuda and target.is_cuda and out.dtype == target.dtype == torch.float32 and out.shape == target.shape
            and out.is_contiguous() and target.is_contiguous() and not target.requires_grad and out.numel() > 0):
        return _MSELoss.apply(out, target)
    return F.mse_loss(out, target)


def _fusable(model, target):
    return (type(model) is ImageFitter and target.is_cuda and target.dtype == torch.float32
            and target.is_contiguous() and target.dim() == 4 and target.shape[0] == 1
            and target.shape[1] == model.color.shape[-1])


def _eager_step(model, opt, target, fused=True):
    """One optimiser step on mean((render - target)^2).  fused: render, loss and gradients in
    one library call where the model and the target allow it (same numbers as the autograd
    route to fp32 rounding)."""
    if fused and _fusable(model, target):
        loss = model.mse_loss_and_backward(target)
        opt.step()
        return loss
    opt.zero_grad(set_to_none=False)
    loss = mse_loss(model(target.shape[-2:]), target)
    loss.backward()
    opt.step()
    return loss.detach()


class GraphedStep:
    """forward + MSE + backward + optimiser step captured once, replayed per call.

    Capture must come after at least one eager step at the same size, so that everything
    built lazily exists (optimizer moments, the grids, the library's kernel attributes).
    The target lives in a static buffer (``set_target`` copies into it); the returned loss
    tensor is overwritten by every replay.
    """

    def __init__(self, model, opt, target):
        self.model, self.opt = model, opt
        self.target = target.clone()
        model.grids(target.shape[-2:])
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.loss = _eager_step(model, opt, self.target)

    def set_target(self, target):
        self.target.copy_(target)

    def __call__(self):
        self.graph.replay()
        return self.loss


GRAPH_MIN_STEPS = 64  # capturing costs ~0.16 s; below this many steps at one size it does not pay


def fit(model, target, steps, lr=1e-2, graph=True, schedule=None, betas=(0.9, 0.999), grad_mode=None):
    """Optimises ``model`` against ``target`` [1,C,H,W] for ``steps`` Adam steps.

    ``graph``: replay a captured CUDA graph per step (sizes with fewer than
    ``GRAPH_MIN_STEPS`` steps run eagerly).  Measured on B200 at N=2048, 256x256: 0.15 ms
    per Adam step replayed against 0.18 ms issued from Python (one library call and a
    single-kernel Adam per step leave a graph little to save; at 16384 gaussians and
    1024x1024 both take the device's 0.33 ms).
    ``grad_mode``: "reference" / "exact" (see igs_b200.gs2d); None keeps the current one.

    ``schedule``: optional list of (scale, steps) pairs, e.g. [(4, 300), (2, 200), (1, 100)]:
    the target is area-averaged down by ``scale`` for that many steps (the reference
    trains 256 -> 512 -> 1024 px, scripts/2dgs_img_comp.py:152-155).  Returns the loss of
    every step as a CPU tensor (one synchronisation, at the end).
    """
    if not target.is_cuda:
        raise RuntimeError("fit() runs on CUDA tensors only")
    if grad_mode is not None:
        from . import gs2d

        with gs2d.grad_mode(grad_mode):
            return fit(model, target, steps, lr, graph, schedule, betas, None)
    if isinstance(model, ShardedImageFitter):
        graph = False  # (a step holds a collective: issued eagerly, never captured)
    schedule = schedule or [(1, steps)]
    # (torch's single-kernel Adam: the default one issues a dozen small launches per step, which
    # a host-bound eager step pays for in full)
    opt = torch.optim.Adam(model.parameters(), lr=lr, betas=betas, capturable=bool(graph), fused=True)
    for p in model.parameters():  # Adam must see gradients from the first (captured) step on
        p.grad = torch.zeros_like(p)
    history = torch.zeros(sum(n for _, n in schedule), device=target.device)
    i = 0
    for scale, n in schedule:
        tgt = target if scale == 1 else F.avg_pool2d(target, scale)
        stepper = None
        for k in range(n):
            if graph and k == 2 and n >= GRAPH_MIN_STEPS:
                stepper = GraphedStep(model, opt, tgt)  # the first steps of a size run eagerly
            loss = stepper() if stepper is not None else _eager_step(model, opt, tgt)
            history[i].copy_(loss)
            i += 1
    return history.cpu()


# ---------------------------------------------------------------------------
# feature -> image experiment with a random number of active features per step
# ---------------------------------------------------------------------------
class ProgressiveSplatter(nn.Module):
    """Learned feature vectors rendered through the module, coarse to fine: the image of the
    first k features must already resemble the target (the reference's
    ``ProgressiveGaussianSplatter``, scripts/gs2d_test.py:28-51)."""

    def __init__(self, num_features, feature_dim, gaussians_per_feature, channels=3):
        super().__init__()
        self.num_features = int(num_features)
        self.feature = nn.Parameter(torch.randn(1, num_features, feature_dim))
        self.gs = GaussianSplatting2D(gaussians_per_feature, feature_dim, channels)

    def forward(self, num_active_features=None, size=None):
        k = self.num_features if num_active_features is None else min(int(num_active_features), self.num_features)
        return self.gs(self.feature[:, :k], size)


def fit_progressive(model, target, steps, lr=1e-4, chunk=4, ratios=(1 / 16, 1 / 8, 1 / 4, 1 / 2, 1.0),
                    reg_weight=0.01, clip=0.1, seed=0):
    """The training loop of the reference's feature -> image experiment
    (scripts/gs2d_test.py:154-189): every step draws a fraction of the features, renders
    only those, and steps AdamW on ``reconstruction + reg_weight * koleo(features[:k])``
    with the gradient norm clipped to ``clip``.  The reconstruction term is L1 + 0.5 MSE
    (:53-60 without its MS-SSIM term, whose package is not available here).  Returns
    (losses [steps], the k of every step) on the CPU."""
    from .reg import koleo_diversity_loss

    if not target.is_cuda:
        raise RuntimeError("fit_progressive() runs on CUDA tensors only")
    gen = torch.Generator().manual_seed(seed)
    opt = torch.optim.AdamW(model.parameters(), lr=lr, eps=EPS, fused=True)
    size = target.shape[-2:]
    n = model.num_features
    history = torch.zeros(steps, device=target.device)
    ks = []
    for i in range(steps):
        ratio = ratios[int(torch.randint(len(ratios), (1,), generator=gen))]
        k = int(round(ratio * n / chunk) * chunk)
        k = max(chunk, min(n, k))
        ks.append(k)
        out, _ = model(num_active_features=k, size=size)
        recon = F.l1_loss(out, target) + 0.5 * mse_loss(out, target)
        loss = recon + reg_weight * koleo_diversity_loss(model.feature[:, :k])
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        opt.step()
        history[i].copy_(loss.detach())
    return history.cpu(), ks
