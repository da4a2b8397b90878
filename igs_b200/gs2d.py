"""Drop-in for ``igs.gs2d`` (KohakuBlueleaf/IGS, src/igs/gs2d.py) on B200.

Same public names, arguments and shapes as the reference module:

* ``GaussianSplatting2D`` -- the nn.Module (reference :479-689) with
  ``forward``, ``xy_grid`` and ``render``;
* ``gaussian_splatting_2d`` -- alias of ``GaussianSplatting2D.render`` (:692);
* ``GaussianSplatting2DKernel`` -- the autograd Function taking inverse-covariance
  entries (:47-262 / :265-465), with ``.apply(x, y, position, cov_inv_00, cov_inv_01,
  cov_inv_11, alphas, colors, eps)``;
* ``naive_gaussian_2d``, ``log_vram`` and the ``Torch*`` / ``*Chunked*`` aliases that
  the reference module exports.

Underneath there is one implementation: hand-written sm_100a CUDA kernels reached
through the C ABI of ``libigs_b200.so``.  There is no Triton, no back-end selection
(reference :7-14, :468-476) and no CPU path: tensors must be fp32 on a CUDA device.

Gradient semantics.  The reference's hand-written backward uses
``gS = -sum_c g_c^2 / S^2`` for the per-pixel normalisation term (:370), which is not
the derivative of its own forward.  That is the default here too (parity with the
reference); ``set_grad_mode("exact")`` switches to the true derivative
(``gS = -sum_c (g_c/S) out_c``, what autograd of ``naive_gaussian_2d`` gives).
"""
from __future__ import annotations

import contextlib
import functools

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd.function import once_differentiable

from . import _lib

__all__ = [
    "GaussianSplatting2D", "gaussian_splatting_2d", "GaussianSplatting2DKernel",
    "GaussianSplatting2DChunkedKernel", "TorchGaussianSplatting2DKernel", "TorchGaussianSplatting2DChunked",
    "naive_gaussian_2d", "log_vram", "set_grad_mode", "get_grad_mode", "grad_mode",
]

_GRAD_MODES = {"reference": _lib.GRAD_REFERENCE, "exact": _lib.GRAD_EXACT}
_grad_mode = "reference"


def set_grad_mode(mode: str) -> None:
    """'reference' (default, matches the reference's backward) or 'exact'."""
    global _grad_mode
    if mode not in _GRAD_MODES:
        raise ValueError(f"grad mode must be one of {sorted(_GRAD_MODES)}, got {mode!r}")
    _grad_mode = mode


def get_grad_mode() -> str:
    return _grad_mode


@contextlib.contextmanager
def grad_mode(mode: str):
    prev = get_grad_mode()
    set_grad_mode(mode)
    try:
        yield
    finally:
        set_grad_mode(prev)


def log_vram(prefix=""):
    """No-op hook kept for import compatibility (reference :20-21)."""
    return


def naive_gaussian_2d(x, y, position, cov_inv_00, cov_inv_01, cov_inv_11, alphas, colors, eps=1e-6):
    """Dense debugging path (reference :24-44): materialises the [B,N,H,W] weights with
    plain torch ops on whatever device the tensors live on; differentiable by autograd.
    Only ``render(..., fused=False)`` reaches it."""
    dx = x - position[..., 0, None, None]
    dy = y - position[..., 1, None, None]
    quad = dx * dx * cov_inv_00 + 2 * dx * dy * cov_inv_01 + dy * dy * cov_inv_11
    weight = torch.exp(-0.5 * quad) * alphas[..., None, None]
    norm = weight / (weight.sum(dim=1, keepdim=True) + eps)
    return torch.einsum("bnhw,bnc->bchw", norm, colors)


# ---------------------------------------------------------------------------
# argument checking shared by the two Functions
# ---------------------------------------------------------------------------
def _require_cuda_f32(name, t):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} is on {t.device}: igs_b200 runs on CUDA devices only (no CPU path)")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32 (the reference computes in fp32), got {t.dtype}")


def _save_call(ctx, info, x, y, *tensors):
    """Saves a forward's tensors plus what the call decided (grid views' kind, hints,
    processing order) so that the backward runs the same kernels on the same views."""
    ctx.save_for_backward(x, y, *tensors, info.order if info.order is not None else x.new_empty(0))
    ctx.has_order = info.order is not None
    ctx.hints = info.hints
    ctx.grid_views = (info.x3, info.y3)  # views of the saved x, y (whose versions autograd checks)
    info.x3 = info.y3 = info.order = None  # only the memos stay on the info object
    ctx.call_info = info


def _saved_call(ctx):
    """-> (the saved tensors without the order, x3, y3, order or None)."""
    *tensors, order = ctx.saved_tensors
    x3, y3 = ctx.grid_views
    return tensors, x3, y3, (order if ctx.has_order else None)


def _check_gaussians(position, alphas, colors):
    if position.dim() != 3 or position.shape[-1] != 2:
        raise ValueError(f"positions must be [B,N,2], got {tuple(position.shape)}")
    B, N, _ = position.shape
    if colors.dim() != 3 or colors.shape[:2] != (B, N) or colors.shape[2] < 1:
        raise ValueError(f"colors must be [B,N,C] with B={B}, N={N}; got {tuple(colors.shape)}")
    if alphas.shape != (B, N):
        raise ValueError(f"alphas must be [B,N] = {(B, N)}, got {tuple(alphas.shape)}")
    return B, N, colors.shape[2]


def _same_device(*ts):
    dev = ts[0].device
    for t in ts:
        if t.device != dev:
            raise RuntimeError(f"all tensors must be on one device; got {dev} and {t.device}")
    return dev


def _reduce_like(g, ref_shape):
    """Sums a [B,...] gradient down to a broadcast input's batch of 1."""
    if ref_shape[0] == 1 and g.shape[0] != 1:
        g = g.sum(dim=0, keepdim=True)
    return g.reshape(ref_shape)


# ---------------------------------------------------------------------------
# autograd Functions
# ---------------------------------------------------------------------------
class GaussianSplatting2DKernel(torch.autograd.Function):
    """Fused splat from inverse-covariance entries (reference :47-262, :265-465).

    x, y: [B,1,H,W]; position [B,N,2]; cov_inv_00/01/11 [B,N,1,1] (anything that
    reshapes to [B,N]); alphas [B,N]; colors [B,N,C]  ->  [B,C,H,W].
    backward returns the reference's nine values (:455-465); the upstream gradient
    and the saved weight sum are left untouched (the reference mutates both, :369-371).
    """

    @staticmethod
    def forward(ctx, x, y, position, cov_inv_00, cov_inv_01, cov_inv_11, alphas, colors, eps=1e-6):
        names = ("x", "y", "position", "cov_inv_00", "cov_inv_01", "cov_inv_11", "alphas", "colors")
        tensors = (x, y, position, cov_inv_00, cov_inv_01, cov_inv_11, alphas, colors)
        for n, t in zip(names, tensors):
            _require_cuda_f32(n, t)
        _same_device(*tensors)
        B, N, C = _check_gaussians(position, alphas, colors)
        cov = []
        for n, t in zip(names[3:6], tensors[3:6]):
            if t.numel() != B * N:
                raise ValueError(f"{n} must hold B*N = {B * N} values, got shape {tuple(t.shape)}")
            cov.append(t.reshape(B, N).contiguous())
        pos, al, col = position.contiguous(), alphas.contiguous(), colors.contiguous()
        info = _lib.prepare_call(x, y, pos)
        out, wsum = _lib.forward("cov", pos, cov[0], cov[1], cov[2], al, col, info.x3, info.y3, eps,
                                 order=info.order, hints=info.hints, info=info)
        _save_call(ctx, info, x, y, pos, cov[0], cov[1], cov[2], al, col, wsum, out)
        ctx.eps = float(eps)
        ctx.grad_mode = _GRAD_MODES[_grad_mode]
        ctx.cov_shapes = tuple(t.shape for t in tensors[3:6])
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_result):
        (x, y, pos, c00, c01, c11, al, col, wsum, out), x3, y3, order = _saved_call(ctx)
        want_xy = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        g = _lib.backward("cov", pos, c00, c01, c11, al, col, x3, y3, wsum, out, grad_result.contiguous(),
                          ctx.eps, ctx.grad_mode, want_xy, order=order, hints=ctx.hints, info=ctx.call_info)
        gx = _reduce_like(g["x"][:, None], x.shape) if want_xy else None
        gy = _reduce_like(g["y"][:, None], y.shape) if want_xy else None
        s00, s01, s11 = ctx.cov_shapes
        return (gx, gy, g["positions"], g["c00"].reshape(s00), g["c01"].reshape(s01), g["c11"].reshape(s11),
                g["alphas"], g["colors"], None)


class _SplatFromScaleRotation(torch.autograd.Function):
    """What ``render`` runs: scales/rotations -> inverse covariance (reference :549-580)
    fused in front of the splat, and its closed-form derivative fused behind the
    backward, so autograd never sees the 2x2 matrix algebra."""

    @staticmethod
    def forward(ctx, positions, colors, scales, rotations, alphas, x, y, eps):
        names = ("positions", "colors", "scales", "rotations", "alphas", "x_grid", "y_grid")
        tensors = (positions, colors, scales, rotations, alphas, x, y)
        for n, t in zip(names, tensors):
            _require_cuda_f32(n, t)
        _same_device(*tensors)
        B, N, C = _check_gaussians(positions, alphas, colors)
        if scales.shape != (B, N, 2):
            raise ValueError(f"scales must be [B,N,2] = {(B, N, 2)}, got {tuple(scales.shape)}")
        if rotations.shape != (B, N):
            raise ValueError(f"rotations must be [B,N] = {(B, N)}, got {tuple(rotations.shape)}")
        pos, col, sc, rot, al = (t.contiguous() for t in (positions, colors, scales, rotations, alphas))
        # grid views, hints and one spatial order per step (if the policy wants one), shared by
        # forward and backward
        info = _lib.prepare_call(x, y, pos, scales=sc, rotations=rot)
        out, wsum = _lib.forward("sr", pos, sc, rot, None, al, col, info.x3, info.y3, eps, order=info.order,
                                 hints=info.hints, info=info)
        _save_call(ctx, info, x, y, pos, col, sc, rot, al, wsum, out)
        ctx.eps = float(eps)
        ctx.grad_mode = _GRAD_MODES[_grad_mode]
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_result):
        (x, y, pos, col, sc, rot, al, wsum, out), x3, y3, order = _saved_call(ctx)
        want_xy = ctx.needs_input_grad[5] or ctx.needs_input_grad[6]
        g = _lib.backward("sr", pos, sc, rot, None, al, col, x3, y3, wsum, out, grad_result.contiguous(), ctx.eps,
                          ctx.grad_mode, want_xy, order=order, hints=ctx.hints, info=ctx.call_info)
        gx = _reduce_like(g["x"][:, None], x.shape) if want_xy else None
        gy = _reduce_like(g["y"][:, None], y.shape) if want_xy else None
        return g["positions"], g["colors"], g["scales"], g["rotations"], g["alphas"], gx, gy, None


class _SplatFromFeature(torch.autograd.Function):
    """What the module runs: the splat fed by the projection output itself.  The split into
    position / log-scale / rotation / colour, ``exp(log_scale) + eps``, the all-ones
    opacities and the optional position offset (reference :637-673) happen inside the
    prologue kernel, and the backward writes the gradient of the whole [B,N,6+C] tensor, so
    autograd sees one node instead of a dozen small ones."""

    @staticmethod
    def forward(ctx, gs_feature, pos_offset, x, y, eps):
        _require_cuda_f32("gs_feature", gs_feature)
        _require_cuda_f32("x_grid", x)
        _require_cuda_f32("y_grid", y)
        _same_device(gs_feature, x, y)
        if gs_feature.dim() != 3 or gs_feature.shape[-1] < 7:
            raise ValueError(f"gs_feature must be [B,N,6+C], got {tuple(gs_feature.shape)}")
        B, N, _ = gs_feature.shape
        feat = gs_feature.contiguous()
        off = None
        if pos_offset is not None:
            _require_cuda_f32("pos_map", pos_offset)
            if pos_offset.shape != (B, N, 2):
                raise ValueError(f"the position offsets must be [B,N,2] = {(B, N, 2)}, got {tuple(pos_offset.shape)}")
            off = pos_offset.contiguous()
        info = _lib.prepare_call(x, y, None, feat, off)
        out, wsum = _lib.forward_feature(feat, off, info.x3, info.y3, eps, order=info.order, hints=info.hints,
                                         info=info)
        _save_call(ctx, info, x, y, feat, off if off is not None else feat.new_empty(0), wsum, out)
        ctx.has_off = off is not None
        ctx.eps = float(eps)
        ctx.grad_mode = _GRAD_MODES[_grad_mode]
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_result):
        (x, y, feat, off, wsum, out), x3, y3, order = _saved_call(ctx)
        d_feat = _lib.backward_feature(feat, off if ctx.has_off else None, x3, y3, wsum, out,
                                       grad_result.contiguous(), ctx.eps, ctx.grad_mode, order=order, hints=ctx.hints,
                                       info=ctx.call_info)
        d_off = d_feat[..., :2] if (ctx.has_off and ctx.needs_input_grad[1]) else None
        return d_feat, d_off, None, None, None


# names the reference module also exports (:265, :468-469); one implementation here
GaussianSplatting2DChunkedKernel = GaussianSplatting2DKernel
TorchGaussianSplatting2DKernel = GaussianSplatting2DKernel
TorchGaussianSplatting2DChunked = GaussianSplatting2DKernel


# ---------------------------------------------------------------------------
# nn.Module
# ---------------------------------------------------------------------------
class GaussianSplatting2D(nn.Module):
    """Feature vectors -> gaussian parameters -> image (reference :479-689).

    ``proj`` maps each of the F feature vectors to ``num_gaussians_per_emb`` gaussians of
    ``6 + output_dim`` numbers: position (2), log-scale (2), rotation (1), opacity
    logit (1, unused: alphas are fixed to 1, reference :673) and colour.
    """

    def __init__(self, num_gaussians_per_emb, emb_dim, output_dim=3, pos_map_offset=False):
        super().__init__()
        self.num_gaussians_per_emb = num_gaussians_per_emb
        self.emb_dim = emb_dim
        self.chunk_size = 0
        self.output_dim = output_dim
        self.pos_map_offset = pos_map_offset

        per = 6 + output_dim
        self.proj = nn.Linear(emb_dim, num_gaussians_per_emb * per)
        nn.init.normal_(self.proj.weight, mean=0.0, std=0.01)
        # reference :498-501: small random bias, zero position offset, log-scale -4
        bias = torch.randn(num_gaussians_per_emb, per) * 0.01
        bias[:, :2] = 0
        bias[:, 2:4] = -4
        with torch.no_grad():
            self.proj.bias.copy_(bias.view_as(self.proj.bias))

    @staticmethod
    def xy_grid(size=None, device=None):
        """Pixel-centre coordinates (reference :503-522): endpoints inclusive, the longer
        side spans more than [-1,1] so that x_range * y_range = 1.  Returns two [1,H,W]
        tensors that are expanded (stride-0) views of one row / one column ON the target
        device: same values as the reference's, no H*W copy, and the splat kernels can see
        from the strides alone that the grid is separable.  The row and the column are kept
        and shared by every call with the same size and device: treat the returned views as
        read-only (clone them before an in-place change)."""
        h, w = size
        aspect = h / w
        h_range = aspect ** 0.5
        w_range = 1 / aspect ** 0.5
        dev = torch.device(device or "cpu")
        if dev.type == "cuda" and dev.index is None:  # "cuda" means the current device, whichever that is now
            dev = torch.device("cuda", torch.cuda.current_device())
        xs, ys = _grid_axes(int(h), int(w), float(w_range), float(h_range), str(dev))
        return xs.view(1, 1, w).expand(1, h, w), ys.view(1, h, 1).expand(1, h, w)

    @staticmethod
    def render(positions, colors, scales, rotations, alphas, x_grid, y_grid, eps=1e-6, fused=True):
        """positions [B,N,2], colors [B,N,C], scales [B,N,2], rotations [B,N], alphas
        [B,N], x_grid / y_grid [B,1,H,W]  ->  [B,C,H,W]   (reference :524-609).

        ``fused=False`` is the reference's dense debugging path (:598-609): torch ops,
        O(B*N*H*W) memory, gradients by autograd."""
        if fused:
            return _SplatFromScaleRotation.apply(positions, colors, scales, rotations, alphas, x_grid, y_grid, eps)
        c00, c01, c11 = _cov_inv_torch(scales, rotations, eps)
        return naive_gaussian_2d(x_grid, y_grid, positions, c00, c01, c11, alphas, colors, eps)

    def forward(self, feature, size=None, grid=None, pos_map=None, eps=1e-6, fused=True, scale=None):
        """feature [B,F,D] -> (image [B,C,H,W], gs_feature [B, F*n, 6+C])  (reference :611-689)."""
        per = 6 + self.output_dim
        gs_feature = self.proj(feature).unflatten(-1, (-1, per)).flatten(1, 2)
        b = gs_feature.shape[0]

        if grid is None:
            x_grid, y_grid = _batched_grid(int(size[0]), int(size[1]), str(feature.device), b)  # [B,1,H,W], stride 0
        else:
            # [B,2,H,W] with the row coordinate first (reference :651-653)
            y_grid, x_grid = grid.split([1, 1], dim=1)
        if self.pos_map_offset:
            pos_map = torch.cat([x_grid, y_grid], dim=1)
            if scale is not None:
                pos_map = F.interpolate(pos_map, scale_factor=1 / scale, mode="bilinear", align_corners=True)
            pos_map = pos_map.flatten(2, 3).transpose(1, 2)
            assert pos_map.size(1) == feature.size(1)
            pos_map = pos_map[..., None, :].repeat(1, 1, self.num_gaussians_per_emb, 1).flatten(1, 2)

        if fused and not (x_grid.requires_grad or y_grid.requires_grad):
            # the kernels read the projection output in place (same arithmetic as below)
            offset = pos_map if self.pos_map_offset else None
            return _SplatFromFeature.apply(gs_feature, offset, x_grid, y_grid, eps), gs_feature

        positions, log_scales, rotations, logit_opacity, colors = gs_feature.split(
            [2, 2, 1, 1, self.output_dim], dim=-1)
        if self.pos_map_offset:
            positions = positions + pos_map
        alphas = torch.ones_like(logit_opacity[..., 0])
        scales = torch.exp(log_scales) + eps
        rotations = rotations[..., 0]
        output = self.render(positions, colors, scales, rotations, alphas, x_grid, y_grid, eps, fused)
        return output, gs_feature


@functools.lru_cache(maxsize=64)
def _batched_grid(h, w, device, b):
    """xy_grid(size) as the [B,1,H,W] stride-0 views the module's forward hands to the splat;
    kept per (size, device, batch), so a training loop builds them once."""
    x_grid, y_grid = GaussianSplatting2D.xy_grid((h, w), device)
    return x_grid[None].expand(b, -1, -1, -1), y_grid[None].expand(b, -1, -1, -1)


@functools.lru_cache(maxsize=64)
def _grid_axes(h, w, w_range, h_range, device):
    """The W column and H row coordinates on ``device``; computed on the host like the
    reference does (same bits) and kept, so that repeated calls -- in particular calls
    inside a CUDA-graph capture -- copy nothing."""
    xs = torch.linspace(-w_range, w_range, w).to(device)
    ys = torch.linspace(-h_range, h_range, h).to(device)
    return xs, ys


def _cov_inv_torch(scales, rotations, eps):
    """Inverse covariance entries [B,N,1,1] with torch ops, for the dense debug path only."""
    c, s = torch.cos(rotations), torch.sin(rotations)
    p, q = scales[..., 0] ** 2, scales[..., 1] ** 2
    a = c * c * p + s * s * q + eps
    b = c * s * (p - q)
    d = s * s * p + c * c * q + eps
    det = a * d - b * b
    return (d / det)[..., None, None], (-b / det)[..., None, None], (a / det)[..., None, None]


gaussian_splatting_2d = GaussianSplatting2D.render
