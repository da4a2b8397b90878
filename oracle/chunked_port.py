"""torch restatement of the reference's CHUNKED CPU path, used as the timed CPU baseline.

TEST / MEASUREMENT INFRASTRUCTURE ONLY: imported by ``tests/`` and by the CPU-baseline
legs of ``bench.py``; never by the product package.

The reference's CPU implementation is a sequence of torch elementwise passes over
``[B, 32, H, W]`` blocks (src/igs/gs2d.py:265-465, ``N_CHUNK_SIZE = 32`` at :273) behind a
small batch of 2x2 matrix operations (:549-580).  The C oracle (splat_oracle.c) computes
the same numbers with one fused loop, which is a different cost structure; to report
what the reference's own path costs on the host cores, this module keeps the
reference's structure: gaussians in chunks of 32, one torch op per term, einsum for
the colour contraction, ``torch.inverse`` for the covariance.  It is pinned to the
reference's outputs by tests/test_oracle_golden.py.
"""
from __future__ import annotations

import torch

CHUNK = 32  # src/igs/gs2d.py:273


def cov_inv(scales, rotations, eps):
    """[B,N,2], [B,N] -> three [B,N,1,1] tensors; differentiable (src/igs/gs2d.py:549-580)."""
    B, N, _ = scales.shape
    c, s = torch.cos(rotations), torch.sin(rotations)
    R = torch.stack((torch.stack((c, -s), -1), torch.stack((s, c), -1)), -2)  # [B,N,2,2]
    S = torch.diag_embed(scales)                                              # [B,N,2,2]
    RS = torch.bmm(R.reshape(-1, 2, 2), S.reshape(-1, 2, 2))
    cov = torch.bmm(RS, RS.transpose(1, 2)).reshape(B, N, 2, 2)
    inv = torch.inverse(cov + eps * torch.eye(2, dtype=cov.dtype))
    return inv[..., 0, 0, None, None], inv[..., 0, 1, None, None], inv[..., 1, 1, None, None]


def _weights(x, y, pos, c00, c01, c11, lo, hi):
    dx = x - pos[:, lo:hi, 0, None, None]
    dy = y - pos[:, lo:hi, 1, None, None]
    dist = c00[:, lo:hi] * dx ** 2 + c11[:, lo:hi] * dy ** 2 + c01[:, lo:hi] * (2 * dx * dy)
    return dx, dy, torch.exp(-0.5 * dist)


@torch.no_grad()
def forward(x, y, pos, c00, c01, c11, alphas, colors, eps=1e-6):
    """x, y [B,1,H,W] -> (out [B,C,H,W], wsum [B,H,W] without eps)  (src/igs/gs2d.py:288-337)."""
    B, _, H, W = x.shape
    N, C = colors.shape[1:]
    num = x.new_zeros(B, C, H, W)
    wsum = x.new_zeros(B, H, W)
    for lo in range(0, N, CHUNK):
        hi = min(lo + CHUNK, N)
        _, _, e = _weights(x, y, pos, c00, c01, c11, lo, hi)
        w = e * alphas[:, lo:hi, None, None]
        num += torch.einsum("bnhw,bnc->bchw", w, colors[:, lo:hi])
        wsum += w.sum(1)
    return num / (wsum + eps)[:, None], wsum


@torch.no_grad()
def backward(x, y, pos, c00, c01, c11, alphas, colors, wsum, gout, eps=1e-6):
    """Reference-mode backward (src/igs/gs2d.py:353-465); inputs are not modified."""
    B, _, H, W = x.shape
    N, C = colors.shape[1:]
    S = wsum + eps
    gS = -(gout * gout).sum(1) / S ** 2                      # :370
    gn = gout / S[:, None]                                   # :371
    gx, gy = torch.zeros_like(x), torch.zeros_like(y)
    gpos = torch.zeros_like(pos)
    g00, g01, g11 = (torch.zeros_like(t) for t in (c00, c01, c11))
    gal, gcol = torch.zeros_like(alphas), torch.zeros_like(colors)
    for lo in range(0, N, CHUNK):
        hi = min(lo + CHUNK, N)
        dx, dy, e = _weights(x, y, pos, c00, c01, c11, lo, hi)
        w = e * alphas[:, lo:hi, None, None]
        A = torch.einsum("bchw,bnc->bnhw", gn, colors[:, lo:hi])                 # :376-378
        gcol[:, lo:hi] = (gn[:, None] * w[:, :, None]).sum((3, 4))                # :406-408
        G = A + gS[:, None]                                                       # :411-413
        gal[:, lo:hi] = (G * e).sum((2, 3))                                       # :417-419
        cf = G * w * -0.5                                                         # :422
        gdx = cf * (2 * c00[:, lo:hi] * dx + 2 * c01[:, lo:hi] * dy)              # :425-427
        gdy = cf * (2 * c11[:, lo:hi] * dy + 2 * c01[:, lo:hi] * dx)              # :428-430
        gx += gdx.sum(1, keepdim=True)                                            # :433-434
        gy += gdy.sum(1, keepdim=True)
        gpos[:, lo:hi, 0] = -gdx.sum((2, 3))                                      # :437-442
        gpos[:, lo:hi, 1] = -gdy.sum((2, 3))
        g00[:, lo:hi] = (cf * dx ** 2).sum((2, 3), keepdim=True)                  # :445-453
        g11[:, lo:hi] = (cf * dy ** 2).sum((2, 3), keepdim=True)
        g01[:, lo:hi] = (cf * (2 * dx * dy)).sum((2, 3), keepdim=True)
    return {"x": gx, "y": gy, "positions": gpos, "c00": g00, "c01": g01, "c11": g11, "alphas": gal,
            "colors": gcol}


def render_fwd_bwd(positions, colors, scales, rotations, alphas, x, y, gout_fn, eps=1e-6):
    """Full ``gaussian_splatting_2d`` forward + backward on CPU tensors.

    Returns (out, grads) with grads for positions, colors, scales, rotations, alphas --
    the same work one training step of the reference does on its torch path."""
    sc = scales.detach().clone().requires_grad_()
    rt = rotations.detach().clone().requires_grad_()
    c00, c01, c11 = cov_inv(sc, rt, eps)
    d = [t.detach() for t in (c00, c01, c11)]
    out, wsum = forward(x, y, positions, *d, alphas, colors, eps)
    g = backward(x, y, positions, *d, alphas, colors, wsum, gout_fn(out), eps)
    torch.autograd.backward([c00, c01, c11], [g["c00"], g["c01"], g["c11"]])
    return out, {"positions": g["positions"], "colors": g["colors"], "scales": sc.grad, "rotations": rt.grad,
                 "alphas": g["alphas"]}
