"""Seeded synthetic workloads: the five benchmark configurations and helpers to draw
inputs with their shapes and value distributions.

The reference measures on no public dataset (its scripts read local image files that
are not part of its repository), so every input here is synthetic: drawn on the CPU
from ``torch.Generator().manual_seed(seed)`` in a fixed order (positions, colors,
scales, rotations, alphas, target) and then moved to the device, so that a CPU checker
and the CUDA kernels see identical bits.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class SplatConfig:
    name: str
    B: int
    N: int
    H: int
    W: int
    C: int
    scale_lo: float
    scale_hi: float
    normal_colors: bool = False
    seed: int = 0
    loss: str = "mse"  # "mse" (mean) or "sse" (sum of squares)


CONFIGS = {
    # B=1, N=2048, 256x256, C=3: the reference's own CPU-runnable case
    "cfg0": SplatConfig("cfg0", 1, 2048, 256, 256, 3, 0.25, 0.75, seed=0, loss="sse"),
    # headline: batched training shape
    "cfg2": SplatConfig("cfg2", 16, 8192, 256, 256, 3, 0.25, 0.75, seed=2),
    # the headline shape cut down (B=4, N=4096) for profiler captures that must stay short
    "cfg2_small": SplatConfig("cfg2_small", 4, 4096, 256, 256, 3, 0.25, 0.75, seed=2),
    # single-image fit, sharded over gaussian ranges when run on several GPUs
    "cfg3": SplatConfig("cfg3", 1, 16384, 512, 512, 3, 0.05, 0.30, seed=3),
    # large feature-map render
    "cfg4": SplatConfig("cfg4", 64, 65536, 512, 512, 16, 0.02, 0.20, normal_colors=True, seed=4),
    # the regime of the reference's per-image fit (scripts/2dgs_img_comp.py: thousands of
    # gaussians of scale ~e^-5 on a 1024x1024 image): almost every (gaussian, pixel) weight is
    # exactly zero, which the lossless culling exploits
    "narrow": SplatConfig("narrow", 1, 16384, 1024, 1024, 3, 0.004, 0.012, seed=7),
    # the image-compression regime at a larger gaussian count (reference: 2dgs_img_comp.py trains
    # tens of thousands of gaussians of scale ~e^-5.5 at 1024 px)
    "narrow64k": SplatConfig("narrow64k", 1, 65536, 1024, 1024, 3, 0.002, 0.006, seed=8),
    # config 4 cut down (one batch element, a quarter of the gaussians) for profiler captures
    "cfg4_small": SplatConfig("cfg4_small", 1, 16384, 512, 512, 16, 0.02, 0.20, normal_colors=True, seed=4),
    # one GPU's share of config 4 when its batch of 64 is spread over 8 GPUs
    "cfg4_b8": SplatConfig("cfg4_b8", 8, 65536, 512, 512, 16, 0.02, 0.20, normal_colors=True, seed=4),
}


def xy_grid(H, W, B, device="cpu", expand=False):
    """[B,1,H,W] pixel-centre coordinates, same values as the reference's
    ``GaussianSplatting2D.xy_grid`` (src/igs/gs2d.py:503-522) repeated over the batch."""
    hr = (H / W) ** 0.5
    wr = 1 / hr
    xs = torch.linspace(-wr, wr, W)
    ys = torch.linspace(-hr, hr, H)
    x = xs.view(1, 1, 1, W).expand(B, 1, H, W)
    y = ys.view(1, 1, H, 1).expand(B, 1, H, W)
    if not expand:
        x, y = x.contiguous(), y.contiguous()
    return x.to(device), y.to(device)


def draw(cfg: SplatConfig, B=None, N=None, device="cpu", with_target=True):
    """Returns a dict of CPU-drawn tensors moved to ``device``."""
    B = cfg.B if B is None else B
    N = cfg.N if N is None else N
    gen = torch.Generator().manual_seed(cfg.seed)
    pos = torch.rand(B, N, 2, generator=gen) * 2 - 1
    if cfg.normal_colors:
        col = torch.randn(B, N, cfg.C, generator=gen)
    else:
        col = torch.rand(B, N, cfg.C, generator=gen)
    sc = torch.rand(B, N, 2, generator=gen) * (cfg.scale_hi - cfg.scale_lo) + cfg.scale_lo
    rot = torch.rand(B, N, generator=gen) * 2 * math.pi
    al = torch.rand(B, N, generator=gen)
    out = {"positions": pos, "colors": col, "scales": sc, "rotations": rot, "alphas": al}
    if with_target:
        out["target"] = torch.rand(B, cfg.C, cfg.H, cfg.W, generator=gen)
    x, y = xy_grid(cfg.H, cfg.W, B)
    out["x"], out["y"] = x, y
    return {k: v.to(device) for k, v in out.items()}


def evals(cfg: SplatConfig, B=None, N=None) -> int:
    """gaussian x pixel evaluations of one pass over the configuration."""
    return (cfg.B if B is None else B) * (cfg.N if N is None else N) * cfg.H * cfg.W
