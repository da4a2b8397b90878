"""``igs.reg`` under its reference name: the KoLeo-style diversity regulariser the
reference's feature -> image experiment adds to its loss (src/igs/reg.py:5-40,
used at scripts/gs2d_test.py:146,172).  Not on the splat path: an O(N^2 D) batched
matrix product, left to torch (cuBLAS); works on any device.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def koleo_diversity_loss(features: torch.Tensor) -> torch.Tensor:
    """features [B,N,D] -> scalar: mean over all vectors of relu(1 + cosine similarity to
    the nearest other vector of the same batch element); 0 when N <= 1."""
    n = features.shape[1]
    if n <= 1:
        return torch.tensor(0.0, device=features.device)
    unit = F.normalize(features, p=2, dim=-1)
    sim = torch.bmm(unit, unit.transpose(1, 2))
    eye = torch.eye(n, dtype=torch.bool, device=features.device)
    nearest = sim.masked_fill(eye, float("-inf")).amax(dim=-1)
    return F.relu(nearest + 1.0).mean()
