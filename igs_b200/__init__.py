"""igs_b200 -- B200 (sm_100a) implementation of IGS's differentiable 2D gaussian
splatting, behind the reference's ``igs.gs2d`` names.

    from igs_b200 import GaussianSplatting2D
    from igs_b200.gs2d import gaussian_splatting_2d, GaussianSplatting2DKernel

Importing the package does not load the CUDA library; the first call does, and fails
loudly if it is missing (there is no CPU or PyTorch fallback).
"""
from ._lib import set_backward_sort, set_culling
from .gs2d import (GaussianSplatting2D, GaussianSplatting2DKernel, gaussian_splatting_2d, get_grad_mode,
                   grad_mode, set_grad_mode)

__all__ = ["GaussianSplatting2D", "GaussianSplatting2DKernel", "gaussian_splatting_2d", "set_grad_mode",
           "get_grad_mode", "grad_mode", "set_culling", "set_backward_sort"]
__version__ = "0.1.0"
