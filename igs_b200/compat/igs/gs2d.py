"""``igs.gs2d`` under its reference name: re-exports ``igs_b200.gs2d``."""
from igs_b200.gs2d import *  # noqa: F401,F403
from igs_b200.gs2d import (GaussianSplatting2D, GaussianSplatting2DChunkedKernel,  # noqa: F401
                           GaussianSplatting2DKernel, TorchGaussianSplatting2DChunked,
                           TorchGaussianSplatting2DKernel, gaussian_splatting_2d, log_vram, naive_gaussian_2d)
