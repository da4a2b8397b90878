"""Import shim: put ``igs_b200/compat`` on ``sys.path`` and existing code that does
``from igs import GaussianSplatting2D`` / ``import igs.gs2d`` (reference
src/igs/__init__.py:1) picks up the B200 implementation unchanged."""
from igs_b200.gs2d import GaussianSplatting2D  # noqa: F401
