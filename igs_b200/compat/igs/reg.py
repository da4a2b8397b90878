"""``igs.reg`` under its reference name: re-exports ``igs_b200.reg``."""
from igs_b200.reg import koleo_diversity_loss  # noqa: F401
