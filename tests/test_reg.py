"""igs_b200.reg.koleo_diversity_loss against the reference's own output (fixture)."""
import numpy as np
import torch

from tests._util import load_golden


def test_koleo_matches_reference_fixture():
    from igs_b200.reg import koleo_diversity_loss

    g = load_golden("koleo")
    f = torch.from_numpy(g["features"]).requires_grad_()
    loss = koleo_diversity_loss(f)
    loss.backward()
    assert abs(float(loss.detach()) - float(g["loss"])) <= 1e-6
    assert np.abs(f.grad.numpy() - g["g_features"]).max() <= 1e-6


def test_koleo_degenerate_and_compat_import():
    import os
    import sys

    from igs_b200.reg import koleo_diversity_loss

    assert float(koleo_diversity_loss(torch.zeros(2, 1, 4))) == 0.0
    compat = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "igs_b200", "compat")
    sys.path.insert(0, compat)
    try:
        import igs
        import igs.gs2d
        import igs.reg

        assert igs.reg.koleo_diversity_loss is koleo_diversity_loss
        assert igs.GaussianSplatting2D is igs.gs2d.GaussianSplatting2D
    finally:
        sys.path.remove(compat)
        for k in [k for k in sys.modules if k == "igs" or k.startswith("igs.")]:
            del sys.modules[k]
