"""igs_forward_sr_static: the forward for hosts that cannot allocate device memory.

Some users of the C ABI are not PyTorch and own no allocator: a plug-in living inside
another application's fixed memory budget, or a render loop that must never call into
the driver's allocator once it runs.  For them the library carries its scratch in a
fixed device array, and this entry point takes no workspace.  The test calls it through
the C ABI only (ctypes; torch merely provides the input and output buffers, which such a
host would own already) and checks it against igs_forward_sr, the entry point that takes
a caller-allocated workspace, on two calls in a row with different inputs: the array is
shared and keeps the previous call's contents, so the second call proves that nothing
stale is consumed.  Collected last so that a run stopping at the first failure has
already exercised every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests._util import assert_close

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20  # IGS_STATIC_SCRATCH_BYTES in include/igs_b200.h


def _inputs(B, N, H, W, C, seed, dev):
    gen = torch.Generator().manual_seed(seed)
    t = {
        "pos": torch.rand(B, N, 2, generator=gen) * 2 - 1,
        "scales": torch.rand(B, N, 2, generator=gen) * 0.4 + 0.1,
        "rot": torch.rand(B, N, generator=gen) * 6.2831853,
        "alpha": torch.rand(B, N, generator=gen),
        "col": torch.rand(B, N, C, generator=gen),
        "x": (torch.rand(B, H, W, generator=gen) * 2 - 1),
        "y": (torch.rand(B, H, W, generator=gen) * 2 - 1),
    }
    return {k: v.to(dev).contiguous() for k, v in t.items()}


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(lib, static, t, B, N, H, W, C, dev, normalize=1):
    """Runs one of the two entry points on the current stream; returns (rc, out, wsum)."""
    planes = C if normalize else C + 1
    out = torch.full((B, planes, H, W), float("nan"), device=dev)
    wsum = torch.full((B, H, W), float("nan"), device=dev)
    strides = (ctypes.c_int64 * 3)(H * W, W, 1)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    head = (_p(t["pos"]), _p(t["scales"]), _p(t["rot"]), _p(t["alpha"]), _p(t["col"]), _p(t["x"]), strides, _p(t["y"]),
            strides, B, N, H, W, C, 1e-6, normalize, _p(out), _p(wsum))
    if static:
        rc = lib.igs_forward_sr_static(*head, dev.index, stream)
    else:
        fb, bb = ctypes.c_size_t(0), ctypes.c_size_t(0)
        assert lib.igs_workspace_bytes(B, N, H, W, C, dev.index, ctypes.byref(fb), ctypes.byref(bb)) == 0
        ws = torch.empty(max(fb.value, 256), dtype=torch.uint8, device=dev)
        rc = lib.igs_forward_sr(*head, None, _p(ws), ws.numel(), dev.index, stream)
    torch.cuda.synchronize(dev)
    return rc, out, wsum


def test_static_scratch_forward_matches_workspace_forward():
    from igs_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    # two calls in a row, the second with fewer gaussians, another image size and other
    # values: whatever the first call left in the shared array must not leak into it
    shapes = [(2, 700, 40, 36, 3, 101), (1, 130, 25, 31, 3, 202)]
    for B, N, H, W, C, seed in shapes:
        t = _inputs(B, N, H, W, C, seed, dev)
        rc_ref, out_ref, wsum_ref = _call(lib, False, t, B, N, H, W, C, dev)
        rc, out, wsum = _call(lib, True, t, B, N, H, W, C, dev)
        assert rc_ref == 0 and rc == 0, (rc_ref, rc, lib.igs_strerror(rc))
        assert_close(out.cpu().numpy(), out_ref.cpu().numpy(), 1e-5, f"image B={B} N={N}")
        assert_close(wsum.cpu().numpy(), wsum_ref.cpu().numpy(), 1e-5, f"weight sum B={B} N={N}")


def test_static_scratch_unnormalised_sums_and_limit():
    from igs_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, N, H, W, C = 1, 300, 20, 20, 3
    t = _inputs(B, N, H, W, C, 303, dev)
    rc_ref, sums_ref, _ = _call(lib, False, t, B, N, H, W, C, dev, normalize=0)
    rc, sums, _ = _call(lib, True, t, B, N, H, W, C, dev, normalize=0)
    assert rc_ref == 0 and rc == 0
    assert_close(sums.cpu().numpy(), sums_ref.cpu().numpy(), 1e-5, "un-normalised sums")

    # records alone take 48 bytes per gaussian at C=3: this many cannot fit the array
    n_big = STATIC_SCRATCH_BYTES // 48 + 4096
    big = _inputs(1, n_big, 8, 8, 3, 404, dev)
    rc, out, _ = _call(lib, True, big, 1, n_big, 8, 8, 3, dev)
    assert rc == -3, lib.igs_strerror(rc)          # IGS_ERR_LIMIT, nothing launched
    assert bool(torch.isnan(out).all())
    assert b"static" in lib.igs_strerror(rc)
