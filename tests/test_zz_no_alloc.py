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


def _call(lib, static, t, B, N, H, W, C, dev, normalize=1, check_memory=False):
    """Runs one of the two entry points on the current stream; returns (rc, out, wsum).
    check_memory: the device's free memory (cudaMemGetInfo) must be the same before and after
    the call -- the entry point's promise."""
    planes = C if normalize else C + 1
    out = torch.full((B, planes, H, W), float("nan"), device=dev)
    wsum = torch.full((B, H, W), float("nan"), device=dev)
    xs, ys = (ctypes.c_int64 * 3)(*t["x"].stride()), (ctypes.c_int64 * 3)(*t["y"].stride())
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    head = (_p(t["pos"]), _p(t["scales"]), _p(t["rot"]), _p(t["alpha"]), _p(t["col"]), _p(t["x"]), xs, _p(t["y"]),
            ys, B, N, H, W, C, 1e-6, normalize, _p(out), _p(wsum))
    if static:
        torch.cuda.synchronize(dev)
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = lib.igs_forward_sr_static(*head, dev.index, stream)
        torch.cuda.synchronize(dev)
        if check_memory:
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the device's free memory"
    else:
        fb, bb = ctypes.c_size_t(0), ctypes.c_size_t(0)
        assert lib.igs_workspace_bytes(B, N, H, W, C, dev.index, ctypes.byref(fb), ctypes.byref(bb)) == 0
        ws = torch.empty(max(fb.value, 256), dtype=torch.uint8, device=dev)
        rc = lib.igs_forward_sr(*head, None, 0, _p(ws), ws.numel(), dev.index, stream)
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


def _oracle_image(t, eps=1e-6):
    from oracle import splat_oracle as so

    n = {k: v.cpu().numpy() for k, v in t.items()}
    return so.render(n["pos"], n["col"], n["scales"], n["rot"], n["alpha"], np.ascontiguousarray(n["x"]),
                     np.ascontiguousarray(n["y"]), eps, dtype=np.float64)


def _with_xy_grid(t, B, H, W, dev, materialised):
    """Replaces the random sample points by the reference's pixel grid: x by column, y by row,
    so that the separable (and, with narrow gaussians, the culling) kernels run."""
    from tests._util import xy_grid_np

    x, y = xy_grid_np(H, W, B)
    t = dict(t)
    t["x"], t["y"] = torch.from_numpy(x).to(dev), torch.from_numpy(y).to(dev)
    if not materialised:  # stride-0 views: separable by construction, nothing is checked
        t["x"], t["y"] = t["x"][:, :1, :].expand(B, H, W), t["y"][:, :, :1].expand(B, H, W)
    return t


@pytest.mark.parametrize("grid", ["points", "xy_grid", "xy_grid_views"])
@pytest.mark.parametrize("narrow", [False, True])
def test_static_scratch_forward_against_the_oracle(grid, narrow):
    """Against the fp64 oracle, not only against the other entry point: arbitrary sample
    points (general kernels), a materialised pixel grid (checked on the device, separable
    kernels) and stride-0 views of one; wide gaussians and narrow ones (the culling
    instantiations).  Device memory must not move, and no kernel may report a timed-out
    wait through the array's status word."""
    from igs_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, N, H, W, C = 2, 900, 48, 80, 3
    t = _inputs(B, N, H, W, C, 505, dev)
    if narrow:
        t["scales"] = (t["scales"] * 0.05).contiguous()
    if grid != "points":
        t = _with_xy_grid(t, B, H, W, dev, materialised=(grid == "xy_grid"))
    want, want_wsum = _oracle_image(t)
    for _ in range(2):  # twice: the second call finds the first one's leftovers in the array
        rc, out, wsum = _call(lib, True, t, B, N, H, W, C, dev, check_memory=True)
        assert rc == 0, lib.igs_strerror(rc)
        assert_close(out.cpu().numpy(), want, 1e-4, f"image ({grid}, narrow={narrow})")
        assert_close(wsum.cpu().numpy(), want_wsum, 1e-4, f"weight sum ({grid}, narrow={narrow})")
    status = ctypes.c_int(-1)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    assert lib.igs_read_status_static(dev.index, stream, ctypes.byref(status)) == 0
    assert status.value == 0


def test_static_scratch_drops_the_gaussian_splits_when_only_the_records_fit():
    """B=1, N=4096 on 512x512: the records take 192 KiB, but the plan would split the
    gaussians over several CTAs per tile and each split's partial sums take 4 MiB, which does
    not fit the 8 MiB array.  The entry point then runs one split per tile.  Same result as
    igs_forward_sr up to the order of summation, normalised or not; also held to the oracle at
    sampled pixels."""
    from igs_b200 import _lib
    from oracle import splat_oracle as so

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    B, N, H, W, C = 1, 4096, 512, 512, 3
    plan = _lib.describe_plan(B, N, H, W, C, dev)
    assert plan["fwd_splits"] * B * (C + 1) * H * W * 4 > STATIC_SCRATCH_BYTES, plan  # the branch under test
    t = _with_xy_grid(_inputs(B, N, H, W, C, 606, dev), B, H, W, dev, materialised=True)
    for normalize in (1, 0):
        rc_ref, out_ref, wsum_ref = _call(lib, False, t, B, N, H, W, C, dev, normalize=normalize)
        rc, out, wsum = _call(lib, True, t, B, N, H, W, C, dev, normalize=normalize, check_memory=True)
        assert rc_ref == 0 and rc == 0, (rc_ref, rc)
        assert_close(out.cpu().numpy(), out_ref.cpu().numpy(), 1e-5, f"normalize={normalize}")
        if normalize:
            assert_close(wsum.cpu().numpy(), wsum_ref.cpu().numpy(), 1e-5, "weight sum")
    rng = np.random.default_rng(6)
    idx = rng.choice(H * W, size=256, replace=False)
    n = {k: v.cpu().numpy() for k, v in t.items()}
    xs, ys = n["x"].reshape(B, -1)[:, idx][:, None, :], n["y"].reshape(B, -1)[:, idx][:, None, :]
    want, _ = so.render(n["pos"], n["col"], n["scales"], n["rot"], n["alpha"], xs, ys, 1e-6, dtype=np.float64)
    rc, out, _ = _call(lib, True, t, B, N, H, W, C, dev)
    assert_close(out.cpu().numpy().reshape(B, C, -1)[:, :, idx][:, :, None, :], want, 1e-4, "image at sampled pixels")
