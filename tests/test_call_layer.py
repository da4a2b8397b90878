"""Host logic of the call layer (igs_b200/_lib.py), no GPU: what is remembered about grids,
how the ordering key is formed, what the policy decides before anything is launched."""
import math

import pytest
import torch


@pytest.fixture
def lib(monkeypatch):
    from igs_b200 import _lib

    # (the capture query needs a CUDA context; none of this logic does)
    monkeypatch.setattr(torch.cuda, "is_current_stream_capturing", lambda: False)
    _lib.forget_what_calls_learnt()
    yield _lib
    _lib.forget_what_calls_learnt()


def _grid(B, H, W):
    x = torch.linspace(-1, 1, W).view(1, 1, 1, W).expand(B, 1, H, W).contiguous()
    y = torch.linspace(-1, 1, H).view(1, 1, H, 1).expand(B, 1, H, W).contiguous()
    return x, y


def test_remembered_grids(lib):
    B, H, W = 2, 8, 32
    x, y = _grid(B, H, W)
    x3, y3, hints, entry = lib.grid_for_call(x, y, B)
    assert hints == 0 and entry is not None and entry.kind is None
    assert x3.stride(1) != 0  # nothing known yet: the tensors as they are
    # still unknown on the next call: the same entry wants to learn
    assert lib.grid_for_call(x, y, B)[3] is entry
    entry.kind = "separable"  # what a status read would have filled in
    x3, y3, hints, again = lib.grid_for_call(x, y, B)
    assert again is None and hints == 0
    assert x3.stride(1) == 0 and y3.stride(2) == 0 and x3.shape == (B, H, W)
    assert torch.equal(x3, x[:, 0]) and torch.equal(y3, y[:, 0])
    # an in-place change moves the version counter: the entry no longer applies
    x.add_(0.01)
    x3, y3, hints, fresh = lib.grid_for_call(x, y, B)
    assert fresh is not None and fresh is not entry and fresh.kind is None and x3.stride(1) != 0
    fresh.kind = "general"
    x3, y3, hints, none = lib.grid_for_call(x, y, B)
    assert hints == lib.HINT_GENERAL_GRID and none is None and x3.stride(1) != 0
    # another pair of tensors with the same values is another pair
    x2, y2 = _grid(B, H, W)
    assert lib.grid_for_call(x2, y2, B)[3].kind is None
    # stride-0 views and tiny images need no entry at all
    xv, yv = x2[:, :, :1].expand(B, 1, H, W), y2[:, :, :, :1].expand(B, 1, H, W)
    assert lib.grid_for_call(xv, yv, B)[3] is None
    xs, ys = _grid(1, 2, 8)
    assert lib.grid_for_call(xs, ys, 1)[3] is None
    # dead tensors are forgotten when the next new pair arrives
    n_before = len(lib._grid_memos)
    del x2, y2, xv, yv
    x4, y4 = _grid(B, H, W)
    lib.grid_for_call(x4, y4, B)
    assert len(lib._grid_memos) <= n_before


def test_grid_argument_errors(lib):
    x, y = _grid(2, 8, 32)
    with pytest.raises(ValueError):
        lib.grid_for_call(x[:, 0], y[:, 0], 2)
    with pytest.raises(ValueError):
        lib.grid_for_call(x, y[:, :, :4], 2)
    with pytest.raises(ValueError):
        lib.grid_for_call(x, y, 3)


def test_a_new_image_size_starts_from_what_the_same_gaussians_showed(lib):
    """Narrow or wide is judged against the sampled extent, so the answer carries over to another
    image size of the same (device, B, N) as a first guess; other gaussian counts start unknown."""
    dev = torch.device("cuda", 0)
    lib.forget_what_calls_learnt()
    small = lib._shape_memo(dev, 1, 500, 64, 64)
    assert small.narrow is None
    small.narrow = True
    lib._family_narrow[small.family] = True  # (what folding a completed read into the memo does)
    big = lib._shape_memo(dev, 1, 500, 128, 128)
    assert big is not small and big.narrow is True and big.calls == 0 and not big.pending
    assert lib._shape_memo(dev, 1, 501, 128, 128).narrow is None
    assert lib._shape_memo(dev, 2, 500, 128, 128).narrow is None
    lib.forget_what_calls_learnt()
    assert lib._shape_memo(dev, 1, 500, 256, 256).narrow is None
    lib.forget_what_calls_learnt()


def test_policy_decides_without_launching(lib):
    B, N, H, W = 1, 64, 16, 16
    x, y = _grid(B, H, W)
    pos = torch.rand(B, N, 2)
    lib.set_backward_sort("off")
    try:
        memo = lib._shape_memo(torch.device("cuda", 0), B, N, H, W)
        assert lib.order_by_policy(memo, pos, None, None, x[:, 0], y[:, 0]) is None
        lib.set_backward_sort("auto")
        memo = lib._shape_memo(torch.device("cuda", 0), B, N, H, W)
        assert memo.narrow is None and lib.order_by_policy(memo, pos, None, None, x[:, 0], y[:, 0]) is None
        memo.narrow = False
        assert lib.order_by_policy(memo, pos, None, None, x[:, 0], y[:, 0]) is None
        memo.narrow = True  # narrow, but far below the size from which "auto" orders eager calls
        assert lib.order_by_policy(memo, pos, None, None, x[:, 0], y[:, 0]) is None
        with pytest.raises(ValueError):
            lib.set_backward_sort("sometimes")
    finally:
        lib.set_backward_sort("auto")
