"""Multi-GPU use of the splat: one process per GPU (torchrun), ``torch.distributed``.

Two ways the work shards (nothing in the reference is distributed; this is the scheme
the batch / gaussian structure of ``src/igs/gs2d.py:275-337`` allows):

* **Batch** (B >= world size): batch elements are independent, so every rank renders its
  own block with the ordinary ``gaussian_splatting_2d`` and there is no collective on the
  data path.  ``batch_range`` gives the block.
* **Gaussian ranges** (B = 1, or any B with many gaussians): numerator and weight sum are
  plain sums over gaussians.  Every rank renders the un-normalised sums of its own range
  over the full image, one ``all_reduce(SUM)`` of ``[B, C+1, H, W]`` combines them, every
  rank normalises, and the backward is local: a rank produces the gradients of its own
  gaussians only.  ``sharded_gaussian_splatting_2d`` does this.

Before a group's first collective on a given shape the ranks compare shapes on the host
(``check_consistent``), so a rank that was handed a different image size raises on every
rank instead of hanging or corrupting the reduction.  The comparison costs a collective of
its own and a device-to-host read, so it runs once per (group, shape), not per step: it
catches a job that was set up inconsistently, not a rank whose shape changes later while
the others' stay.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.autograd.function import once_differentiable

from . import gs2d


def batch_range(B: int, world: int, rank: int):
    """Contiguous block [lo, hi) of the batch owned by ``rank``; sizes differ by at most 1."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(B, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gaussian_range(N: int, world: int, rank: int):
    """Contiguous range [lo, hi) of the gaussians owned by ``rank``."""
    return batch_range(N, world, rank)


_checked = set()  # (id of the group, the values) that have passed check_consistent


def check_consistent_once(values, group=None):
    """check_consistent the first time this process sees `values` for `group`; nothing after."""
    key = (id(group) if group is not None else 0, tuple(int(v) for v in values))
    if key in _checked:
        return
    check_consistent(values, group)
    _checked.add(key)


def check_consistent(values, group=None):
    """All ranks must pass the same integers (image size, channels, batch): gathers them on
    the host side of the collective and raises ValueError on every rank if they differ."""
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    mine = torch.tensor([int(v) for v in values], dtype=torch.int64, device=dev)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    rows = [tuple(t.tolist()) for t in gathered]
    if any(r != rows[0] for r in rows):
        raise ValueError(f"ranks disagree on (B, C, H, W): {rows}")


class CudaSplatBackend:
    """The three device calls the sharded op is built from (libigs_b200.so).  `info` is what
    `prepare` returned for the step: grid views, hints and the memos of the call layer."""

    @staticmethod
    def prepare(x, y, pos, scales=None, rotations=None):
        from . import _lib

        return _lib.prepare_call(x, y, pos, scales=scales, rotations=rotations)

    @staticmethod
    def forward_sums(pos, col, sc, rot, al, x3, y3, eps, info=None):
        from . import _lib

        sums, _ = _lib.forward("sr", pos, sc, rot, None, al, col, x3, y3, eps, normalize=False,
                               order=info.order if info else None, hints=info.hints if info else 0, info=info)
        return sums

    @staticmethod
    def normalize(sums, eps):
        from . import _lib

        return _lib.normalize(sums, eps)

    @staticmethod
    def backward(pos, col, sc, rot, al, x3, y3, wsum, out, gout, eps, grad_mode, info=None, order=None):
        from . import _lib

        return _lib.backward("sr", pos, sc, rot, None, al, col, x3, y3, wsum, out, gout, eps, grad_mode, False,
                             order=order, hints=info.hints if info else 0, info=info)


def _plain_views(x, y, B):
    H, W = x.shape[2], x.shape[3]
    return x[:, 0].expand(B, H, W), y[:, 0].expand(B, H, W)


class _ShardedSplat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, positions, colors, scales, rotations, alphas, x, y, eps, group, backend):
        B = positions.shape[0]
        pos, col, sc, rot, al = (t.contiguous() for t in (positions, colors, scales, rotations, alphas))
        check_consistent_once((B, col.shape[2], x.shape[2], x.shape[3]), group)
        if hasattr(backend, "prepare"):
            info = backend.prepare(x, y, pos, sc, rot)
            sums = backend.forward_sums(pos, col, sc, rot, al, info.x3, info.y3, eps, info=info)
        else:
            info = None
            x3, y3 = _plain_views(x, y, B)
            sums = backend.forward_sums(pos, col, sc, rot, al, x3, y3, eps)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM, group=group)
        out, wsum = backend.normalize(sums, eps)
        if info is not None:
            gs2d._save_call(ctx, info, x, y, pos, col, sc, rot, al, wsum, out)
        else:
            ctx.save_for_backward(x, y, pos, col, sc, rot, al, wsum, out)
            ctx.call_info = None
        ctx.eps, ctx.backend = float(eps), backend
        ctx.grad_mode = gs2d._GRAD_MODES[gs2d.get_grad_mode()]
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_result):
        if ctx.needs_input_grad[5] or ctx.needs_input_grad[6]:
            raise NotImplementedError("gradients of x_grid / y_grid are not available in the gaussian-sharded op")
        if ctx.call_info is not None:
            (x, y, pos, col, sc, rot, al, wsum, out), x3, y3, order = gs2d._saved_call(ctx)
            g = ctx.backend.backward(pos, col, sc, rot, al, x3, y3, wsum, out, grad_result.contiguous(), ctx.eps,
                                     ctx.grad_mode, info=ctx.call_info, order=order)
        else:
            x, y, pos, col, sc, rot, al, wsum, out = ctx.saved_tensors
            x3, y3 = _plain_views(x, y, pos.shape[0])
            g = ctx.backend.backward(pos, col, sc, rot, al, x3, y3, wsum, out, grad_result.contiguous(), ctx.eps,
                                     ctx.grad_mode)
        return (g["positions"], g["colors"], g["scales"], g["rotations"], g["alphas"], None, None, None, None, None)


def sharded_gaussian_splatting_2d(positions, colors, scales, rotations, alphas, x_grid, y_grid, eps=1e-6,
                                  group=None, backend=None):
    """``gaussian_splatting_2d`` over gaussians spread across the ranks of ``group``.

    Each rank passes ITS OWN gaussians (``[B, N_local, ...]``; ranges from
    ``gaussian_range``) and the SAME grids; every rank receives the full image
    ``[B, C, H, W]``.  The upstream gradient must be the same on all ranks (a loss computed
    from the full image is); backward returns gradients for the local gaussians.  One
    all-reduce of ``B*(C+1)*H*W`` floats per forward, none in backward.
    """
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised (launch with torchrun)")
    if backend is None:
        backend = CudaSplatBackend
        for n, t in (("positions", positions), ("colors", colors), ("scales", scales), ("rotations", rotations),
                     ("alphas", alphas), ("x_grid", x_grid), ("y_grid", y_grid)):
            gs2d._require_cuda_f32(n, t)
    gs2d._check_gaussians(positions, alphas, colors)
    return _ShardedSplat.apply(positions, colors, scales, rotations, alphas, x_grid, y_grid, eps, group, backend)
