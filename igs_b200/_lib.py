"""ctypes binding of ``libigs_b200.so`` (declared in ``include/igs_b200.h``).

There is no fallback: if the shared object is missing and cannot be built, or a call
is made with tensors that are not on a CUDA device, an exception is raised.  torch is
used here only for device memory (``tensor.data_ptr()``), the current stream and the
scratch allocations the library asks for.
"""
from __future__ import annotations

import ctypes
import functools
import os
import threading
import weakref

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libigs_b200.so")

GRAD_REFERENCE = 0
GRAD_EXACT = 1
# `hints` of the forward / backward entry points (include/igs_b200.h)
HINT_WIDE_GAUSSIANS = 1
HINT_GENERAL_GRID = 2
STATUS_WORDS = 8

_lock = threading.Lock()
_lib = None

_F = ctypes.POINTER(ctypes.c_float)
_I64 = ctypes.POINTER(ctypes.c_int64)
_vp, _i, _f, _sz, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t, ctypes.c_int64

# name -> (restype, argtypes); mirrors include/igs_b200.h one to one
SIGNATURES = {
    "igs_version": (_i, []),
    "igs_strerror": (ctypes.c_char_p, [_i]),
    "igs_launch_count": (ctypes.c_longlong, []),
    "igs_workspace_bytes": (_i, [_i] * 6 + [ctypes.POINTER(_sz)] * 2),
    "igs_forward_sr": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _i, _vp, _sz, _i, _vp]),
    "igs_forward_cov": (_i, [_vp] * 7 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _i, _vp, _sz, _i, _vp]),
    "igs_forward_sr_static": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _i, _vp]),
    "igs_normalize": (_i, [_vp] + [_i] * 4 + [_f, _vp, _vp, _i, _vp]),
    "igs_backward_sr": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 8
                        + [_i, _vp, _sz, _i, _vp]),
    "igs_backward_cov": (_i, [_vp] * 7 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 9
                         + [_i, _vp, _sz, _i, _vp]),
    "igs_forward_feature": (_i, [_vp] * 3 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _i, _vp, _sz, _i,
                                                                           _vp]),
    "igs_backward_feature": (_i, [_vp] * 3 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 2
                             + [_i, _vp, _sz, _i, _vp]),
    "igs_read_status": (_i, [_vp, _i, _vp, ctypes.POINTER(_i)]),
    "igs_read_status_static": (_i, [_i, _vp, ctypes.POINTER(_i)]),
    "igs_read_status_words": (_i, [_vp, _i, _vp, _vp]),
    "igs_set_culling": (_i, [_i]),
    "igs_spatial_order_workspace_bytes": (_sz, [_i, _i]),
    "igs_spatial_order": (_i, [_vp, _vp, _I64, _vp, _I64] + [_i] * 4 + [_vp, _vp, _sz, _i, _vp]),
    "igs_spatial_order_boxes": (_i, [_vp, _i64, _vp, _vp, _i64, _i, _vp, _i64, _vp, _I64, _vp, _I64] + [_i] * 4
                                + [_vp, _vp, _sz, _i, _vp]),
    "igs_read_narrow_count": (_i, [_vp, _i, _vp, _vp]),
    "igs_read_executed": (_i, [_vp, _i, _vp, ctypes.POINTER(ctypes.c_ulonglong)]),
    "igs_render_mse_workspace_bytes": (_i, [_i] * 6 + [ctypes.POINTER(_sz)]),
    "igs_render_mse_sr": (_i, [_vp] * 5 + [_i, _vp, _I64, _vp, _I64, _vp] + [_i] * 5 + [_f, _i] + [_vp] * 9
                          + [_i, _vp, _sz, _i, _vp]),
    "igs_mse_loss": (_i, [_vp, _vp, ctypes.c_longlong, _vp, _vp, _sz, _i, _vp]),
    "igs_mse_grad": (_i, [_vp, _vp, ctypes.c_longlong, _vp, _vp, _i, _vp]),
    "igs_profile_enable": (_i, [_i]),
    "igs_profile_reset": (_i, []),
    "igs_profile_read": (_i, [_i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_longlong)]),
    "igs_describe_plan": (_i, [_i] * 6 + [ctypes.POINTER(_i)] * 4),
    "igs_describe_kernels": (_i, [_i] + [ctypes.POINTER(_i)] * 2),
}


class IgsError(RuntimeError):
    """A call into libigs_b200.so returned a non-zero code."""

    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} failed with code {code}: {msg}")
        self.code = code


def load() -> ctypes.CDLL:
    """Loads the shared object, building it first when it is missing or was built from
    other sources than the tree holds now (``build.is_stale``: a hash of the sources)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import build as _build

        if _build.is_stale():
            try:
                _build.build()
            except Exception as exc:  # noqa: BLE001 - surfaced verbatim below
                raise ImportError(
                    f"igs_b200: {LIB_PATH} is missing or out of date and could not be built ({exc}). "
                    "Run `python -m igs_b200.build`; there is no CPU or PyTorch fallback.") from exc
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                raise AttributeError(f"{LIB_PATH} does not export {name}: header and library out of sync")
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(fn: str, code: int) -> None:
    if code != 0:
        raise IgsError(fn, code, load().igs_strerror(code).decode())


def launch_count() -> int:
    return int(load().igs_launch_count())


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


# torch's current stream on a device as a raw handle, without building a Stream object for it
# (a few microseconds per call, twice per step on a host-bound step)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device: torch.device):
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(device.index))
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _strides3(t: torch.Tensor):
    """Element strides (batch, row, column) of a [B,H,W] view as a C int64[3]."""
    return (ctypes.c_int64 * 3)(*t.stride())


@functools.lru_cache(maxsize=256)
def _workspace_bytes(B, N, H, W, C, index):
    f, b = _sz(0), _sz(0)
    check("igs_workspace_bytes", load().igs_workspace_bytes(B, N, H, W, C, index, ctypes.byref(f), ctypes.byref(b)))
    return int(f.value), int(b.value)


def workspace_bytes(B, N, H, W, C, device: torch.device):
    """(forward, backward) scratch bytes; a pure function of the shape and the device."""
    return _workspace_bytes(int(B), int(N), int(H), int(W), int(C), device.index)


def describe_plan(B, N, H, W, C, device: torch.device):
    v = [_i(0) for _ in range(4)]
    check("igs_describe_plan", load().igs_describe_plan(B, N, H, W, C, device.index, *[ctypes.byref(k) for k in v]))
    return {"fwd_tile_pixels": v[0].value, "fwd_splits": v[1].value, "bwd_threads": v[2].value,
            "bwd_slabs": v[3].value}


def separable_kernels(C: int):
    """(forward, backward): whether separable-grid kernels exist for C channels."""
    f, b = _i(0), _i(0)
    check("igs_describe_kernels", load().igs_describe_kernels(int(C), ctypes.byref(f), ctypes.byref(b)))
    return bool(f.value), bool(b.value)


def _workspace(nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def read_status(ws: torch.Tensor) -> int:
    host = _i(0)
    rc = load().igs_read_status(_ptr(ws), ws.device.index, _stream(ws.device), ctypes.byref(host))
    if rc not in (0, -5):
        check("igs_read_status", rc)
    return int(host.value)


def read_executed(ws: torch.Tensor) -> int:
    """(gaussian, pixel) evaluations the culling kernel of the last call on ws did not skip;
    0 when the plain kernel ran."""
    host = ctypes.c_ulonglong(0)
    check("igs_read_executed", load().igs_read_executed(_ptr(ws), ws.device.index, _stream(ws.device),
                                                         ctypes.byref(host)))
    return int(host.value)


# ---------------------------------------------------------------------------
# What earlier calls found out about the data
# ---------------------------------------------------------------------------
# Without help the library decides on the device which kernel instantiations the data calls
# for (separable grid or not, narrow gaussians or not) and launches all candidates; those
# not chosen return at once.  The facts end up in the workspace's status words.  Here they
# are read back without blocking (a 32-byte copy into pinned memory plus an event, picked up
# by a later call once the event has completed; only the very first call on a device and
# gaussian count nothing is known about waits for its own answer, see _queue_read) and
# remembered, so that later calls pass hints and launch only what will run:
#   * per (device, B, N, H, W): whether at least one gaussian in eight is narrow -- looked at
#     during the first calls and every 32nd after that; "not narrow" becomes
#     HINT_WIDE_GAUSSIANS, "narrow" lets the set_backward_sort policy order the gaussians.
#     A stale answer costs time only: the plain kernels are correct for any data.
#   * per pair of grid tensors (the very same tensor objects, unmodified: weak references
#     and torch's version counters): whether the library's device check found them
#     separable.  If so, later calls hand the library stride-0 views (first row of x, first
#     column of y), which are separable by construction; if not, HINT_GENERAL_GRID.
#   * word 0, a kernel that gave up on a bounded wait: raised as IgsError by the next call.
_memo_lock = threading.Lock()
_pending = []       # reads in flight: _PendingRead
_free_hosts = []    # pinned int32[STATUS_WORDS] buffers to reuse
_shape_memos = {}   # (device index, B, N, H, W) -> _ShapeMemo
_family_narrow = {}  # (device index, B, N) -> the latest answer any image size gave
_grid_memos = {}    # (id(x), id(y)) -> _GridMemo
GRID_CHECKED_BIT = 8
GRID_NOT_SEPARABLE_BIT = 1


class _ShapeMemo:
    EVERY = 32  # after the first few calls, look again every this many

    __slots__ = ("total", "narrow", "calls", "pending", "family")

    def __init__(self, total, family=None):
        self.total = total
        self.narrow = None  # unknown until the first read has come back
        self.calls = 0
        self.pending = False
        self.family = family  # (device index, B, N): the same gaussians at any image size


class _GridMemo:
    __slots__ = ("xref", "yref", "xv", "yv", "kind", "pending", "views")

    def __init__(self, x, y):
        self.xref, self.yref = weakref.ref(x), weakref.ref(y)
        self.xv, self.yv = x._version, y._version
        self.kind = None  # None = not known yet; "separable", "general", "unchecked"
        self.pending = False
        self.views = None  # (B, x3, y3) handed out last time, for the kind that is known

    def matches(self, x, y):
        return self.xref() is x and self.yref() is y and self.xv == x._version and self.yv == y._version


class _PendingRead:
    __slots__ = ("host", "event", "shape", "grid")


def _drain_reads():
    """Folds every status read whose copy has completed into the memos."""
    if not _pending or torch.cuda.is_current_stream_capturing():
        return
    failed = False
    with _memo_lock:
        keep = []
        for r in _pending:
            if not r.event.query():
                keep.append(r)
                continue
            words = r.host.tolist()
            _free_hosts.append(r.host)
            failed |= words[0] != 0
            if r.shape is not None:
                r.shape.pending = False
                r.shape.narrow = words[2] * 8 >= r.shape.total
                if r.shape.family is not None:
                    _family_narrow[r.shape.family] = r.shape.narrow
            if r.grid is not None:
                r.grid.pending = False
                if r.grid.kind is None:
                    if words[1] & GRID_CHECKED_BIT:
                        r.grid.kind = "general" if words[1] & GRID_NOT_SEPARABLE_BIT else "separable"
                    else:
                        r.grid.kind = "unchecked"  # the call did not have to look: nothing learnt
        _pending[:] = keep
    if failed:
        raise IgsError("igs_read_status_words", -5, "an earlier call's kernel gave up on a bounded wait; its result "
                                                    "is invalid")


def _queue_read(ws, shape, grid):
    """After a forward / backward on workspace ws: queue a status read if a memo wants one."""
    if shape is not None:
        shape.calls += 1
    want_shape = shape is not None and not shape.pending and (shape.calls <= 4 or shape.calls % shape.EVERY == 0)
    want_grid = grid is not None and grid.kind is None and not grid.pending
    if not (want_shape or want_grid) or torch.cuda.is_current_stream_capturing():
        return
    dev = ws.device
    with _memo_lock:
        host = _free_hosts.pop() if _free_hosts else torch.zeros(STATUS_WORDS, dtype=torch.int32, pin_memory=True)
        r = _PendingRead()
        r.host, r.shape, r.grid = host, (shape if want_shape else None), (grid if want_grid else None)
        check("igs_read_status_words",
              load().igs_read_status_words(_ptr(ws), dev.index, _stream(dev), ctypes.c_void_p(host.data_ptr())))
        r.event = torch.cuda.Event()
        r.event.record(torch.cuda.current_stream(dev))
        if want_shape:
            shape.pending = True
        if want_grid:
            grid.pending = True
        _pending.append(r)
        first_look = want_shape and shape.narrow is None
    if first_look:
        # The very first call on gaussians nothing is known about: wait for its answer (the one
        # place the call layer blocks, once per device and gaussian count).  A loop issues steps
        # far faster than the device runs the unordered kernels on narrow gaussians, so without
        # the wait dozens of such steps are queued before the answer to the first one arrives:
        # measured, 16384 narrow gaussians at 1024 x 1024, the first 27 steps at 8 ms each
        # instead of 0.5 ms.
        r.event.synchronize()
        _drain_reads()


def _shape_memo(dev, B, N, H, W):
    key = (dev.index, B, N, H, W)
    m = _shape_memos.get(key)
    if m is None:
        if len(_shape_memos) > 256:
            _shape_memos.clear()
        # Whether gaussians are narrow is judged against the sampled extent, not against the
        # pixel count, so a new image size starts from what the same number of gaussians showed
        # at the last one (a fit that moves up its resolution schedule keeps its ordered kernels
        # instead of running the first steps of every size without an order).  A guess: the
        # first reads of the new shape confirm or correct it, and it only ever costs time.
        family = (dev.index, B, N)
        m = _shape_memos[key] = _ShapeMemo(B * N, family)
        m.narrow = _family_narrow.get(family)
    return m


def forget_what_calls_learnt() -> None:
    """Drops every remembered fact (tests; after changing the culling switch)."""
    with _memo_lock:
        _shape_memos.clear()
        _family_narrow.clear()
        _grid_memos.clear()


def grid_for_call(x, y, B):
    """x, y [B,1,H,W] or [1,1,H,W] -> (x3, y3, hints, memo): [B,H,W] views without a copy,
    the grid part of the call's hints, and the memo entry that wants to learn from this call
    (or None).  Grids remembered as separable come back as stride-0 views."""
    if x.dim() != 4 or y.dim() != 4 or x.shape[1] != 1 or y.shape[1] != 1:
        raise ValueError(f"x and y must be [B,1,H,W]; got {tuple(x.shape)} and {tuple(y.shape)}")
    if x.shape != y.shape:
        raise ValueError(f"x {tuple(x.shape)} and y {tuple(y.shape)} differ")
    if x.shape[0] not in (B, 1):
        raise ValueError(f"x/y batch {x.shape[0]} does not match the gaussians' batch {B}")
    H, W = x.shape[2], x.shape[3]
    key = (id(x), id(y))
    entry = _grid_memos.get(key)
    if entry is not None and entry.matches(x, y) and entry.kind in ("separable", "general"):
        v = entry.views
        if v is None or v[0] != B:
            v = entry.views = (B, *grid_views(x, y, B, entry.kind == "separable"))
        return v[1], v[2], (HINT_GENERAL_GRID if entry.kind == "general" else 0), None
    x3, y3 = x[:, 0].expand(B, H, W), y[:, 0].expand(B, H, W)
    if H < 4 or W < 16 or ((x3.stride(1) == 0 or H == 1) and (y3.stride(2) == 0 or W == 1)):
        return x3, y3, 0, None  # tiny, or separable by construction: the library needs no help
    if entry is None or not entry.matches(x, y):
        if torch.cuda.is_current_stream_capturing():
            return x3, y3, 0, None
        with _memo_lock:
            # forget grids that are gone (their entries hold views, i.e. device memory)
            for k in [k for k, e in _grid_memos.items() if e.xref() is None or e.yref() is None]:
                del _grid_memos[k]
            if len(_grid_memos) > 64:
                _grid_memos.clear()
            entry = _grid_memos[key] = _GridMemo(x, y)
        return x3, y3, 0, entry
    return x3, y3, 0, (entry if entry.kind is None else None)


def grid_views(x, y, B, as_separable=False):
    """[B,1,H,W] (or [1,1,H,W]) sample coordinates -> [B,H,W] views, no copy; as_separable:
    the stride-0 views of a grid known to be separable (first row of x, first column of y)."""
    H, W = x.shape[2], x.shape[3]
    if as_separable:
        return x[:, 0, :1].expand(B, H, W), y[:, 0, :, :1].expand(B, H, W)
    return x[:, 0].expand(B, H, W), y[:, 0].expand(B, H, W)


class CallInfo:
    """What one forward decided, kept for its backward: the grid views, the hints, the
    processing order, and the memos that learn from the call."""
    __slots__ = ("x3", "y3", "hints", "order", "shape", "grid")


KEEP_ORDER = "keep"  # prepare_call(order=...): use the caller's order, or none at all, instead of the policy's


def prepare_call(x, y, pos, feat=None, pos_off=None, scales=None, log_scales=False, rotations=None, order=None):
    """Everything a forward (and the backward after it) needs beyond the tensors: grid views,
    hints from what earlier calls learnt, and the processing order the set_backward_sort
    policy wants, if any.  pos [B,N,2], or None with feat [B,N,6+C] (+ pos_off); scales
    [B,N,2] and rotations [B,N] when the caller has them.  order: None = by the policy; a
    (KEEP_ORDER, tensor or None) pair = exactly that order, e.g. one kept from an earlier step."""
    _drain_reads()
    B, N = (pos if pos is not None else feat).shape[:2]
    info = CallInfo()
    info.x3, info.y3, info.hints, info.grid = grid_for_call(x, y, B)
    _, H, W = info.x3.shape
    info.shape = _shape_memo(x.device, B, N, H, W) if B * N * H * W > 0 else None
    info.order = None
    if info.shape is not None:
        if info.shape.narrow is False and _BACKWARD_SORT != "on":
            info.hints |= HINT_WIDE_GAUSSIANS
        if order is not None and order[0] == KEEP_ORDER:
            info.order = order[1]
        else:
            info.order = order_by_policy(info.shape, pos, feat, pos_off, info.x3, info.y3, scales, log_scales,
                                         rotations)
    return info


def forward(kind, pos, s0, s1, s2, alphas, colors, x3, y3, eps, normalize=True, keep_workspace=False, order=None,
            hints=0, info=None):
    """kind 'sr': s0 = scales, s1 = rotations; kind 'cov': s0, s1, s2 = cov_inv_00/01/11.
    x3, y3 are [B,H,W] views (any strides).  Returns (out, wsum) or, with
    normalize=False, (sums [B,C+1,H,W], None).  order: [B,N] int32 permutation in which the
    gaussians are summed, or None.  info: a CallInfo whose memos learn from this call."""
    dev = pos.device
    B, N, C = colors.shape
    _, H, W = x3.shape
    fb, _ = workspace_bytes(B, N, H, W, C, dev)
    ws = _workspace(fb, dev)
    if normalize:
        out = torch.empty(B, C, H, W, dtype=torch.float32, device=dev)
        wsum = torch.empty(B, H, W, dtype=torch.float32, device=dev)
    else:
        out = torch.empty(B, C + 1, H, W, dtype=torch.float32, device=dev)
        wsum = None
    tail = (_ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), B, N, H, W, C, float(eps), int(bool(normalize)),
            _ptr(out), _ptr(wsum), _ptr(order), int(hints), _ptr(ws), ws.numel(), dev.index, _stream(dev))
    lib = load()
    if kind == "sr":
        check("igs_forward_sr", lib.igs_forward_sr(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(alphas), _ptr(colors), *tail))
    else:
        check("igs_forward_cov",
              lib.igs_forward_cov(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(s2), _ptr(alphas), _ptr(colors), *tail))
    if info is not None and N > 0:
        _queue_read(ws, info.shape, info.grid)
    if keep_workspace:
        return out, wsum, ws
    return out, wsum


def forward_feature(feat, pos_off, x3, y3, eps, order=None, keep_workspace=False, hints=0, info=None):
    """The forward on the module's projection output feat [B,N,6+C] (contiguous); pos_off
    [B,N,2] or None.  Returns (out, wsum)."""
    dev = feat.device
    B, N, per = feat.shape
    C = per - 6
    _, H, W = x3.shape
    fb, _ = workspace_bytes(B, N, H, W, C, dev)
    ws = _workspace(fb, dev)
    out = torch.empty(B, C, H, W, dtype=torch.float32, device=dev)
    wsum = torch.empty(B, H, W, dtype=torch.float32, device=dev)
    check("igs_forward_feature",
          load().igs_forward_feature(_ptr(feat), _ptr(pos_off), _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), B, N,
                                     H, W, C, float(eps), 1, _ptr(out), _ptr(wsum), _ptr(order), int(hints), _ptr(ws),
                                     ws.numel(), dev.index, _stream(dev)))
    if info is not None and N > 0:
        _queue_read(ws, info.shape, info.grid)
    if keep_workspace:
        return out, wsum, ws
    return out, wsum


def backward_feature(feat, pos_off, x3, y3, wsum, out, gout, eps, grad_mode, order=None, hints=0, info=None):
    """Gradient with respect to feat, [B,N,6+C] (the unused column gets zeros)."""
    dev = feat.device
    B, N, per = feat.shape
    C = per - 6
    _, H, W = x3.shape
    _, bb = workspace_bytes(B, N, H, W, C, dev)
    ws = _workspace(bb, dev)
    d_feat = torch.empty_like(feat)
    check("igs_backward_feature",
          load().igs_backward_feature(_ptr(feat), _ptr(pos_off), _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3),
                                      _ptr(wsum), _ptr(out), _ptr(gout), B, N, H, W, C, float(eps), int(grad_mode),
                                      _ptr(d_feat), _ptr(order), int(hints), _ptr(ws), ws.numel(), dev.index,
                                      _stream(dev)))
    if info is not None and N > 0 and H * W > 0:
        _queue_read(ws, info.shape, None)
    return d_feat


def normalize(sums: torch.Tensor, eps: float):
    """sums [B,C+1,H,W] -> (out [B,C,H,W], wsum [B,H,W])."""
    dev = sums.device
    B, C1, H, W = sums.shape
    out = torch.empty(B, C1 - 1, H, W, dtype=torch.float32, device=dev)
    wsum = torch.empty(B, H, W, dtype=torch.float32, device=dev)
    check("igs_normalize", load().igs_normalize(_ptr(sums), B, H, W, C1 - 1, float(eps), _ptr(out), _ptr(wsum),
                                                 dev.index, _stream(dev)))
    return out, wsum


def spatial_order(pos, x3, y3):
    """[B,N] int32 permutation putting spatial neighbours next to each other (the `order`
    argument of the forward and the backward)."""
    dev = pos.device
    B, N, _ = pos.shape
    _, H, W = x3.shape
    lib = load()
    ws = _workspace(int(lib.igs_spatial_order_workspace_bytes(B, N)), dev)
    order = torch.empty(B, N, dtype=torch.int32, device=dev)
    check("igs_spatial_order",
          lib.igs_spatial_order(_ptr(pos), _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), B, N, H, W, _ptr(order),
                                _ptr(ws), ws.numel(), dev.index, _stream(dev)))
    return order


def _rows(t, width):
    """(tensor to keep alive, floats from one gaussian's entry to the next) for reading `width`
    consecutive floats per gaussian where they lie: a slice t = full[..., a:a+width] (or
    full[..., a]) of a contiguous [B,N,K] tensor is taken in place, anything else is made
    contiguous first."""
    B, N = t.shape[:2]
    st = t.stride()
    inner_ok = t.dim() == 2 or st[2] == 1
    if inner_ok and (N <= 1 or st[1] >= width) and (B <= 1 or st[0] == N * st[1]):
        return t, (st[1] if N > 1 else width)
    return t.contiguous(), width


def spatial_order_boxes(pos, x3, y3, scales=None, log_scales=False, rotations=None, pos_off=None):
    """[B,N] int32 permutation along the Hilbert curve of, per gaussian, the centre of its
    zero-weight box clipped to the sampled extent (igs_spatial_order_boxes): pos [B,N,2],
    scales [B,N,2] (their logarithms with log_scales), rotations [B,N] or None (then the larger
    scale stands in for both axes), pos_off [B,N,2] or None (added to pos).  The tensors may be
    slices of one [B,N,K] tensor; they are read in place."""
    dev = pos.device
    B, N, _ = pos.shape
    _, H, W = x3.shape
    lib = load()
    ws = _workspace(int(lib.igs_spatial_order_workspace_bytes(B, N)), dev)
    order = torch.empty(B, N, dtype=torch.int32, device=dev)
    pos, ps = _rows(pos.detach(), 2)
    sc, ss = _rows(scales.detach(), 2) if scales is not None else (None, 2)
    rot, rs = _rows(rotations.detach(), 1) if rotations is not None and scales is not None else (None, 1)
    off = pos_off.detach().contiguous() if pos_off is not None else None
    check("igs_spatial_order_boxes",
          lib.igs_spatial_order_boxes(_ptr(pos), ps, _ptr(off), _ptr(sc), ss, 1 if log_scales else 0, _ptr(rot), rs,
                                      _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), B, N, H, W, _ptr(order),
                                      _ptr(ws), ws.numel(), dev.index, _stream(dev)))
    return order


_BACKWARD_SORT = "auto"
# Below this many gaussian x pixel pairs per call, "auto" does not order: the four extra
# launches cost an eager step more host time than the skipping saves on the device
# (measured: 2.7e8 pairs, 4096 gaussians at 256x256: 0.50 ms ordered against 0.44 ms; 1.1e9
# pairs, 4096 at 512x512: 0.42 against 0.88 ms).
AUTO_ORDER_MIN_EVALS = 5e8


def set_backward_sort(mode: str) -> None:
    """'auto' (default): forward and backward take their gaussians in spatial order once the
    shape's recent calls have shown mostly narrow gaussians; 'on' / 'off': always / never.
    The gradients are the same bit for bit in every mode; only the time differs."""
    global _BACKWARD_SORT
    if mode not in ("auto", "on", "off"):
        raise ValueError("mode must be 'auto', 'on' or 'off'")
    _BACKWARD_SORT = mode
    forget_what_calls_learnt()


def order_by_policy(shape, pos, feat, pos_off, x3, y3, scales=None, log_scales=False, rotations=None):
    """The processing order one forward + backward should use under the set_backward_sort
    policy, or None.  shape: the call's _ShapeMemo; pos [B,N,2], or None with feat
    [B,N,6+C] (+ pos_off) to take the positions from; scales [B,N,2] if at hand (lets the
    order keep wide and narrow gaussians apart)."""
    B, N = (pos if pos is not None else feat).shape[:2]
    _, H, W = x3.shape
    if B * N == 0 or _BACKWARD_SORT == "off":
        return None
    if _BACKWARD_SORT == "auto":
        if not shape.narrow:
            return None
        # small problems: ordering costs an eager step more on the host than it saves on the
        # device; inside a graph capture the host cost is paid once, so there it always pays
        if B * N * H * W < AUTO_ORDER_MIN_EVALS and not torch.cuda.is_current_stream_capturing():
            return None
    if pos is None:
        return spatial_order_boxes(feat[..., :2], x3, y3, feat[..., 2:4], True, feat[..., 4], pos_off)
    return spatial_order_boxes(pos, x3, y3, scales, log_scales, rotations if scales is not None else None)


def backward(kind, pos, s0, s1, s2, alphas, colors, x3, y3, wsum, out, gout, eps, grad_mode, want_xy,
             keep_workspace=False, order=None, hints=0, info=None):
    """Returns dict of gradients; d_x / d_y only when want_xy.  order: an explicit [B,N] int32
    permutation or None."""
    dev = pos.device
    B, N, C = colors.shape
    _, H, W = x3.shape
    _, bb = workspace_bytes(B, N, H, W, C, dev)
    ws = _workspace(bb, dev)
    f32 = dict(dtype=torch.float32, device=dev)
    d_pos = torch.empty(B, N, 2, **f32)
    d_alpha = torch.empty(B, N, **f32)
    d_col = torch.empty(B, N, C, **f32)
    d_x = torch.empty(B, H, W, **f32) if want_xy else None
    d_y = torch.empty(B, H, W, **f32) if want_xy else None
    head = (_ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), _ptr(wsum), _ptr(out), _ptr(gout), B, N, H, W, C,
            float(eps), int(grad_mode))
    tail = (_ptr(d_alpha), _ptr(d_col), _ptr(d_x), _ptr(d_y), _ptr(order), int(hints), _ptr(ws), ws.numel(),
            dev.index, _stream(dev))
    lib = load()
    if kind == "sr":
        d_s0 = torch.empty(B, N, 2, **f32)
        d_s1 = torch.empty(B, N, **f32)
        check("igs_backward_sr",
              lib.igs_backward_sr(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(alphas), _ptr(colors), *head, _ptr(d_pos),
                                  _ptr(d_s0), _ptr(d_s1), *tail))
        res = {"positions": d_pos, "scales": d_s0, "rotations": d_s1, "alphas": d_alpha, "colors": d_col}
    else:
        d_s0, d_s1, d_s2 = (torch.empty(B, N, **f32) for _ in range(3))
        check("igs_backward_cov",
              lib.igs_backward_cov(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(s2), _ptr(alphas), _ptr(colors), *head,
                                   _ptr(d_pos), _ptr(d_s0), _ptr(d_s1), _ptr(d_s2), *tail))
        res = {"positions": d_pos, "c00": d_s0, "c01": d_s1, "c11": d_s2, "alphas": d_alpha, "colors": d_col}
    if info is not None and N > 0 and H * W > 0:
        _queue_read(ws, info.shape, None)
    if want_xy:
        res["x"], res["y"] = d_x, d_y
    if keep_workspace:
        res["_workspace"] = ws
    return res


@functools.lru_cache(maxsize=256)
def _render_mse_workspace_bytes(B, N, H, W, C, index):
    n = _sz(0)
    check("igs_render_mse_workspace_bytes", load().igs_render_mse_workspace_bytes(B, N, H, W, C, index, ctypes.byref(n)))
    return int(n.value)


def render_mse(pos, scales, rot, alphas, colors, x3, y3, target, eps, grad_mode, log_scales=False, upstream=None,
               want_image=False, order=None, hints=0, info=None):
    """Render + mean-squared-error loss + all gradients in one library call
    (igs_render_mse_sr).  Returns (loss, gradients, image or None); gradients keyed
    positions, scales (of the log-scales when log_scales), rotations, colors and, when alphas
    is given, alphas.  alphas None = all ones."""
    dev = pos.device
    B, N, C = colors.shape
    _, H, W = x3.shape
    ws = _workspace(_render_mse_workspace_bytes(B, N, H, W, C, dev.index), dev)
    f32 = dict(dtype=torch.float32, device=dev)
    loss = torch.empty((), **f32)
    image = torch.empty(B, C, H, W, **f32) if want_image else None
    g = {"positions": torch.empty(B, N, 2, **f32), "scales": torch.empty(B, N, 2, **f32),
         "rotations": torch.empty(B, N, **f32), "colors": torch.empty(B, N, C, **f32)}
    if alphas is not None:
        g["alphas"] = torch.empty(B, N, **f32)
    check("igs_render_mse_sr",
          load().igs_render_mse_sr(_ptr(pos), _ptr(scales), _ptr(rot), _ptr(alphas), _ptr(colors), int(bool(log_scales)),
                                   _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3), _ptr(target), B, N, H, W, C,
                                   float(eps), int(grad_mode), _ptr(upstream), _ptr(loss), _ptr(image),
                                   _ptr(g["positions"]), _ptr(g["scales"]), _ptr(g["rotations"]), _ptr(g.get("alphas")),
                                   _ptr(g["colors"]), _ptr(order), int(hints), _ptr(ws), ws.numel(), dev.index,
                                   _stream(dev)))
    if info is not None:
        _queue_read(ws, info.shape, info.grid)
    return loss, g, image


MSE_WORKSPACE_BYTES = 4096


def mse_loss(out: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """mean((out - target)^2) as a device scalar; both contiguous fp32 of one shape."""
    dev = out.device
    loss = torch.empty((), dtype=torch.float32, device=dev)
    ws = _workspace(MSE_WORKSPACE_BYTES, dev)
    check("igs_mse_loss", load().igs_mse_loss(_ptr(out), _ptr(target), out.numel(), _ptr(loss), _ptr(ws), ws.numel(),
                                              dev.index, _stream(dev)))
    return loss


def mse_grad(out: torch.Tensor, target: torch.Tensor, upstream: torch.Tensor | None) -> torch.Tensor:
    """upstream * 2 (out - target) / n, shaped like out; upstream a device scalar or None."""
    dev = out.device
    gout = torch.empty_like(out)
    check("igs_mse_grad", load().igs_mse_grad(_ptr(out), _ptr(target), out.numel(), _ptr(upstream), _ptr(gout),
                                              dev.index, _stream(dev)))
    return gout


KERNEL_NAMES = ("pack", "forward", "reduce_normalize", "pixel_terms", "backward", "finalize", "coord_grad", "grid_check")


def set_culling(on: bool) -> None:
    """Process-wide switch of the lossless (gaussian, pixel tile) culling; default on."""
    check("igs_set_culling", load().igs_set_culling(int(bool(on))))
    forget_what_calls_learnt()


def profile_enable(on) -> None:
    """False / 0: off; True / 1: every kernel; 2: the forward and backward splat kernels only."""
    check("igs_profile_enable", load().igs_profile_enable(int(on)))


def profile_reset() -> None:
    check("igs_profile_reset", load().igs_profile_reset())


def profile_read():
    """{kernel name: (total device ms, launches)} since the last reset."""
    res = {}
    for k, name in enumerate(KERNEL_NAMES):
        ms, n = ctypes.c_double(0), ctypes.c_longlong(0)
        check("igs_profile_read", load().igs_profile_read(k, ctypes.byref(ms), ctypes.byref(n)))
        res[name] = (ms.value, int(n.value))
    return res
