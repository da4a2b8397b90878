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

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# IGS_B200_LIB: development override, a differently tuned build of the same library
LIB_PATH = os.environ.get("IGS_B200_LIB") or os.path.join(_HERE, "libigs_b200.so")

GRAD_REFERENCE = 0
GRAD_EXACT = 1

_lock = threading.Lock()
_lib = None

_F = ctypes.POINTER(ctypes.c_float)
_I64 = ctypes.POINTER(ctypes.c_int64)
_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/igs_b200.h one to one
SIGNATURES = {
    "igs_version": (_i, []),
    "igs_strerror": (ctypes.c_char_p, [_i]),
    "igs_launch_count": (ctypes.c_longlong, []),
    "igs_workspace_bytes": (_i, [_i] * 6 + [ctypes.POINTER(_sz)] * 2),
    "igs_forward_sr": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "igs_forward_cov": (_i, [_vp] * 7 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "igs_forward_sr_static": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _i, _vp]),
    "igs_normalize": (_i, [_vp] + [_i] * 4 + [_f, _vp, _vp, _i, _vp]),
    "igs_backward_sr": (_i, [_vp] * 6 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 9 + [_sz, _i, _vp]),
    "igs_backward_cov": (_i, [_vp] * 7 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 10 + [_sz, _i, _vp]),
    "igs_forward_feature": (_i, [_vp] * 3 + [_I64, _vp, _I64] + [_i] * 5 + [_f, _i, _vp, _vp, _vp, _vp, _sz, _i, _vp]),
    "igs_backward_feature": (_i, [_vp] * 3 + [_I64, _vp, _I64] + [_vp] * 3 + [_i] * 5 + [_f, _i] + [_vp] * 3
                             + [_sz, _i, _vp]),
    "igs_read_status": (_i, [_vp, _i, _vp, ctypes.POINTER(_i)]),
    "igs_set_culling": (_i, [_i]),
    "igs_spatial_order_workspace_bytes": (_sz, [_i, _i]),
    "igs_spatial_order": (_i, [_vp, _vp, _I64, _vp, _I64] + [_i] * 4 + [_vp, _vp, _sz, _i, _vp]),
    "igs_read_narrow_count": (_i, [_vp, _i, _vp, _vp]),
    "igs_read_executed": (_i, [_vp, _i, _vp, ctypes.POINTER(ctypes.c_ulonglong)]),
    "igs_mse_loss": (_i, [_vp, _vp, ctypes.c_longlong, _vp, _vp, _sz, _i, _vp]),
    "igs_mse_grad": (_i, [_vp, _vp, ctypes.c_longlong, _vp, _vp, _i, _vp]),
    "igs_profile_enable": (_i, [_i]),
    "igs_profile_reset": (_i, []),
    "igs_profile_read": (_i, [_i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_longlong)]),
    "igs_describe_plan": (_i, [_i] * 6 + [ctypes.POINTER(_i)] * 4),
    "igs_probe_fp32_rate": (_i, [_i, _i, ctypes.POINTER(ctypes.c_double)]),
    "igs_probe_ex2_rate": (_i, [_i, ctypes.POINTER(ctypes.c_double)]),
    "igs_probe_mix_rate": (_i, [_i, _i, ctypes.POINTER(ctypes.c_double)]),
}


class IgsError(RuntimeError):
    """A call into libigs_b200.so returned a non-zero code."""

    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} failed with code {code}: {msg}")
        self.code = code


def load() -> ctypes.CDLL:
    """Loads (building first if the source tree is newer) the shared object."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            try:
                from . import build as _build

                _build.build()
            except Exception as exc:  # noqa: BLE001 - surfaced verbatim below
                raise ImportError(
                    f"igs_b200: {LIB_PATH} is missing and could not be built ({exc}). "
                    "Run `python -m igs_b200.build`; there is no CPU or PyTorch fallback.") from exc
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                if os.environ.get("IGS_B200_LIB"):
                    continue  # an older development build without this entry point
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


def _stream(device: torch.device):
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


def forward(kind, pos, s0, s1, s2, alphas, colors, x3, y3, eps, normalize=True, keep_workspace=False, order=None):
    """kind 'sr': s0 = scales, s1 = rotations; kind 'cov': s0, s1, s2 = cov_inv_00/01/11.
    x3, y3 are [B,H,W] views (any strides).  Returns (out, wsum) or, with
    normalize=False, (sums [B,C+1,H,W], None).  order: [B,N] int32 permutation in which the
    gaussians are summed, or None."""
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
            _ptr(out), _ptr(wsum), _ptr(order), _ptr(ws), ws.numel(), dev.index, _stream(dev))
    lib = load()
    if kind == "sr":
        check("igs_forward_sr", lib.igs_forward_sr(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(alphas), _ptr(colors), *tail))
    else:
        check("igs_forward_cov",
              lib.igs_forward_cov(_ptr(pos), _ptr(s0), _ptr(s1), _ptr(s2), _ptr(alphas), _ptr(colors), *tail))
    if keep_workspace:
        return out, wsum, ws
    return out, wsum


def forward_feature(feat, pos_off, x3, y3, eps, order=None, keep_workspace=False):
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
                                     H, W, C, float(eps), 1, _ptr(out), _ptr(wsum), _ptr(order), _ptr(ws), ws.numel(),
                                     dev.index, _stream(dev)))
    if keep_workspace:
        return out, wsum, ws
    return out, wsum


def backward_feature(feat, pos_off, x3, y3, wsum, out, gout, eps, grad_mode, order=None, policy=True):
    """Gradient with respect to feat, [B,N,6+C] (the unused column gets zeros).  order /
    policy as for backward()."""
    dev = feat.device
    B, N, per = feat.shape
    C = per - 6
    _, H, W = x3.shape
    probe = None
    if order is None and policy:
        order, probe = order_by_policy(None, feat, pos_off, x3, y3)
    _, bb = workspace_bytes(B, N, H, W, C, dev)
    ws = _workspace(bb, dev)
    d_feat = torch.empty_like(feat)
    check("igs_backward_feature",
          load().igs_backward_feature(_ptr(feat), _ptr(pos_off), _ptr(x3), _strides3(x3), _ptr(y3), _strides3(y3),
                                      _ptr(wsum), _ptr(out), _ptr(gout), B, N, H, W, C, float(eps), int(grad_mode),
                                      _ptr(d_feat), _ptr(order), _ptr(ws), ws.numel(), dev.index, _stream(dev)))
    if probe is not None:
        probe.queue(ws)
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
    argument of the backward)."""
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


class _NarrowProbe:
    """Host-side memory of whether a shape's gaussians were narrow at its recent backward
    calls, learnt without ever blocking: now and then a backward queues a copy of the
    device's narrow-gaussian count into pinned memory, and a later call picks the value up
    once the copy's event has completed."""

    EVERY = 32  # after the first few calls, look again every this many

    def __init__(self):
        self.host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        self.event = None
        self.calls = 0
        self.narrow = False

    def poll(self, total):
        if self.event is not None and not torch.cuda.is_current_stream_capturing() and self.event.query():
            self.narrow = int(self.host[0]) * 8 >= total
            self.event = None
        return self.narrow

    def queue(self, ws):
        self.calls += 1
        if self.event is not None or not (self.calls <= 4 or self.calls % self.EVERY == 0):
            return
        dev = ws.device
        if torch.cuda.is_current_stream_capturing():
            return
        check("igs_read_narrow_count",
              load().igs_read_narrow_count(_ptr(ws), dev.index, _stream(dev), ctypes.c_void_p(self.host.data_ptr())))
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(dev))


_BACKWARD_SORT = "auto"
_probes = {}
# Below this many gaussian x pixel pairs per call, "auto" does not order: the half dozen
# extra launches cost an eager step more host time than the skipping saves on the device
# (measured: 2.7e8 pairs, 4096 gaussians at 256x256: 0.61 ms ordered against 0.51 ms; 1.1e9
# pairs, 4096 at 512x512: 0.42 against 0.88 ms).
AUTO_ORDER_MIN_EVALS = 5e8


def set_backward_sort(mode: str) -> None:
    """'auto' (default): the backward takes its gaussians in spatial order once the shape's
    recent calls have shown mostly narrow gaussians; 'on' / 'off': always / never.  The
    gradients are the same bit for bit in every mode; only the time differs."""
    global _BACKWARD_SORT
    if mode not in ("auto", "on", "off"):
        raise ValueError("mode must be 'auto', 'on' or 'off'")
    _BACKWARD_SORT = mode
    _probes.clear()


def order_by_policy(pos, feat, pos_off, x3, y3):
    """(order or None, probe or None) for one forward / backward under the set_backward_sort
    policy.  pos [B,N,2], or None with feat [B,N,6+C] (+ pos_off) to take the positions
    from.  The caller hands the probe the workspace of a call it made (probe.queue(ws)), so
    that later calls learn how narrow the gaussians are."""
    B, N = (pos if pos is not None else feat).shape[:2]
    _, H, W = x3.shape
    if B * N == 0 or _BACKWARD_SORT == "off":
        return None, None
    dev = x3.device
    probe = None
    if _BACKWARD_SORT == "auto":
        probe = _probes.setdefault((dev.index, B, N, H, W), _NarrowProbe())
        if not probe.poll(B * N):
            return None, probe
        # small problems: ordering costs an eager step more on the host than it saves on the
        # device; inside a graph capture the host cost is paid once, so there it always pays
        if B * N * H * W < AUTO_ORDER_MIN_EVALS and not torch.cuda.is_current_stream_capturing():
            return None, probe
    if pos is None:
        pos = feat[..., :2] if pos_off is None else feat[..., :2] + pos_off
    return spatial_order(pos.contiguous(), x3, y3), probe


def backward(kind, pos, s0, s1, s2, alphas, colors, x3, y3, wsum, out, gout, eps, grad_mode, want_xy,
             keep_workspace=False, order=None, policy=True):
    """Returns dict of gradients; d_x / d_y only when want_xy.  order: an explicit [B,N] int32
    permutation, or None: then by the set_backward_sort policy if ``policy``, else none."""
    dev = pos.device
    B, N, C = colors.shape
    _, H, W = x3.shape
    probe = None
    if order is None and policy:
        order, probe = order_by_policy(pos, None, None, x3, y3)
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
    tail = (_ptr(d_alpha), _ptr(d_col), _ptr(d_x), _ptr(d_y), _ptr(order), _ptr(ws), ws.numel(), dev.index,
            _stream(dev))
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
    if probe is not None:
        probe.queue(ws)
    if want_xy:
        res["x"], res["y"] = d_x, d_y
    if keep_workspace:
        res["_workspace"] = ws
    return res


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


def profile_enable(on: bool) -> None:
    check("igs_profile_enable", load().igs_profile_enable(int(bool(on))))


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


def probe_rates(device: torch.device):
    """Measured issue rates of the FP32 FMA pipe (scalar, packed) and of MUFU ex2."""
    lib = load()
    vals = {}
    for key, packed in (("fp32_scalar_lane_instr_per_s", 0), ("fp32_packed_lane_instr_per_s", 1)):
        d = ctypes.c_double(0)
        check("igs_probe_fp32_rate", lib.igs_probe_fp32_rate(device.index, packed, ctypes.byref(d)))
        vals[key] = d.value
    d = ctypes.c_double(0)
    check("igs_probe_ex2_rate", lib.igs_probe_ex2_rate(device.index, ctypes.byref(d)))
    vals["ex2_results_per_s"] = d.value
    for key, bwd in (("fp32_forward_mix_lane_instr_per_s", 0), ("fp32_backward_mix_lane_instr_per_s", 1)):
        d = ctypes.c_double(0)
        check("igs_probe_mix_rate", lib.igs_probe_mix_rate(device.index, bwd, ctypes.byref(d)))
        vals[key] = d.value
    return vals
