"""numpy front-end of the CPU oracle (``liboracle.so`` built from splat_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and
by the CPU-baseline leg of ``bench.py`` as the checker.  The product package never
imports it.

The functions mirror the reference's call chain
(``src/igs/gs2d.py``: ``render`` :524-609 -> ``GaussianSplatting2DChunkedKernel``
:265-465) with plain contiguous arrays:

    x, y [B,H,W]; positions [B,N,2]; colors [B,N,C]; scales [B,N,2];
    rotations [B,N]; alphas [B,N]; cov_inv_xx [B,N]; out/gout [B,C,H,W]

``dtype=np.float32`` computes in the reference's arithmetic type, ``np.float64``
is the ground truth evaluated from the same inputs.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

MODE_REFERENCE = 0  # gS = -sum_c g_c^2 / S^2   (src/igs/gs2d.py:370)
MODE_EXACT = 1      # gS = -sum_c gn_c * out_c  (autograd of src/igs/gs2d.py:24-44)


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file; returns its path."""
    so = os.path.join(_HERE, "liboracle.so")
    srcs = [os.path.join(_HERE, f) for f in ("splat_oracle.c", "splat_oracle_impl.h", "Makefile")]
    stale = (not os.path.exists(so)) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in srcs)
    if force or stale:
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.oracle_num_threads.restype = ctypes.c_int
    return _LIB


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def _suffix(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle computes in float32 or float64, not {dtype}")


def _arr(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a), dtype=dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _real(v, dtype):
    return ctypes.c_float(v) if np.dtype(dtype) == np.float32 else ctypes.c_double(v)


def cov_inv(scales, rotations, eps=1e-6, dtype=np.float32):
    """scales [...,2], rotations [...] -> (c00, c01, c11), each shaped like rotations."""
    sc, rt = _arr(scales, dtype), _arr(rotations, dtype)
    m = rt.size
    outs = [np.empty(rt.shape, dtype) for _ in range(3)]
    fn = getattr(lib(), f"oracle_cov_inv_{_suffix(dtype)}")
    fn(_ptr(sc), _ptr(rt), _real(eps, dtype), ctypes.c_int64(m), *[_ptr(o) for o in outs])
    return tuple(outs)


def cov_inv_backward(scales, rotations, g00, g01, g11, eps=1e-6, dtype=np.float32):
    """Chain d(cov_inv entries) back to (d_scales, d_rotations)."""
    sc, rt = _arr(scales, dtype), _arr(rotations, dtype)
    g = [_arr(v, dtype).reshape(rt.shape) for v in (g00, g01, g11)]
    gs, gr = np.empty(sc.shape, dtype), np.empty(rt.shape, dtype)
    fn = getattr(lib(), f"oracle_cov_inv_backward_{_suffix(dtype)}")
    fn(_ptr(sc), _ptr(rt), _real(eps, dtype), ctypes.c_int64(rt.size), *[_ptr(v) for v in g],
       _ptr(gs), _ptr(gr))
    return gs, gr


def _dims(x, positions, colors):
    B, H, W = x.shape
    N = positions.shape[1]
    C = colors.shape[2]
    return B, N, H, W, C


def forward(x, y, positions, c00, c01, c11, alphas, colors, eps=1e-6, dtype=np.float32):
    """Returns (out [B,C,H,W], wsum [B,H,W]); wsum is the weight sum without eps."""
    x, y = _arr(x, dtype), _arr(y, dtype)
    if x.ndim == 4:
        x, y = x[:, 0], y[:, 0]
    x, y = np.ascontiguousarray(x), np.ascontiguousarray(y)
    pos, col, al = _arr(positions, dtype), _arr(colors, dtype), _arr(alphas, dtype)
    B, N, H, W, C = _dims(x, pos, col)
    cs = [_arr(c, dtype).reshape(B, N) for c in (c00, c01, c11)]
    out = np.zeros((B, C, H, W), dtype)
    wsum = np.zeros((B, H, W), dtype)
    fn = getattr(lib(), f"oracle_forward_{_suffix(dtype)}")
    fn(_ptr(x), _ptr(y), _ptr(pos), *[_ptr(c) for c in cs], _ptr(al), _ptr(col), _real(eps, dtype),
       *[ctypes.c_int(v) for v in (B, N, H, W, C)], _ptr(out), _ptr(wsum))
    return out, wsum


def backward(x, y, positions, c00, c01, c11, alphas, colors, wsum, out, gout, eps=1e-6,
             mode=MODE_REFERENCE, want_xy=True, dtype=np.float32):
    """Returns a dict with x, y, positions, c00, c01, c11, alphas, colors gradients."""
    x, y = _arr(x, dtype), _arr(y, dtype)
    if x.ndim == 4:
        x, y = x[:, 0], y[:, 0]
    x, y = np.ascontiguousarray(x), np.ascontiguousarray(y)
    pos, col, al = _arr(positions, dtype), _arr(colors, dtype), _arr(alphas, dtype)
    B, N, H, W, C = _dims(x, pos, col)
    cs = [_arr(c, dtype).reshape(B, N) for c in (c00, c01, c11)]
    wsum, out, gout = _arr(wsum, dtype), _arr(out, dtype), _arr(gout, dtype)
    gx = np.zeros((B, H, W), dtype) if want_xy else None
    gy = np.zeros((B, H, W), dtype) if want_xy else None
    gpos = np.zeros((B, N, 2), dtype)
    g00, g01, g11, gal = (np.zeros((B, N), dtype) for _ in range(4))
    gcol = np.zeros((B, N, C), dtype)
    fn = getattr(lib(), f"oracle_backward_{_suffix(dtype)}")
    fn(_ptr(x), _ptr(y), _ptr(pos), *[_ptr(c) for c in cs], _ptr(al), _ptr(col), _ptr(wsum),
       _ptr(out), _ptr(gout), _real(eps, dtype), ctypes.c_int(int(mode)),
       *[ctypes.c_int(v) for v in (B, N, H, W, C)], _ptr(gx), _ptr(gy), _ptr(gpos), _ptr(g00),
       _ptr(g01), _ptr(g11), _ptr(gal), _ptr(gcol))
    return {"x": gx, "y": gy, "positions": gpos, "c00": g00, "c01": g01, "c11": g11,
            "alphas": gal, "colors": gcol}


def render(positions, colors, scales, rotations, alphas, x, y, eps=1e-6, dtype=np.float32):
    """``gaussian_splatting_2d`` (src/igs/gs2d.py:524-596, fused branch): image only."""
    c00, c01, c11 = cov_inv(scales, rotations, eps, dtype)
    return forward(x, y, positions, c00, c01, c11, alphas, colors, eps, dtype)


def render_with_grads(positions, colors, scales, rotations, alphas, x, y, gout_fn, eps=1e-6,
                      mode=MODE_REFERENCE, want_xy=False, dtype=np.float32):
    """Forward, upstream gradient ``gout_fn(out) -> d loss / d out``, backward.

    Returns (out, wsum, grads) with grads keyed positions, colors, scales,
    rotations, alphas (and x, y when want_xy) -- what autograd hands back to a
    caller of the reference's ``gaussian_splatting_2d``.
    """
    c00, c01, c11 = cov_inv(scales, rotations, eps, dtype)
    out, wsum = forward(x, y, positions, c00, c01, c11, alphas, colors, eps, dtype)
    gout = np.asarray(gout_fn(out), dtype=dtype)
    g = backward(x, y, positions, c00, c01, c11, alphas, colors, wsum, out, gout, eps, mode,
                 want_xy, dtype)
    gs, gr = cov_inv_backward(scales, rotations, g["c00"], g["c01"], g["c11"], eps, dtype)
    grads = {"positions": g["positions"], "colors": g["colors"], "scales": gs, "rotations": gr,
             "alphas": g["alphas"]}
    if want_xy:
        grads["x"], grads["y"] = g["x"], g["y"]
    return out, wsum, grads
