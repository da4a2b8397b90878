"""Roofline denominators measured on the GPU at hand: issue rates of the FP32 FMA pipe
(scalar FFMA, packed f32x2 FMA, and the splat kernels' FMA : ex2 mixes with every
dependency removed) and of the MUFU ex2 unit.

Bench tooling, kept out of the splat library: ``probe.cu`` builds into its own
``libigs_probes.so`` (``build()``), which ``bench.py`` loads through ``rates()``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

from .. import build as _lib_build

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCE = os.path.join(HERE, "probe.cu")
LIB_PATH = os.path.join(HERE, "libigs_probes.so")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [SOURCE, os.path.join(_lib_build.CSRC, "common.cuh"), os.path.join(_lib_build.INCLUDE, "igs_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False) -> str:
    """nvcc, sm_100a, same flags as the splat library."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_lib_build._nvcc(), *_lib_build.NVCC_FLAGS, "-I", _lib_build.INCLUDE, "-o", LIB_PATH, SOURCE]
    if os.path.exists("/usr/bin/g++"):
        cmd[1:1] = ["-ccbin", "/usr/bin/g++"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + (res.stdout + res.stderr)[-4000:])
    return LIB_PATH


def rates(device_index: int) -> dict:
    """Measured rates on one device: lane-instructions per second of the FMA pipe (scalar,
    packed with shared operands, packed with three distinct register operands, forward mix
    11 FMA : 2 ex2, backward mix 22 : 2) and ex2 results per second."""
    lib = ctypes.CDLL(build())
    dbl = ctypes.POINTER(ctypes.c_double)
    lib.igs_probe_fp32_rate.argtypes = [ctypes.c_int, ctypes.c_int, dbl]
    lib.igs_probe_mix_rate.argtypes = [ctypes.c_int, ctypes.c_int, dbl]
    lib.igs_probe_ex2_rate.argtypes = [ctypes.c_int, dbl]

    def call(fn, *args):
        d = ctypes.c_double(0)
        rc = fn(*args, ctypes.byref(d))
        if rc != 0:
            raise RuntimeError(f"{fn.__name__} failed with code {rc}")
        return d.value

    return {
        "fp32_scalar_lane_instr_per_s": call(lib.igs_probe_fp32_rate, device_index, 0),
        "fp32_packed_lane_instr_per_s": call(lib.igs_probe_fp32_rate, device_index, 1),
        # f32x2 FMAs with three different register operands each (what an accumulation a*b + v
        # is): the register file, not the pipe, sets this rate
        "fp32_packed_3operand_lane_instr_per_s": call(lib.igs_probe_fp32_rate, device_index, 2),
        "ex2_results_per_s": call(lib.igs_probe_ex2_rate, device_index),
        "fp32_forward_mix_lane_instr_per_s": call(lib.igs_probe_mix_rate, device_index, 0),
        "fp32_backward_mix_lane_instr_per_s": call(lib.igs_probe_mix_rate, device_index, 1),
    }
