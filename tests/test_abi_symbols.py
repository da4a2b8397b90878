"""The C-ABI library loads without a GPU and exports every function the header declares
(no compute calls here)."""
import ctypes
import os
import re

import pytest

from tests._util import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "igs_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(igs_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared()
    for must in ("igs_forward_sr", "igs_forward_cov", "igs_backward_sr", "igs_backward_cov", "igs_normalize",
                 "igs_workspace_bytes", "igs_strerror", "igs_version", "igs_launch_count", "igs_read_status"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from igs_b200 import _lib, build

    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in _declared():
        assert hasattr(lib, name), f"{name} declared in include/igs_b200.h but not exported"
    # and the Python binding declares a signature for each of them
    assert sorted(_lib.SIGNATURES) == _declared()


def test_error_strings_and_argument_errors_without_gpu():
    from igs_b200 import _lib

    lib = _lib.load()
    assert lib.igs_version() >= 100
    assert b"workspace" in lib.igs_strerror(-2)
    assert b"ok" == lib.igs_strerror(0)
    # argument validation happens before any CUDA call
    assert lib.igs_profile_read(99, None, None) == -1
    assert lib.igs_forward_sr(None, None, None, None, None, None, None, None, None, 1, 1, 4, 4, 0, 1e-6, 1,
                              None, None, None, 0, None, 0, 0, None) == -1
    one = ctypes.c_void_p(16)  # never dereferenced: the unknown hint bit is refused first
    assert lib.igs_forward_sr(one, one, one, one, one, one, None, one, None, 1, 1, 4, 4, 3, 1e-6, 1,
                              one, one, None, 64, one, 1 << 20, 0, None) == -1


def test_added_entry_points_validate_arguments_without_gpu():
    """Null pointers, bad sizes and missing workspaces are refused before any CUDA call."""
    from igs_b200 import _lib

    lib = _lib.load()
    strides = (ctypes.c_int64 * 3)(16, 4, 1)
    one = ctypes.c_void_p(16)  # never dereferenced: every call below fails its argument checks first
    assert lib.igs_spatial_order(None, one, strides, one, strides, 1, 8, 4, 4, one, one, 1 << 20, 0, None) == -1
    assert lib.igs_spatial_order(one, one, strides, one, strides, 1, 8, 0, 4, one, one, 1 << 20, 0, None) == -1
    assert lib.igs_spatial_order(one, one, strides, one, strides, 1, 8, 4, 4, one, None, 0, 0, None) == -2
    assert lib.igs_spatial_order(one, one, strides, one, strides, 1, 8, 4, 4, one, one, 16, 0, None) == -2
    assert lib.igs_spatial_order(one, one, strides, one, strides, 0, 8, 4, 4, one, one, 16, 0, None) == 0  # nothing to do
    assert lib.igs_spatial_order_workspace_bytes(2, 3000) >= 2 * 3 * 4096 * 4 + 2 * 3000 * 2
    boxes = lambda *head: lib.igs_spatial_order_boxes(*head, one, strides, one, strides, 1, 8, 4, 4, one, one, 1 << 20,
                                                      0, None)
    assert boxes(one, 1, None, one, 2, 0, one, 1) == -1   # a centre is two floats
    assert boxes(one, 2, None, one, 1, 0, one, 1) == -1   # so are the scales
    assert boxes(one, 2, None, None, 2, 0, one, 1) == -1  # rotations without scales
    assert boxes(None, 2, None, one, 2, 0, one, 1) == -1
    assert lib.igs_mse_loss(None, one, 10, one, one, 4096, 0, None) == -1
    assert lib.igs_mse_loss(one, one, 0, one, one, 4096, 0, None) == -1
    assert lib.igs_mse_loss(one, one, 10, one, one, 16, 0, None) == -2
    assert lib.igs_mse_grad(one, one, 10, None, None, 0, None) == -1
    assert lib.igs_read_narrow_count(None, 0, None, None) == -1
    assert lib.igs_read_executed(None, 0, None, None) == -1
    assert lib.igs_forward_feature(None, None, one, strides, one, strides, 1, 1, 4, 4, 0, 1e-6, 1, one, one, None, 0,
                                   one, 1 << 20, 0, None) == -1
    assert lib.igs_backward_feature(None, None, one, strides, one, strides, one, one, one, 1, 1, 4, 4, 3, 1e-6, 0,
                                    None, None, 0, one, 1 << 20, 0, None) == -1
    assert lib.igs_backward_feature(one, None, one, strides, one, strides, one, one, one, 1, 1, 4, 4, 3, 1e-6, 7,
                                    one, None, 0, one, 1 << 20, 0, None) == -1  # unknown gradient mode
    assert lib.igs_read_status_words(None, 0, None, None) == -1
    assert lib.igs_read_status_static(0, None, None) == -1


def test_product_package_never_imports_the_oracle():
    """The oracle is test infrastructure; nothing under igs_b200/ may reach it."""
    for dirpath, _, files in os.walk(os.path.join(ROOT, "igs_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src, f"{f} mentions the oracle"


def test_cpu_tensors_are_rejected_not_emulated():
    import torch

    from igs_b200.gs2d import GaussianSplatting2DKernel, gaussian_splatting_2d

    z = torch.zeros
    with pytest.raises(RuntimeError, match="no CPU path"):
        gaussian_splatting_2d(z(1, 2, 2), z(1, 2, 3), z(1, 2, 2) + 1, z(1, 2), z(1, 2), z(1, 1, 3, 3), z(1, 1, 3, 3))
    with pytest.raises(RuntimeError, match="no CPU path"):
        GaussianSplatting2DKernel.apply(z(1, 1, 3, 3), z(1, 1, 3, 3), z(1, 2, 2), z(1, 2, 1, 1), z(1, 2, 1, 1),
                                        z(1, 2, 1, 1), z(1, 2), z(1, 2, 3))
