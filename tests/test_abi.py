"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments with a status code (no compute call is made)."""
import ctypes
import os
import re

import pytest

from ecml23_sparse_b200 import _lib, build

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "ffi_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ffi_[a-z_0-9]+)\s*\(", text)))


def test_library_builds_and_loads():
    path = build.build()
    assert os.path.exists(path)
    lib = _lib.load()
    assert lib.ffi_version() >= 100


def test_every_declared_symbol_is_exported():
    lib = _lib.load()
    names = declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/ffi_b200.h but not exported"
    assert set(names) == set(_lib.EXPORTED_SYMBOLS)


def test_null_and_bad_shapes_return_status_not_abort():
    lib = _lib.load()
    assert lib.ffi_forward(None, None, None, None, None, 1, 1, 1, 1, 0, 0, None, 0, None) == 1
    assert b"NULL" in lib.ffi_last_error()
    one = ctypes.c_void_p(16)
    assert lib.ffi_forward(one, one, one, None, one, 0, 4, 4, 2, 0, 0, None, 0, None) == 1
    assert lib.ffi_forward(one, one, one, None, one, 4, 4, 4, 2, 0, 7, None, 0, None) == 2
    assert lib.ffi_forward(one, one, one, None, one, 4, 4, 1 << 31, 2, 0, 0, None, 0, None) == 2
    assert lib.ffi_backward(one, one, one, None, None, None, None, None, 4, 4, 4, 2, 0, 0, None, 0, None) == 1
    # grad_x without a plan is an argument error
    assert lib.ffi_backward(one, one, one, one, None, one, None, None, 4, 4, 4, 2, 0, 0, None, 0, None) == 1
    assert lib.ffi_adam_step(None, None, None, None, 4, 1e-3, 0.9, 0.999, 1e-7, 1, 0, None) == 1
    assert lib.ffi_adam_step(one, one, one, one, 4, 1e-3, 0.9, 0.999, 1e-7, 0, 0, None) == 1
    assert lib.ffi_bce_grad(None, None, None, None, None, 1, 1, 1, 0, None, 0, None) == 1
    handle = ctypes.c_void_p()
    assert lib.ffi_plan_create(None, 4, 2, 4, None, ctypes.byref(handle)) == 1
    assert lib.ffi_plan_create(one, 4, 0, 4, None, ctypes.byref(handle)) == 1
    assert lib.ffi_plan_destroy(None) == 0
    with pytest.raises(_lib.FFIError):
        _lib.check(1)


def test_ops_refuse_cpu_tensors():
    import torch

    import ecml23_sparse_b200 as ffi

    x = torch.zeros(2, 3)
    idx = torch.zeros(4, 2, dtype=torch.int32)
    w = torch.zeros(4, 2)
    with pytest.raises(ValueError, match="no CPU path"):
        ffi.fan_in_sparse_matmul(x, idx, w)
    with pytest.raises(ValueError, match="no CPU path"):
        ffi.fan_in_sparse_matmul_grad_tp(x.t().contiguous(), idx, w, torch.zeros(2, 4))
