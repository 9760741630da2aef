"""ctypes binding of ``libffi_b200.so`` (the C ABI declared in ``include/ffi_b200.h``).

There is no CPU fallback: if the CUDA library cannot be loaded (or built), importing the
ops raises.  The library is built in-tree by :mod:`ecml23_sparse_b200.build`.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

FFI_OK = 0
STATUS_NAMES = {
    0: "FFI_OK",
    1: "FFI_ERR_INVALID_ARGUMENT",
    2: "FFI_ERR_UNSUPPORTED",
    3: "FFI_ERR_WORKSPACE",
    4: "FFI_ERR_CUDA",
    5: "FFI_ERR_STALE_PLAN",
    6: "FFI_ERR_INDEX_RANGE",
    7: "FFI_ERR_ALLOC",
}
FFI_F32 = 0
FFI_BF16 = 1
FFI_LOSS_BCE = 0
FFI_LOSS_SQUARED_HINGE = 1
FFI_LOSS_HINGE = 2

# Every symbol include/ffi_b200.h declares.
EXPORTED_SYMBOLS = (
    "ffi_last_error", "ffi_version", "ffi_set_debug_bounds",
    "ffi_forward_workspace_bytes", "ffi_forward",
    "ffi_plan_create", "ffi_plan_rebuild", "ffi_plan_destroy", "ffi_plan_info", "ffi_plan_export", "ffi_plan_export_chunked",
    "ffi_backward_workspace_bytes", "ffi_backward",
    "ffi_grad_x_static_max_scratch_bytes", "ffi_grad_x_static",
    "ffi_transposed_gradient_stride", "ffi_transpose_gradient",
    "ffi_backward_from_transposed", "ffi_forward_bce_workspace_bytes", "ffi_forward_bce", "ffi_forward_loss", "ffi_wait_timeouts",
    "ffi_set_wait_limit_ticks",
    "ffi_forward_topk_workspace_bytes", "ffi_forward_topk", "ffi_peer_sum",
    "ffi_bce_workspace_bytes", "ffi_bce_grad", "ffi_adam_step",
    "ffi_rewire_workspace_bytes", "ffi_rewire",
)


class FFIError(RuntimeError):
    """A call into the CUDA library returned a non-zero ffi_status."""

    def __init__(self, status: int, message: str):
        self.status = status
        super().__init__(f"{STATUS_NAMES.get(status, status)}: {message}")


_lib = None


def _declare(lib):
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    f32 = ctypes.c_float
    lib.ffi_last_error.restype = ctypes.c_char_p
    lib.ffi_last_error.argtypes = []
    lib.ffi_version.restype = i32
    lib.ffi_set_debug_bounds.restype = i32
    lib.ffi_set_debug_bounds.argtypes = [i32]
    lib.ffi_forward_workspace_bytes.restype = sz
    lib.ffi_forward_workspace_bytes.argtypes = [i64, i64, i64, i64, i32, i32]
    lib.ffi_forward.restype = i32
    lib.ffi_forward.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_plan_create.restype = i32
    lib.ffi_plan_create.argtypes = [vp, i64, i64, i64, vp, ctypes.POINTER(vp)]
    lib.ffi_plan_rebuild.restype = i32
    lib.ffi_plan_rebuild.argtypes = [vp, vp, vp]
    lib.ffi_plan_destroy.restype = i32
    lib.ffi_plan_destroy.argtypes = [vp]
    lib.ffi_plan_info.restype = i32
    lib.ffi_plan_info.argtypes = [vp] + [ctypes.POINTER(i64)] * 6
    lib.ffi_plan_export.restype = i32
    lib.ffi_plan_export.argtypes = [vp, vp, vp, vp]
    lib.ffi_plan_export_chunked.restype = i32
    lib.ffi_plan_export_chunked.argtypes = [vp, vp, vp, vp]
    lib.ffi_backward_workspace_bytes.restype = sz
    lib.ffi_backward_workspace_bytes.argtypes = [vp, i64, i64, i64, i64, i32, i32, i32, i32]
    lib.ffi_backward.restype = i32
    lib.ffi_backward.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_grad_x_static_max_scratch_bytes.restype = sz
    lib.ffi_grad_x_static_max_scratch_bytes.argtypes = []
    lib.ffi_grad_x_static.restype = i32
    lib.ffi_grad_x_static.argtypes = [vp, vp, i64, vp, vp, i64, i64, i64, i64, i32, vp]
    lib.ffi_transposed_gradient_stride.restype = i64
    lib.ffi_transposed_gradient_stride.argtypes = [i64]
    lib.ffi_transpose_gradient.restype = i32
    lib.ffi_transpose_gradient.argtypes = [vp, vp, vp, i64, i64, vp]
    lib.ffi_backward_from_transposed.restype = i32
    lib.ffi_backward_from_transposed.argtypes = [vp, vp, vp, vp, i64, vp, vp, vp, vp, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_forward_bce_workspace_bytes.restype = sz
    lib.ffi_forward_bce_workspace_bytes.argtypes = [i64, i64, i64, i64, i32, i32]
    lib.ffi_forward_bce.restype = i32
    lib.ffi_forward_bce.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_forward_loss.restype = i32
    lib.ffi_forward_loss.argtypes = [i32, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_forward_topk_workspace_bytes.restype = sz
    lib.ffi_forward_topk_workspace_bytes.argtypes = [i64, i64, i64, i64, i32, i32]
    lib.ffi_forward_topk.restype = i32
    lib.ffi_forward_topk.argtypes = [vp, vp, vp, vp, vp, vp, i32, i64, i64, i64, i64, i64, i32, i32, vp, sz, vp]
    lib.ffi_peer_sum.restype = i32
    lib.ffi_peer_sum.argtypes = [vp, vp, i32, i32, i64, ctypes.c_uint32, vp, vp]
    lib.ffi_set_wait_limit_ticks.restype = i32
    lib.ffi_set_wait_limit_ticks.argtypes = [i64]
    lib.ffi_wait_timeouts.restype = i32
    lib.ffi_wait_timeouts.argtypes = [vp]
    lib.ffi_bce_workspace_bytes.restype = sz
    lib.ffi_bce_workspace_bytes.argtypes = [i64, i64]
    lib.ffi_bce_grad.restype = i32
    lib.ffi_bce_grad.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, vp, sz, vp]
    lib.ffi_rewire_workspace_bytes.restype = sz
    lib.ffi_rewire_workspace_bytes.argtypes = []
    lib.ffi_rewire.restype = i32
    lib.ffi_rewire.argtypes = [vp, vp, vp, vp, i64, i64, i64, ctypes.c_uint64, vp, vp, vp, sz, vp]
    lib.ffi_adam_step.restype = i32
    lib.ffi_adam_step.argtypes = [vp, vp, vp, vp, i64, f32, f32, f32, f32, i64, i32, vp]


def lib_path() -> str:
    return _build.LIB_PATH


def load(rebuild_if_stale: bool = True):
    """Returns the loaded library, building it first when sources are newer (needs nvcc)."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if rebuild_if_stale:
        try:
            path = _build.build()
        except Exception as exc:  # no nvcc on this machine: use the shipped library if there is one
            if not os.path.exists(path):
                raise ImportError(f"libffi_b200.so is missing and could not be built: {exc}") from exc
    if not os.path.exists(path):
        raise ImportError(f"{path} not found; run `python -m ecml23_sparse_b200.build`")
    lib = ctypes.CDLL(path)
    _declare(lib)
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != FFI_OK:
        raise FFIError(status, load().ffi_last_error().decode("utf-8", "replace"))
