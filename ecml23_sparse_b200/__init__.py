"""B200 (sm_100a) fixed-fan-in (FFI) sparse layer: CUDA kernels behind a C ABI, with a
host-side mirror of the reference's op binding and layer.

Importing this package does not need a GPU; calling an op does (there is no CPU path).
"""
from .ops import (FFIPlan, fan_in_sparse_matmul, fan_in_sparse_matmul_grad, fan_in_sparse_matmul_grad_tp,
                  fan_in_sparse_matmul_tp, ffi_matmul, ffi_matmul_tp, get_plan)
from .layer import FFILayer
from .loss import sparse_bce_with_logits
from .optimizer import FusedAdam

__all__ = [
    "FFIPlan", "FFILayer", "FusedAdam", "fan_in_sparse_matmul", "fan_in_sparse_matmul_tp",
    "fan_in_sparse_matmul_grad", "fan_in_sparse_matmul_grad_tp", "ffi_matmul", "ffi_matmul_tp",
    "get_plan", "sparse_bce_with_logits",
]
