"""TEST INFRASTRUCTURE ONLY: Python face of the parity oracle.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this
package; the product (``ecml23_sparse_b200``) never does.

Three layers, each checking the next:

* ``ref_forward`` / ``ref_backward``: the reference's own CPU kernels
  (tfsparse/cc/kernels/forward.cpp, backward.cpp) compiled from their sources against
  stand-in headers (``oracle/_ref/libffi_ref.so``; see ``build_oracle.py``).
* ``forward_f32`` ...: the C restatement in ``ffi_oracle.c`` (same summation order as the
  reference in fp32, plus fp64 variants used as the tolerance reference).
* ``dense_forward`` / ``dense_backward``: numpy restatement of the reference's dense
  test oracle (tfsparse/cc/kernels/reference.cpp:15-82), small shapes only.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build_oracle as _build

_F = ctypes.POINTER(ctypes.c_float)
_D = ctypes.POINTER(ctypes.c_double)
_I = ctypes.POINTER(ctypes.c_int32)
_i64 = ctypes.c_int64
_int = ctypes.c_int

_lib = None
_ref = None


def _ptr(a, ty):
    if a is None:
        return None
    return a.ctypes.data_as(ty)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i32(a):
    a = np.asarray(a)
    if a.dtype == np.uint32:
        a = a.view(np.int32) if a.flags.c_contiguous else a.astype(np.int32)
    return np.ascontiguousarray(a, dtype=np.int32)


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        L = ctypes.CDLL(path)
        L.oracle_max_threads.restype = _int
        L.oracle_forward_f32.argtypes = [_F, _I, _F, _F, _F, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_forward_f64.argtypes = [_F, _I, _F, _F, _D, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_grad_w_f32.argtypes = [_F, _I, _F, _F, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_grad_w_f64.argtypes = [_F, _I, _F, _D, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_grad_x_f32.argtypes = [_I, _F, _F, _F, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_grad_x_f64.argtypes = [_I, _F, _F, _D, _i64, _i64, _i64, _i64, _int, _int]
        L.oracle_grad_bias_f64.argtypes = [_F, _D, _i64, _i64]
        L.oracle_transpose_index.argtypes = [_I, _i64, _i64, _i64, _I, _I]
        L.oracle_transpose_index.restype = _int
        L.oracle_bce_f64.argtypes = [_F, _I, _I, _D, _i64, _i64]
        L.oracle_bce_f64.restype = ctypes.c_double
        L.oracle_hinge_f64.argtypes = [_F, _I, _I, _D, _i64, _i64, ctypes.c_int]
        L.oracle_hinge_f64.restype = ctypes.c_double
        L.oracle_adam_f64.argtypes = [_D, _D, _D, _D, _i64, ctypes.c_double, ctypes.c_double,
                                      ctypes.c_double, ctypes.c_double, _i64]
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _dims(x, idx, transposed):
    x = _f32(x)
    idx = _i32(idx)
    if transposed:
        N, B = x.shape
    else:
        B, N = x.shape
    L, K = idx.shape
    return x, idx, B, N, L, K


def forward_f32(x, idx, W, bias=None, transposed=False, threads=1):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    W = _f32(W)
    bias = None if bias is None else _f32(bias)
    y = np.empty((B, L), np.float32)
    lib().oracle_forward_f32(_ptr(x, _F), _ptr(idx, _I), _ptr(W, _F), _ptr(bias, _F), _ptr(y, _F),
                             B, N, L, K, int(transposed), threads)
    return y


def forward_f64(x, idx, W, bias=None, transposed=False, threads=0):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    W = _f32(W)
    bias = None if bias is None else _f32(bias)
    y = np.empty((B, L), np.float64)
    lib().oracle_forward_f64(_ptr(x, _F), _ptr(idx, _I), _ptr(W, _F), _ptr(bias, _F), _ptr(y, _D),
                             B, N, L, K, int(transposed), threads)
    return y


def grad_w_f32(x, idx, g, transposed=False, threads=1):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    g = _f32(g)
    out = np.empty((L, K), np.float32)
    lib().oracle_grad_w_f32(_ptr(x, _F), _ptr(idx, _I), _ptr(g, _F), _ptr(out, _F), B, N, L, K,
                            int(transposed), threads)
    return out


def grad_w_f64(x, idx, g, transposed=False, threads=0):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    g = _f32(g)
    out = np.empty((L, K), np.float64)
    lib().oracle_grad_w_f64(_ptr(x, _F), _ptr(idx, _I), _ptr(g, _F), _ptr(out, _D), B, N, L, K,
                            int(transposed), threads)
    return out


def grad_x_f32(idx, W, g, N, transposed=False, threads=1):
    idx = _i32(idx)
    W = _f32(W)
    g = _f32(g)
    B, L = g.shape
    K = idx.shape[1]
    out = np.empty((N, B) if transposed else (B, N), np.float32)
    lib().oracle_grad_x_f32(_ptr(idx, _I), _ptr(W, _F), _ptr(g, _F), _ptr(out, _F), B, N, L, K,
                            int(transposed), threads)
    return out


def grad_x_f64(idx, W, g, N, transposed=False, threads=0):
    idx = _i32(idx)
    W = _f32(W)
    g = _f32(g)
    B, L = g.shape
    K = idx.shape[1]
    out = np.empty((N, B) if transposed else (B, N), np.float64)
    lib().oracle_grad_x_f64(_ptr(idx, _I), _ptr(W, _F), _ptr(g, _F), _ptr(out, _D), B, N, L, K,
                            int(transposed), threads)
    return out


def grad_bias_f64(g):
    g = _f32(g)
    B, L = g.shape
    out = np.empty((L,), np.float64)
    lib().oracle_grad_bias_f64(_ptr(g, _F), _ptr(out, _D), B, L)
    return out


def transpose_index(idx, N):
    """(rowptr[N+1], perm[L*K]) of the CSR-by-input index; int32; raises on bad indices."""
    idx = _i32(idx)
    L, K = idx.shape
    rowptr = np.empty((N + 1,), np.int32)
    perm = np.empty((L * K,), np.int32)
    rc = lib().oracle_transpose_index(_ptr(idx, _I), L, K, N, _ptr(rowptr, _I), _ptr(perm, _I))
    if rc != 0:
        raise ValueError("index outside [0, N)" if rc == -1 else "out of memory")
    return rowptr, perm


def transpose_index_np(idx, N):
    """numpy twin of :func:`transpose_index` (stable argsort + bincount)."""
    flat = _i32(idx).ravel()
    perm = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=N)
    rowptr = np.zeros(N + 1, np.int64)
    np.cumsum(counts, out=rowptr[1:])
    return rowptr.astype(np.int32), perm


def make_dense(idx, W, N):
    """[N, L] dense operator; duplicate indices in a row add (reference.cpp:15-27)."""
    idx = _i32(idx)
    L, K = idx.shape
    D = np.zeros((N, L), np.float64)
    cols = np.repeat(np.arange(L), K)
    np.add.at(D, (idx.ravel(), cols), np.asarray(W, np.float64).ravel())
    return D


def dense_forward(x, idx, W, transposed=False):
    """y = x . D  (reference.cpp:29-45), fp64."""
    x = np.asarray(x, np.float64)
    if transposed:
        x = x.T
    return x @ make_dense(idx, W, x.shape[1])


def dense_backward(x, idx, W, g, transposed=False):
    """(grad_x, grad_W) = (g . D^T, (x^T g)[idx[o,k], o])  (reference.cpp:47-82), fp64."""
    x = np.asarray(x, np.float64)
    if transposed:
        x = x.T
    g = np.asarray(g, np.float64)
    idx = _i32(idx)
    D = make_dense(idx, W, x.shape[1])
    gx = g @ D.T
    dense_gw = x.T @ g
    L, K = idx.shape
    gW = dense_gw[idx, np.arange(L)[:, None]]
    if transposed:
        gx = gx.T
    return gx, gW


def bce_f64(z, row_ptr, labels, want_grad=True):
    z = _f32(z)
    B, L = z.shape
    row_ptr = _i32(row_ptr)
    labels = _i32(labels)
    g = np.empty((B, L), np.float64) if want_grad else None
    loss = lib().oracle_bce_f64(_ptr(z, _F), _ptr(row_ptr, _I), _ptr(labels, _I), _ptr(g, _D), B, L)
    return float(loss), g


def hinge_f64(z, row_ptr, labels, squared=True, want_grad=True):
    """(loss, g[B,L]) of the sparse hinge / squared hinge loss (sparse/metrics.py:146-164)."""
    z = _f32(z)
    B, L = z.shape
    row_ptr = _i32(row_ptr)
    labels = _i32(labels)
    g = np.empty((B, L), np.float64) if want_grad else None
    loss = lib().oracle_hinge_f64(_ptr(z, _F), _ptr(row_ptr, _I), _ptr(labels, _I), _ptr(g, _D), B, L,
                                  int(bool(squared)))
    return float(loss), g


def adam_f64(w, m, v, grad, lr, beta1, beta2, eps, step):
    w = np.array(w, np.float64).ravel()
    m = np.array(m, np.float64).ravel()
    v = np.array(v, np.float64).ravel()
    grad = np.ascontiguousarray(grad, np.float64).ravel()
    lib().oracle_adam_f64(_ptr(w, _D), _ptr(m, _D), _ptr(v, _D), _ptr(grad, _D), w.size, lr, beta1,
                          beta2, eps, step)
    return w, m, v


# ---- the reference's own CPU kernels -------------------------------------------------

def ref_lib():
    """ctypes handle of the compiled reference kernels, or None if not available."""
    global _ref
    if _ref is None:
        path = _build.build_reference()
        if path is None or not os.path.exists(path):
            return None
        R = ctypes.CDLL(path)
        R.ref_forward.argtypes = [_F, _I, _F, _F, _i64, _i64, _i64, _i64, _int, _int]
        R.ref_backward.argtypes = [_F, _I, _F, _F, _F, _F, _i64, _i64, _i64, _i64, _int, _int]
        R.ref_hardware_threads.restype = _int
        _ref = R
    return _ref


def ref_available() -> bool:
    return ref_lib() is not None


def ref_forward(x, idx, W, transposed=False, threads=0):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    W = _f32(W)
    y = np.empty((B, L), np.float32)
    ref_lib().ref_forward(_ptr(x, _F), _ptr(idx, _I), _ptr(W, _F), _ptr(y, _F), B, N, L, K,
                          int(transposed), threads)
    return y


def ref_backward(x, idx, W, g, transposed=False, threads=0):
    x, idx, B, N, L, K = _dims(x, idx, transposed)
    W = _f32(W)
    g = _f32(g)
    gx = np.empty(x.shape, np.float32)
    gW = np.empty((L, K), np.float32)
    ref_lib().ref_backward(_ptr(x, _F), _ptr(idx, _I), _ptr(W, _F), _ptr(g, _F), _ptr(gx, _F),
                           _ptr(gW, _F), B, N, L, K, int(transposed), threads)
    return gx, gW
