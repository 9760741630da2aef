"""Host-side mirror of the reference's Python op binding (sparse/ops/fixed_fan_in_ops.py).

Same function names, argument order and return values as the reference's wrappers
(fixed_fan_in_ops.py:15-28), over torch CUDA tensors instead of TensorFlow tensors:

* ``fan_in_sparse_matmul(features[B,N], lookup[L,K], weights[L,K]) -> [B,L]``
* ``fan_in_sparse_matmul_tp(features[N,B], lookup, weights) -> [B,L]``
* ``fan_in_sparse_matmul_grad(features, lookup, weights, out_grad) -> (feature_grad, weight_grad)``
* ``fan_in_sparse_matmul_grad_tp(...)`` likewise for the transposed layout

and the gradient wiring of fixed_fan_in_ops.py:31-40 (``[feature_grad, None, weight_grad]``)
as :class:`torch.autograd.Function` objects behind ``ffi_matmul`` / ``ffi_matmul_tp``.
Every call goes through the C ABI of ``libffi_b200.so``; there is no CPU path.
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Optional

import torch

from . import _lib

_workspaces: dict = {}
_plan_cache: dict = {}
_PLAN_CACHE_MAX = 8


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    """A cached scratch buffer of at least nbytes on `device` (grown, never shrunk)."""
    if nbytes <= 0:
        return None
    key = (device.index, _stream_ptr(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _check_cuda(name: str, t: torch.Tensor, dtypes) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: this library has no CPU path")
    if t.dtype not in dtypes:
        raise TypeError(f"{name} has dtype {t.dtype}, expected one of {dtypes}")
    if t.dim() != 2:
        raise ValueError(f"{name} must have rank 2, got shape {tuple(t.shape)}")
    return t.contiguous()


_INDEX_DTYPES = (torch.int32, torch.uint32) if hasattr(torch, "uint32") else (torch.int32,)


def _as_index(lookup: torch.Tensor) -> torch.Tensor:
    lookup = _check_cuda("lookup", lookup, _INDEX_DTYPES)
    if lookup.dtype != torch.int32:
        lookup = lookup.view(torch.int32)  # values < 2^31 by the reference's contract
    return lookup


def _shapes(features, lookup, weights, transposed):
    if lookup.shape != weights.shape:
        raise ValueError(f"lookup {tuple(lookup.shape)} and weights {tuple(weights.shape)} must have equal shapes")
    if transposed:
        N, B = features.shape
    else:
        B, N = features.shape
    L, K = lookup.shape
    return B, N, L, K


class FFIPlan:
    """Transposed (CSR-by-input) index of one lookup table; owns device memory.

    Build one per lookup table and rebuild it whenever the table changes (rewiring).
    """

    def __init__(self, lookup: torch.Tensor, n_in: int):
        lookup = _as_index(lookup)
        self.device = lookup.device
        self.L, self.K = (int(s) for s in lookup.shape)
        self.N = int(n_in)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().ffi_plan_create(lookup.data_ptr(), self.L, self.K, self.N,
                                                   _stream_ptr(self.device), ctypes.byref(handle)))
        self._handle = handle
        self.builds = 1
        self._finalizer = weakref.finalize(self, _lib.load().ffi_plan_destroy, handle)

    def rebuild(self, lookup: torch.Tensor) -> "FFIPlan":
        """Re-derives the plan in place from a table of the same shape whose contents changed (rewiring);
        the index arrays are reused and, from the second rebuild on, nothing is allocated."""
        lookup = _as_index(lookup)
        if tuple(lookup.shape) != (self.L, self.K) or lookup.device != self.device:
            raise ValueError("rebuild needs a table of the plan's shape on the plan's device")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().ffi_plan_rebuild(self._handle, lookup.data_ptr(), _stream_ptr(self.device)))
        self.builds += 1
        return self

    @property
    def handle(self):
        return self._handle

    def info(self) -> dict:
        vals = [ctypes.c_int64() for _ in range(6)]
        _lib.check(_lib.load().ffi_plan_info(self._handle, *[ctypes.byref(v) for v in vals]))
        names = ("L", "K", "N", "chunk_rows", "n_chunks", "device_bytes")
        return {n: int(v.value) for n, v in zip(names, vals)}

    def export(self, chunked: bool = False):
        """(rowptr[N+1], perm[L*K]) int32 device tensors of the canonical transposed index."""
        rowptr = torch.empty(self.N + 1, dtype=torch.int32, device=self.device)
        perm = torch.empty(self.L * self.K, dtype=torch.int32, device=self.device)
        fn = _lib.load().ffi_plan_export_chunked if chunked else _lib.load().ffi_plan_export
        with torch.cuda.device(self.device):
            _lib.check(fn(self._handle, rowptr.data_ptr(), perm.data_ptr(), _stream_ptr(self.device)))
        return rowptr, perm

    def close(self):
        self._finalizer()


def get_plan(lookup: torch.Tensor, n_in: int) -> FFIPlan:
    """Plan for `lookup`, cached per (storage address, shape, tensor version).

    An in-place update of the table (rewiring) bumps the tensor's version and leads to a
    rebuild of the cached plan in place (`FFIPlan.rebuild`: same object, new contents).  The cache
    keeps a reference to the table so that its address cannot be handed to another tensor while
    the entry lives (at most 8 tables are kept).
    """
    key = (lookup.data_ptr(), tuple(lookup.shape), int(n_in), lookup.device.index)
    hit = _plan_cache.get(key)
    if hit is not None and hit[0] == lookup._version:
        return hit[1]
    if hit is not None:
        plan = hit[1].rebuild(lookup)
        _plan_cache[key] = (lookup._version, plan, lookup)
        return plan
    plan = FFIPlan(lookup, n_in)
    _plan_cache.pop(key, None)
    if len(_plan_cache) >= _PLAN_CACHE_MAX:
        _plan_cache.pop(next(iter(_plan_cache)))
    _plan_cache[key] = (lookup._version, plan, lookup)
    return plan


def clear_caches():
    _plan_cache.clear()
    _workspaces.clear()


_STORAGE_DTYPES = (torch.float32, torch.bfloat16)


def _storage_dtype(features, weights) -> int:
    """x and W share one storage type: fp32, or bf16 (accumulation, y and all gradients stay fp32)."""
    if features.dtype != weights.dtype:
        raise TypeError(f"features ({features.dtype}) and weights ({weights.dtype}) must have the same dtype")
    return _lib.FFI_BF16 if features.dtype == torch.bfloat16 else _lib.FFI_F32


def _forward(features, lookup, weights, bias, transposed: bool) -> torch.Tensor:
    features = _check_cuda("features", features, _STORAGE_DTYPES)
    weights = _check_cuda("weights", weights, _STORAGE_DTYPES)
    dtype = _storage_dtype(features, weights)
    lookup = _as_index(lookup)
    B, N, L, K = _shapes(features, lookup, weights, transposed)
    lib = _lib.load()
    dev = features.device
    if bias is not None:
        if bias.shape != (L,) or bias.dtype != torch.float32 or not bias.is_cuda:
            raise ValueError("bias must be a float32 CUDA tensor of shape [L]")
        bias = bias.contiguous()
    out = torch.empty((B, L), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        ws_bytes = lib.ffi_forward_workspace_bytes(B, N, L, K, int(transposed), dtype)
        ws = _workspace(dev, ws_bytes + 256 if ws_bytes else 0)
        ws_ptr, ws_len = None, 0
        if ws is not None:
            off = (-ws.data_ptr()) % 256
            ws_ptr, ws_len = ws.data_ptr() + off, ws.numel() - off
        _lib.check(lib.ffi_forward(features.data_ptr(), lookup.data_ptr(), weights.data_ptr(),
                                   bias.data_ptr() if bias is not None else None, out.data_ptr(),
                                   B, N, L, K, int(transposed), dtype, ws_ptr, ws_len, _stream_ptr(dev)))
    return out


def _backward(features, lookup, weights, out_grad, transposed: bool, plan: Optional[FFIPlan] = None,
              want_feature_grad=True, want_weight_grad=True, want_bias_grad=False, grad_is_transposed=False,
              feature_grad_out: Optional[torch.Tensor] = None):
    """grad_is_transposed: `out_grad` is gT[L][ldg] (from forward_bce / transpose_gradient), not g[B,L].
    feature_grad_out: a contiguous float32 tensor with the number of elements of `features` that
    receives grad_x instead of a fresh allocation (e.g. a slot of a peer-visible buffer)."""
    features = _check_cuda("features", features, _STORAGE_DTYPES)
    weights = _check_cuda("weights", weights, _STORAGE_DTYPES)
    dtype = _storage_dtype(features, weights)
    out_grad = _check_cuda("out_grad", out_grad, (torch.float32,))
    lookup = _as_index(lookup)
    B, N, L, K = _shapes(features, lookup, weights, transposed)
    if grad_is_transposed:
        if out_grad.shape[0] != L or out_grad.shape[1] < B:
            raise ValueError(f"transposed out_grad has shape {tuple(out_grad.shape)}, expected [{L}, >= {B}]")
    elif tuple(out_grad.shape) != (B, L):
        raise ValueError(f"out_grad has shape {tuple(out_grad.shape)}, expected {(B, L)}")
    lib = _lib.load()
    dev = features.device
    if want_feature_grad and plan is None:
        plan = get_plan(lookup, N)
    gx = None
    if want_feature_grad:
        if feature_grad_out is not None:
            if (feature_grad_out.dtype != torch.float32 or not feature_grad_out.is_contiguous()
                    or feature_grad_out.numel() != features.numel() or feature_grad_out.device != dev):
                raise ValueError("feature_grad_out must be a contiguous float32 tensor of features' size on its device")
            gx = feature_grad_out.view(features.shape)
        else:
            gx = torch.empty(features.shape, dtype=torch.float32, device=dev)
    gw = torch.empty(weights.shape, dtype=torch.float32, device=dev) if want_weight_grad else None
    gb = torch.empty((L,), dtype=torch.float32, device=dev) if want_bias_grad else None
    with torch.cuda.device(dev):
        handle = plan.handle if plan is not None else None
        ws_bytes = lib.ffi_backward_workspace_bytes(handle, B, N, L, K, int(transposed), dtype,
                                                    int(want_feature_grad), int(want_weight_grad or want_bias_grad))
        ws = _workspace(dev, ws_bytes + 256 if ws_bytes else 0)
        ws_ptr = None
        ws_len = 0
        if ws is not None:
            off = (-ws.data_ptr()) % 256
            ws_ptr = ws.data_ptr() + off
            ws_len = ws.numel() - off
        outs = (gx.data_ptr() if gx is not None else None, gw.data_ptr() if gw is not None else None,
                gb.data_ptr() if gb is not None else None)
        if grad_is_transposed:
            _lib.check(lib.ffi_backward_from_transposed(features.data_ptr(), lookup.data_ptr(), weights.data_ptr(),
                                                        out_grad.data_ptr(), out_grad.shape[1], handle, *outs,
                                                        B, N, L, K, int(transposed), dtype, ws_ptr, ws_len,
                                                        _stream_ptr(dev)))
        else:
            _lib.check(lib.ffi_backward(features.data_ptr(), lookup.data_ptr(), weights.data_ptr(), out_grad.data_ptr(),
                                        handle, *outs, B, N, L, K, int(transposed), dtype, ws_ptr, ws_len,
                                        _stream_ptr(dev)))
    return gx, gw, gb


def forward_bce(features, lookup, weights, bias, row_ptr, labels, transposed: bool, total_labels=None,
                label_offset: int = 0, loss: str = "bce", loss_out=None):
    """Forward with the loss gradient fused into its epilogue: returns (loss scalar tensor, gT[L][ldg]).
    `loss` is "bce" (SparseBinaryCrossEntropyLoss), "squared_hinge" (SparseSquaredHingeLoss, the
    one the reference's task files select) or "hinge" (SparseHingeLoss); sparse/metrics.py:132-173.

    The logits are never materialised.  `loss_out` (optional, one fp32 element on the device) receives the
    loss scalar in place, e.g. a slot of the buffer a label-sharded step exchanges."""
    features = _check_cuda("features", features, _STORAGE_DTYPES)
    weights = _check_cuda("weights", weights, _STORAGE_DTYPES)
    dtype = _storage_dtype(features, weights)
    lookup = _as_index(lookup)
    B, N, L, K = _shapes(features, lookup, weights, transposed)
    dev = features.device
    lib = _lib.load()
    row_ptr = row_ptr.to(device=dev, dtype=torch.int32).contiguous()
    labels = labels.to(device=dev, dtype=torch.int32).contiguous()
    if row_ptr.numel() != B + 1:
        raise ValueError("row_ptr must have B+1 entries")
    ldg = int(lib.ffi_transposed_gradient_stride(B))
    gT = torch.empty((L, ldg), dtype=torch.float32, device=dev)
    if loss_out is None:
        loss_out = torch.empty((), dtype=torch.float32, device=dev)
    elif loss_out.dtype != torch.float32 or loss_out.numel() != 1 or loss_out.device != dev:
        raise ValueError("loss_out must be one fp32 element on the features' device")
    with torch.cuda.device(dev):
        ws_bytes = lib.ffi_forward_bce_workspace_bytes(B, N, L, K, int(transposed), dtype)
        ws = _workspace(dev, ws_bytes + 256)
        off = (-ws.data_ptr()) % 256
        kind = {"bce": _lib.FFI_LOSS_BCE, "squared_hinge": _lib.FFI_LOSS_SQUARED_HINGE, "hinge": _lib.FFI_LOSS_HINGE}[loss]
        _lib.check(lib.ffi_forward_loss(kind, features.data_ptr(), lookup.data_ptr(), weights.data_ptr(),
                                        bias.data_ptr() if bias is not None else None, row_ptr.data_ptr(),
                                        labels.data_ptr() if labels.numel() else row_ptr.data_ptr(), gT.data_ptr(),
                                        loss_out.data_ptr(), B, N, L, K, total_labels or L, label_offset,
                                        int(transposed), dtype, ws.data_ptr() + off, ws.numel() - off,
                                        _stream_ptr(dev)))
    return loss_out, gT


def forward_topk(features, lookup, weights, bias, k: int, transposed: bool, label_offset: int = 0):
    """The k highest logits per sample and their labels, (values[B,k], labels[B,k] int32), in the order
    of tf.nn.top_k, without materialising the logits: what PrecisionAtK (sparse/metrics.py:9-70)
    consumes.  With a sharded label dimension call it per shard (`label_offset` = first label of the
    shard) and merge the candidates with `merge_topk`."""
    features = _check_cuda("features", features, (torch.float32, torch.bfloat16))
    weights = _check_cuda("weights", weights, (features.dtype,))
    lookup = _as_index(lookup)
    B, N, L, K = _shapes(features, lookup, weights, transposed)
    dev = features.device
    lib = _lib.load()
    dtype = _lib.FFI_BF16 if features.dtype == torch.bfloat16 else _lib.FFI_F32
    top_val = torch.empty((B, k), dtype=torch.float32, device=dev)
    top_idx = torch.empty((B, k), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        ws_bytes = lib.ffi_forward_topk_workspace_bytes(B, N, L, K, int(transposed), dtype)
        ws = _workspace(dev, ws_bytes + 256)
        off = (-ws.data_ptr()) % 256
        _lib.check(lib.ffi_forward_topk(features.data_ptr(), lookup.data_ptr(), weights.data_ptr(),
                                        bias.data_ptr() if bias is not None else None, top_val.data_ptr(),
                                        top_idx.data_ptr(), k, B, N, L, K, label_offset, int(transposed),
                                        dtype, ws.data_ptr() + off, ws.numel() - off, _stream_ptr(dev)))
    return top_val, top_idx


def merge_topk(candidates, k: int):
    """Best k of several shards' (values, labels) candidate lists, again in tf.nn.top_k order."""
    vals = torch.cat([c[0] for c in candidates], dim=1)
    idxs = torch.cat([c[1] for c in candidates], dim=1)
    # value descending, label ascending on ties: sort by label first, then a stable sort by value
    order = torch.argsort(idxs, dim=1, stable=True)
    vals, idxs = torch.gather(vals, 1, order), torch.gather(idxs, 1, order)
    order = torch.argsort(vals, dim=1, descending=True, stable=True)[:, :k]
    return torch.gather(vals, 1, order), torch.gather(idxs, 1, order)


def precision_at_k(top_labels: torch.Tensor, row_ptr: torch.Tensor, labels: torch.Tensor, k: int) -> float:
    """P@k of a batch as PrecisionAtK accumulates it (sparse/metrics.py:58-70): the number of the k
    top-ranked labels that are true labels, summed over the batch, divided by B*k."""
    top = top_labels[:, :k].to(torch.int64).cpu()
    row_ptr, labels = row_ptr.cpu().to(torch.int64), labels.cpu().to(torch.int64)
    correct = 0
    for b in range(top.shape[0]):
        truth = labels[row_ptr[b]:row_ptr[b + 1]]
        correct += int(torch.isin(top[b], truth).sum())
    return correct / (top.shape[0] * k)


def transpose_gradient(out_grad: torch.Tensor, want_bias_grad: bool = False):
    """g[B,L] -> (gT[L][ldg] zero padded in the batch, grad_bias[L] or None): the transposed copy the
    backward kernels read (and the input of the allocation-free grad_x entry point)."""
    out_grad = _check_cuda("out_grad", out_grad, (torch.float32,))
    B, L = out_grad.shape
    lib = _lib.load()
    ldg = int(lib.ffi_transposed_gradient_stride(B))
    gT = torch.empty((L, ldg), dtype=torch.float32, device=out_grad.device)
    gb = torch.empty((L,), dtype=torch.float32, device=out_grad.device) if want_bias_grad else None
    with torch.cuda.device(out_grad.device):
        _lib.check(lib.ffi_transpose_gradient(out_grad.data_ptr(), gT.data_ptr(), gb.data_ptr() if gb is not None else None,
                                              B, L, _stream_ptr(out_grad.device)))
    return gT, gb


# ---- the reference's four wrappers (sparse/ops/fixed_fan_in_ops.py:15-28) -------------

def fan_in_sparse_matmul(features, lookup, weights):
    return _forward(features, lookup, weights, None, False)


def fan_in_sparse_matmul_tp(features, lookup, weights):
    return _forward(features, lookup, weights, None, True)


def fan_in_sparse_matmul_grad(features, lookup, weights, out_grad):
    gx, gw, _ = _backward(features, lookup, weights, out_grad, False)
    return gx, gw


def fan_in_sparse_matmul_grad_tp(features, lookup, weights, out_grad):
    gx, gw, _ = _backward(features, lookup, weights, out_grad, True)
    return gx, gw


# ---- gradient registration (sparse/ops/fixed_fan_in_ops.py:31-40) ---------------------

class _FanInSparseMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, lookup, weights, bias, transposed):
        ctx.save_for_backward(features, lookup, weights)
        ctx.transposed = transposed
        ctx.has_bias = bias is not None
        return _forward(features, lookup, weights, bias, transposed)

    @staticmethod
    def backward(ctx, grad):
        features, lookup, weights = ctx.saved_tensors
        need_x, _, need_w = ctx.needs_input_grad[:3]
        need_b = ctx.has_bias and ctx.needs_input_grad[3]
        gx, gw, gb = _backward(features, lookup, weights, grad.contiguous(), ctx.transposed,
                               want_feature_grad=need_x, want_weight_grad=need_w, want_bias_grad=need_b)
        return gx, None, gw, gb, None


def ffi_matmul(features, lookup, weights, bias=None):
    """Differentiable FanInSparseMatmul (+ optional fused bias)."""
    return _FanInSparseMatmul.apply(features, lookup, weights, bias, False)


def ffi_matmul_tp(features, lookup, weights, bias=None):
    """Differentiable FanInSparseMatmulTp (features given as [N,B]) (+ optional fused bias)."""
    return _FanInSparseMatmul.apply(features, lookup, weights, bias, True)
