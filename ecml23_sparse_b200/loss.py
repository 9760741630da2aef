"""Sigmoid binary cross-entropy against sparse multi-hot targets.

Mirror of ``SparseBinaryCrossEntropyLoss`` (sparse/metrics.py:167-173) with the base
class's mean over labels (metrics.py:136-139) and the Keras mean over the batch:
``loss = mean_{b,o} bce(z[b,o], t[b,o])``, ``dloss/dz = (sigmoid(z) - t) / (B*L)``.
Targets are CSR (``row_ptr[B+1]``, ``labels[nnz]``, int32, labels of a row distinct).
"""
from __future__ import annotations

import torch

from . import _lib
from .ops import _stream_ptr, _workspace


def sparse_bce_with_logits(logits: torch.Tensor, row_ptr: torch.Tensor, labels: torch.Tensor, *,
                           total_labels: int | None = None, label_offset: int = 0, inplace: bool = False):
    """Returns (loss scalar tensor, grad [B,L]).  With `inplace` the gradient overwrites `logits`.

    `total_labels` / `label_offset` describe a label shard: `logits` is then columns
    [label_offset, label_offset+L) of the full [B,total_labels] matrix and the returned loss is
    this shard's share of the full mean (sum the shares over shards).
    """
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2:
        raise ValueError("logits must be a float32 CUDA matrix")
    logits = logits.contiguous()
    B, L = logits.shape
    row_ptr = row_ptr.to(device=logits.device, dtype=torch.int32).contiguous()
    labels = labels.to(device=logits.device, dtype=torch.int32).contiguous()
    if row_ptr.numel() != B + 1:
        raise ValueError("row_ptr must have B+1 entries")
    grad = logits if inplace else torch.empty_like(logits)
    loss = torch.empty((), dtype=torch.float32, device=logits.device)
    lib = _lib.load()
    with torch.cuda.device(logits.device):
        ws = _workspace(logits.device, lib.ffi_bce_workspace_bytes(B, L) + 8)
        off = (-ws.data_ptr()) % 8
        _lib.check(lib.ffi_bce_grad(logits.data_ptr(), row_ptr.data_ptr(), labels.data_ptr() if labels.numel() else row_ptr.data_ptr(),
                                    grad.data_ptr(), loss.data_ptr(), B, L, total_labels or L, label_offset,
                                    ws.data_ptr() + off, ws.numel() - off, _stream_ptr(logits.device)))
    return loss, grad
