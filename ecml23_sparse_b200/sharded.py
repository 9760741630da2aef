"""Label-dimension sharding of one FFI layer over the GPUs of a node.

The reference runs on one GPU only (run.py:156).  Rows of (idx, W, bias) are independent for
the forward pass, grad_W, grad_bias, the BCE gradient and Adam; only grad_x sums over the
outputs.  Rank r therefore owns a contiguous block of output rows, x is replicated, and the
[B,N] (or [N,B]) grad_x partials are summed with one all-reduce per step.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [lo, hi) of rank `rank`: blocks of ceil(total/world) rows, the last ones shorter or empty."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    per = -(-total // world)
    lo = min(total, rank * per)
    return lo, min(total, lo + per)


def filter_targets(row_ptr: torch.Tensor, labels: torch.Tensor, lo: int, hi: int):
    """CSR targets restricted to labels in [lo, hi) and re-based to the shard (label - lo)."""
    keep = (labels >= lo) & (labels < hi)
    B = row_ptr.numel() - 1
    rows = torch.repeat_interleave(torch.arange(B, device=labels.device), (row_ptr[1:] - row_ptr[:-1]).long())
    counts = torch.bincount(rows[keep], minlength=B)
    new_ptr = torch.zeros(B + 1, dtype=torch.int32, device=labels.device)
    new_ptr[1:] = torch.cumsum(counts, 0).to(torch.int32)
    return new_ptr, (labels[keep] - lo).to(torch.int32)


class LabelShardedStep:
    """One forward+backward step of a label-sharded FFI layer.

    `forward_fn(xT) -> y_shard`, `backward_fn(xT, g_shard) -> (gx, gW, gbias)` are the per-shard
    compute (the CUDA ops on a GPU rank); `gx` partials are all-reduced over `group`.
    """

    def __init__(self, forward_fn: Callable, backward_fn: Callable, group: Optional[dist.ProcessGroup] = None):
        self.forward_fn = forward_fn
        self.backward_fn = backward_fn
        self.group = group

    @property
    def world(self) -> int:
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def step(self, xT: torch.Tensor, g_shard_fn: Callable[[torch.Tensor], torch.Tensor]):
        """y = forward(xT); g = g_shard_fn(y); (gx, gW, gbias) = backward; gx summed over ranks."""
        y = self.forward_fn(xT)
        g = g_shard_fn(y)
        gx, gW, gb = self.backward_fn(xT, g)
        if self.world > 1:
            dist.all_reduce(gx, op=dist.ReduceOp.SUM, group=self.group)
        return y, gx, gW, gb
