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


class PeerSum:
    """Sum of a small per-rank tensor over the GPUs of one node through peer memory (`ffi_peer_sum`):
    every rank leaves its partial in a symmetric buffer, raises a flag at each peer and adds the
    world's partials itself, in rank order.  One kernel launch per call instead of an all-reduce whose
    cost at this size (0.4 MB) is pure latency.

    `PeerSum.create` returns None when symmetric memory cannot be set up (older drivers, no peer
    access); callers then keep `dist.all_reduce`.  All ranks must call `sum` the same number of times.
    """

    def __init__(self, numel: int, device, group, buf, flags, buf_handle, flag_handle):
        import ctypes

        self.numel = numel
        self.device = device
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.buf, self.flags = buf, flags
        self._handles = (buf_handle, flag_handle)  # keep the mappings alive
        self._bufs = (ctypes.c_void_p * self.world)(*[int(p) for p in buf_handle.buffer_ptrs])
        self._flags = (ctypes.c_void_p * self.world)(*[int(p) for p in flag_handle.buffer_ptrs])
        self.step = 0

    @classmethod
    def create(cls, numel: int, device, group=None) -> Optional["PeerSum"]:
        group = group if group is not None else dist.group.WORLD
        ok = torch.zeros(1, device=device)
        made = None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            n = -(-numel // 4) * 4
            buf = symm_mem.empty((2, n), dtype=torch.float32, device=device)
            flags = symm_mem.empty((2, dist.get_world_size(group)), dtype=torch.int32, device=device)
            buf.zero_()
            flags.zero_()
            hb = symm_mem.rendezvous(buf, group)
            hf = symm_mem.rendezvous(flags, group)
            torch.cuda.synchronize(device)
            made = cls(n, device, group, buf, flags, hb, hf)
            ok.fill_(1)
        except Exception:  # noqa: BLE001 - any failure means "not available here"
            made = None
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)  # all ranks or none; also orders the zeroing
        return made if ok.item() == 1 else None

    def slot(self) -> torch.Tensor:
        """The buffer the NEXT call of `sum` reads this rank's partial from: write the partial here."""
        return self.buf[(self.step + 1) & 1, :]

    def sum(self, out: torch.Tensor) -> torch.Tensor:
        """out[numel] = sum over ranks of their `slot()` contents (written on the current stream)."""
        from . import _lib
        from .ops import _stream_ptr

        self.step += 1
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().ffi_peer_sum(self._bufs, self._flags, self.rank, self.world, self.numel, self.step,
                                                out.data_ptr(), _stream_ptr(self.device)))
        return out


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
