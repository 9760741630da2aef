"""Fused Adam on the flat FFI weight vector.

Mirror of ``SparseAdam`` (sparse/optimizer.py:9-23), i.e. ``keras.optimizers.Adam`` with its
defaults as used at run.py:126 (lr 1e-3, beta 0.9/0.999, epsilon 1e-7, no amsgrad): one fused
kernel per parameter instead of Keras' chain of elementwise ops.  ``zero_moments`` is the
moment reset that ``SparseAdam.update_sparse`` performs at rewired positions
(custom_layer.py:20-30).
"""
from __future__ import annotations

import torch

from . import _lib
from .ops import _stream_ptr


class FusedAdam:
    def __init__(self, params, lr: float = 1e-3, beta_1: float = 0.9, beta_2: float = 0.999, epsilon: float = 1e-7):
        self.params = [p for p in params]
        for p in self.params:
            if not p.is_cuda or p.dtype not in (torch.float32, torch.bfloat16) or not p.is_contiguous():
                raise ValueError("FusedAdam needs contiguous float32/bfloat16 CUDA parameters")
        self.lr, self.beta_1, self.beta_2, self.epsilon = lr, beta_1, beta_2, epsilon
        self.iterations = 0
        self.m = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]
        self.v = [torch.zeros(p.shape, dtype=torch.float32, device=p.device) for p in self.params]

    def step(self, grads=None):
        """Applies one update; `grads` defaults to each parameter's `.grad`."""
        self.iterations += 1
        lib = _lib.load()
        for j, p in enumerate(self.params):
            g = grads[j] if grads is not None else p.grad
            if g is None:
                continue
            g = g.contiguous()
            if g.dtype != torch.float32 or g.shape != p.shape:
                raise ValueError("gradient must be float32 with the parameter's shape")
            dtype = _lib.FFI_BF16 if p.dtype == torch.bfloat16 else _lib.FFI_F32
            data = p.data if isinstance(p, torch.nn.Parameter) else p
            with torch.cuda.device(p.device):
                _lib.check(lib.ffi_adam_step(data.data_ptr(), self.m[j].data_ptr(), self.v[j].data_ptr(), g.data_ptr(),
                                             p.numel(), self.lr, self.beta_1, self.beta_2, self.epsilon,
                                             self.iterations, dtype, _stream_ptr(p.device)))

    def zero_moments(self, index: int, locations: torch.Tensor):
        """Zero m and v of parameter `index` at flat positions `locations`."""
        self.m[index].view(-1)[locations] = 0
        self.v[index].view(-1)[locations] = 0
