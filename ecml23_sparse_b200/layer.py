"""The FFI layer: host-side mirror of ``StratifiedRewireLayerV2`` (sparse/custom_layer.py:6-50)
on top of its base class ``RewireLayerBase`` (sparse/layer.py:107-273).

State, as in the reference: a flat ``[units*fan_in]`` index table drawn uniformly *with*
replacement (custom_layer.py:12-15), a flat weight vector of the same length
(layer.py:174-182), an optional bias ``[units]`` initialised to zero (layer.py:192-201).
``forward`` reshapes both to ``[units, fan_in]``, feeds the input transposed to the
``FanInSparseMatmulTp`` op (custom_layer.py:45-50) and adds the bias (layer.py:245-247);
here the bias add is fused into the forward kernel and its gradient into grad_W's.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from . import ops


def _num_selected(fraction: float, connections: int) -> int:
    """round(fraction * connections) as FixedFractionSelector computes it (layer.py:75-76): the product of
    two float32 values, rounded half to even (tf.math.round)."""
    import numpy as np

    return int(np.rint(np.float32(fraction) * np.float32(connections)))


class FFILayer(nn.Module):
    def __init__(self, in_features: int, units: int, fan_in: int, use_bias: bool = True, device=None,
                 seed: int | None = None):
        super().__init__()
        self.in_features = int(in_features)
        self.units = int(units)
        self.fan_in = int(fan_in)
        self.connections = self.units * self.fan_in
        gen = torch.Generator(device="cpu")
        if seed is not None:
            gen.manual_seed(seed)
        # uniform with replacement, as custom_layer.py:15 (tf.random.uniform over [0, dim))
        idx = torch.randint(0, self.in_features, (self.connections,), generator=gen, dtype=torch.int32)
        # glorot_uniform over a [connections] vector (layer.py:110,174-182): limit sqrt(6/(fan_in+fan_out))
        limit = math.sqrt(6.0 / (2 * self.connections)) if self.connections > 0 else 0.0
        w = (torch.rand(self.connections, generator=gen) * 2 - 1) * limit
        self.register_buffer("kernel_indices", idx.to(device))
        self.kernel_weights = nn.Parameter(w.to(device))
        self.bias = nn.Parameter(torch.zeros(self.units, device=device)) if use_bias else None

    def lookup(self) -> torch.Tensor:
        return self.kernel_indices.view(self.units, self.fan_in)

    def weights(self) -> torch.Tensor:
        return self.kernel_weights.view(self.units, self.fan_in)

    def plan(self) -> ops.FFIPlan:
        """Transposed index of the current table (cached until the table is modified in place)."""
        return ops.get_plan(self.lookup(), self.in_features)

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        if inputs.dim() != 2 or inputs.shape[1] != self.in_features:
            raise ValueError(f"expected input of shape [B, {self.in_features}], got {tuple(inputs.shape)}")
        tp_in = inputs.t().contiguous()  # custom_layer.py:48
        return ops.ffi_matmul_tp(tp_in, self.lookup(), self.weights(), self.bias).contiguous()

    # ---- rewiring (sparse/layer.py:62-86,236-237; sparse/custom_layer.py:20-43) -----------------
    def rewire_candidates(self, fraction: float = 0.01) -> torch.Tensor:
        """Flat positions selected by the reference's FixedFractionSelector (layer.py:62-86):
        num_selected = round(fraction * connections); threshold = the num_selected-th smallest |w|;
        every connection with |w| strictly below the threshold is selected."""
        if not 0.0 <= fraction <= 1.0:
            raise ValueError("fraction must lie in [0, 1]")
        flat = self.kernel_weights.detach().abs().reshape(-1)
        num_selected = _num_selected(fraction, flat.numel())
        if num_selected < 1:
            return torch.empty(0, dtype=torch.long, device=flat.device)
        threshold = torch.kthvalue(flat, num_selected).values
        return torch.nonzero(flat < threshold).reshape(-1)

    @torch.no_grad()
    def rewire(self, fraction: float = 0.01, optimizer=None, param_index: int = 0, seed: int = 0):
        """One rewiring step as StratifiedRewireLayerV2._rewire does (custom_layer.py:32-43) with the
        FixedFractionSelector (layer.py:62-86), on the device through `ffi_rewire`: the connections whose
        |w| lies strictly below the round(fraction*connections)-th smallest |w| get a new source uniform
        in [0, in_features) (a counter-based hash of (seed, position): pass a new seed per rewiring
        event); their weights are kept; the optimizer's moments m and v (`optimizer.m[param_index]`,
        `optimizer.v[param_index]`) are zeroed there (custom_layer.py:20-30).  The index table is updated
        in place, so the cached transposed index is rebuilt on the next backward pass.
        Returns (threshold, count) as device tensors; nothing is copied to the host."""
        import ctypes

        from . import _lib

        if not 0.0 <= fraction <= 1.0:
            raise ValueError("fraction must lie in [0, 1]")
        w = self.kernel_weights.detach()
        if not w.is_cuda:
            raise ValueError("rewire() runs on the device: the layer must live on a CUDA device")
        dev = w.device
        num_selected = _num_selected(fraction, self.connections)
        m = v = None
        if optimizer is not None:
            m, v = optimizer.m[param_index].view(-1), optimizer.v[param_index].view(-1)
            if m.numel() != self.connections or m.dtype != torch.float32 or not m.is_cuda:
                raise ValueError("optimizer moments must be float32 CUDA tensors of the weight vector's size")
        lib = _lib.load()
        threshold = torch.zeros((), dtype=torch.float32, device=dev)
        count = torch.zeros((), dtype=torch.int32, device=dev)
        ws = ops._workspace(dev, lib.ffi_rewire_workspace_bytes() + 256)
        off = (-ws.data_ptr()) % 256
        with torch.cuda.device(dev):
            _lib.check(lib.ffi_rewire(w.data_ptr(), self.kernel_indices.data_ptr(),
                                      m.data_ptr() if m is not None else None, v.data_ptr() if v is not None else None,
                                      self.connections, self.in_features, num_selected, ctypes.c_uint64(seed),
                                      threshold.data_ptr(), count.data_ptr(), ws.data_ptr() + off, ws.numel() - off,
                                      ops._stream_ptr(dev)))
        self.kernel_indices.add_(0)  # the table changed behind torch's back: bump its version (plan cache key)
        return threshold, count

    @torch.no_grad()
    def rewire_eager(self, fraction: float = 0.01, optimizer=None, param_index: int = 0, seed: int = 0) -> torch.Tensor:
        """The same step written with plain tensor operations (host restatement of the reference's graph;
        what the tests compare `rewire` with).  Returns the rewired flat positions."""
        from . import synth

        locations = self.rewire_candidates(fraction)
        if locations.numel() == 0:
            return locations
        h = synth.hash64(seed, 0, locations.to("cpu", torch.int64))
        new_sources = (((h >> 1) & ((1 << 63) - 1)) % self.in_features).to(torch.int32)
        self.kernel_indices[locations] = new_sources.to(self.kernel_indices.device)
        if optimizer is not None:
            optimizer.zero_moments(param_index, locations)
        return locations

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, units={self.units}, fan_in={self.fan_in}, bias={self.bias is not None}"
