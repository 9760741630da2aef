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

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, units={self.units}, fan_in={self.fan_in}, bias={self.bias is not None}"
