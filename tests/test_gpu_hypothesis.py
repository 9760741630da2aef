"""Property-based GPU parity on small random shapes: any (B, N, L, K), both layouts, indices with
replacement (duplicates inside a row are legal and add), fp32 and bf16 storage, against the fp64 oracle.
The shapes are drawn so that every dispatch branch with small inputs is hit: K not a multiple of 4,
batches around the 32 / 64 / 128 tile edges, N of a few units up to a few hundred."""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

import oracle
from ecml23_sparse_b200 import ops, synth
from cases import ATOL, RTOL, assert_close, gx_atol, to_cuda

pytestmark = pytest.mark.gpu

shapes = st.tuples(
    st.sampled_from([1, 2, 7, 31, 32, 33, 63, 64, 65, 100, 127, 128, 129, 150]),   # B
    st.integers(min_value=1, max_value=300),                                       # N
    st.integers(min_value=1, max_value=260),                                       # L
    st.sampled_from([1, 2, 3, 4, 5, 8, 12, 16, 24, 31, 32, 33, 40]),               # K
)


@settings(max_examples=60, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
@given(shape=shapes, transposed=st.booleans(), bf16=st.booleans(), seed=st.integers(min_value=0, max_value=10_000))
def test_random_small_shapes_match_the_oracle(cuda_device, shape, transposed, bf16, seed):
    dev = cuda_device
    B, N, L, K = shape
    x = synth.uniform_pm1(seed, 1, (B, N)).numpy()
    idx = synth.indices_with_replacement(seed, 2, L, K, N).numpy()
    W = synth.uniform_pm1(seed, 3, (L, K)).numpy()
    g = synth.uniform_pm1(seed, 4, (B, L)).numpy()
    bias = synth.uniform_pm1(seed, 5, (L,)).numpy()
    if bf16:
        x = torch.from_numpy(x).to(torch.bfloat16).float().numpy()   # the rounded values, exactly
        W = torch.from_numpy(W).to(torch.bfloat16).float().numpy()
    store = torch.bfloat16 if bf16 else torch.float32
    xin = to_cuda(np.ascontiguousarray(x.T) if transposed else x, dev).to(store)
    Wd = to_cuda(W, dev).to(store)
    y = ops._forward(xin, to_cuda(idx, dev), Wd, to_cuda(bias, dev), transposed)
    gx, gw, gb = ops._backward(xin, to_cuda(idx, dev), Wd, to_cuda(g, dev), transposed, want_bias_grad=True)
    what = f"B{B} N{N} L{L} K{K} tp={transposed} bf16={bf16}"
    assert_close(y.cpu().numpy(), oracle.forward_f64(x, idx, W, bias=bias), RTOL, ATOL, what + " y")
    assert_close(gw.cpu().numpy(), oracle.grad_w_f64(x, idx, g), RTOL, ATOL, what + " grad_W")
    gxn = gx.cpu().numpy().T if transposed else gx.cpu().numpy()
    assert_close(gxn, oracle.grad_x_f64(idx, W, g, N), RTOL, gx_atol(L, K, N, term_rms=0.5), what + " grad_x")
    assert_close(gb.cpu().numpy(), oracle.grad_bias_f64(g), RTOL, ATOL * max(1.0, B ** 0.5 / 4), what + " grad_bias")
