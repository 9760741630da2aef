"""Shared test inputs: the reference's size fixtures and seeded input recipes."""
from __future__ import annotations

import os

import numpy as np
import torch

from ecml23_sparse_b200 import synth

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# (B, N, L, K) = (InRows, InCols, OutCols, NNZ) of the reference's TestConfigurations
# (testing/test.cpp:50-59).
REFERENCE_SIZES = [
    (3, 5, 4, 2),
    (12, 8, 8, 4),
    (127, 254, 513, 4),
    (12, 8, 32, 16),
    (17, 12, 63, 44),
    (127, 254, 513, 73),
    (127, 254, 513, 80),
    (1, 32, 4_000_000, 4),
]
SMALL_SIZES = REFERENCE_SIZES[:-1]
HUGE_SIZE = REFERENCE_SIZES[-1]

# The reference's known-answer forward case (testing/test.cpp:13-47).
KAT_X = np.array([[1, 2, 3], [4, 5, 6], [0, 1, 1]], np.float32)
KAT_IDX = np.array([[1, 2], [0, 2]], np.int32)
KAT_W = np.array([[1, 2], [3, 4]], np.float32)
KAT_Y = np.array([[8, 15], [17, 36], [3, 4]], np.float32)


# Bounded device-side waits that tests made run out on purpose (a flag nothing sets); the suite's last
# test checks that no other wait gave up.
EXPECTED_WAIT_TIMEOUTS = 0

# fp32 results against the fp64 oracle: |d| <= ATOL + RTOL*|ref|
RTOL = 1e-5
ATOL = 1e-5


def gx_atol(L, K, N, term_rms=0.25):
    """Absolute floor for grad_x.  grad_x[b,i] sums n = L*K/N products W*g; the rounding error of any
    fp32 summation grows like sqrt(n) times the size of the summands, independently of how close to
    zero the total lands, so the 1e-5 floor (meant for O(1) sums of a few terms) is widened by
    sqrt(n)/32 once n exceeds 1024, and in proportion to the summands' scale where that exceeds the
    0.25 of the benchmark's distributions (W ~ N(0, 1/K) with K >= 16, g ~ N(0,1)).  The reference's
    own fp32 running sum is further from the fp64 value than this (checked on the 4,000,000-unit
    fixture in test_gpu_parity.py)."""
    n = L * K / N
    return ATOL * max(1.0, n ** 0.5 / 32.0) * max(1.0, term_rms / 0.25)


def size_id(size) -> str:
    return "B{}_N{}_L{}_K{}".format(*size)


def reference_style_inputs(size, seed: int = 42, relu_grad: bool = True):
    """Inputs with the distributions of the reference's random tests
    (testing/test_case_templates.h:54-69,100-123): features, weights and out_grad uniform in
    [-1,1), indices uniform in [0,N) with replacement, negative out_grad entries zeroed."""
    B, N, L, K = size
    x = synth.uniform_pm1(seed, 1, (B, N)).numpy()
    idx = synth.indices_with_replacement(seed, 2, L, K, N).numpy()
    W = synth.uniform_pm1(seed, 3, (L, K)).numpy()
    g = synth.uniform_pm1(seed, 4, (B, L)).numpy()
    if relu_grad:
        g = np.where(g < 0, 0, g).astype(np.float32)
    return x, idx, W, g


def config_style_inputs(B, N, L, K, seed: int = 7, w_var_scale: float = 1.0):
    """Inputs with the distributions of the benchmark configurations: x ~ N(0,1), K distinct
    indices per row, W ~ N(0, w_var_scale/K), g ~ N(0,1)."""
    x = synth.normal(seed, 11, (B, N)).numpy()
    idx = synth.indices_without_replacement(seed, 12, L, K, N).numpy()
    W = synth.normal(seed, 13, (L, K), std=(w_var_scale / K) ** 0.5).numpy()
    g = synth.normal(seed, 15, (B, L)).numpy()
    return x, idx, W, g


def golden_path(size) -> str:
    return os.path.join(GOLDEN_DIR, size_id(size) + ".npz")


def assert_close(actual, expected, rtol=1e-5, atol=1e-5, what=""):
    """|actual - expected| <= atol + rtol*|expected| elementwise (two-sided, unlike the reference's
    one-sided maxCoeff checks, testing/test_case_templates.h:82,139-140)."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    assert actual.shape == expected.shape, f"{what}: shape {actual.shape} vs {expected.shape}"
    err = np.abs(actual - expected)
    bound = atol + rtol * np.abs(expected)
    bad = err > bound
    if bad.any():
        j = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} elements off; worst at {j}: "
                             f"{actual[j]!r} vs {expected[j]!r} (err {err[j]:.3e}, bound {bound[j]:.3e})")


def to_cuda(a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(device)
