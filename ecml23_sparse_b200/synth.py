"""Seeded synthetic inputs with the shapes and value distributions of the reference's
workloads (the XMC datasets themselves, run.py:88-93, are not redistributable inputs of
this package).

All randomness comes from a counter-based hash (splitmix64 finaliser) evaluated with
wrapping int64 arithmetic in torch, so the integer streams are identical bits on CPU and
on CUDA; floats derived from them through log/cos may differ in the last place between
devices.
"""
from __future__ import annotations

import math

import torch

_GOLD = -7046029254386353131      # 0x9E3779B97F4A7C15 as int64
_M1 = -4658895280553007687        # 0xBF58476D1CE4E5B9
_M2 = -7723592293110705685        # 0x94D049BB133111EB


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    return (z >> s) & ((1 << (64 - s)) - 1)


def hash64(seed: int, stream: int, counter: torch.Tensor) -> torch.Tensor:
    """splitmix64 of (seed, stream, counter); counter is an int64 tensor."""
    base = (seed * 0x632BE59BD9B4E019 + stream * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF
    if base >= 1 << 63:
        base -= 1 << 64
    z = counter * _GOLD + base
    z = (z ^ _lsr(z, 30)) * _M1
    z = (z ^ _lsr(z, 27)) * _M2
    return z ^ _lsr(z, 31)


def _counter(n: int, device, start: int = 0) -> torch.Tensor:
    return torch.arange(start, start + n, dtype=torch.int64, device=device)


def uniform01(seed: int, stream: int, n: int, device="cpu", start: int = 0) -> torch.Tensor:
    """n float64 values in (0,1) (53 bits, never exactly 0)."""
    h = hash64(seed, stream, _counter(n, device, start))
    return (_lsr(h, 11).to(torch.float64) + 0.5) * (1.0 / (1 << 53))


def uniform_pm1(seed: int, stream: int, shape, device="cpu") -> torch.Tensor:
    """float32 uniform in [-1,1): the distribution of Eigen's Matrix::Random used by the
    reference's tests (testing/test_case_templates.h:54-69)."""
    n = math.prod(shape)
    h = hash64(seed, stream, _counter(n, device))
    u = _lsr(h, 40).to(torch.float32) * (1.0 / (1 << 24))
    return (u * 2 - 1).reshape(shape)


def normal(seed: int, stream: int, shape, std: float = 1.0, device="cpu", start: int = 0) -> torch.Tensor:
    """float32 N(0, std^2) by Box-Muller; `start` offsets the counter (to draw a slice of a larger
    tensor: element j of the slice is element start+j of the whole)."""
    n = math.prod(shape)
    u1 = uniform01(seed, stream, n, device, start)
    u2 = uniform01(seed, stream + 1_000_003, n, device, start)
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
    return (z * std).to(torch.float32).reshape(shape)


def indices_with_replacement(seed: int, stream: int, L: int, K: int, N: int, device="cpu") -> torch.Tensor:
    """int32 [L,K], each entry uniform in [0,N): how the reference draws its table
    (sparse/custom_layer.py:15, testing/test_case_templates.h:59-64); rows may repeat an index."""
    h = hash64(seed, stream, _counter(L * K, device))
    return (_lsr(h, 1) % N).to(torch.int32).reshape(L, K)


def indices_without_replacement(seed: int, stream: int, L: int, K: int, N: int, device="cpu",
                                rows_per_block: int = 32768, row_offset: int = 0) -> torch.Tensor:
    """int32 [L,K]: per row, K distinct inputs drawn uniformly from [0,N) (the K smallest of N
    random keys, listed in key order).  Row r of the result is row row_offset+r of the full table."""
    if K > N:
        raise ValueError("K distinct indices need K <= N")
    out = torch.empty((L, K), dtype=torch.int32, device=device)
    col = torch.arange(N, dtype=torch.int64, device=device)
    for r0 in range(0, L, rows_per_block):
        r1 = min(L, r0 + rows_per_block)
        ctr = (torch.arange(row_offset + r0, row_offset + r1, dtype=torch.int64, device=device)[:, None] * N
               + col[None, :])
        keys = (_lsr(hash64(seed, stream, ctr), 12) << 20) | col[None, :]  # unique within a row
        sel = torch.topk(keys, K, dim=1, largest=False, sorted=True).values
        out[r0:r1] = (sel & ((1 << 20) - 1)).to(torch.int32)
    return out


def multi_hot_targets(seed: int, stream: int, B: int, L: int, device="cpu", zipf_s: float = 1.1,
                      mean_extra: float = 4.0):
    """Sparse multi-hot targets as CSR (row_ptr[B+1], labels[nnz]) int32.

    Per sample 1+Poisson(mean_extra) draws; label ranks are Zipf(zipf_s) over [0,L) and map to
    label ids through a fixed seeded permutation (so that frequent labels spread over the
    label range); duplicates within a sample are dropped; labels of a row come out ascending.
    """
    max_draws = 32
    # Poisson by inversion
    u = uniform01(seed, stream, B, "cpu")
    cdf, p, acc = [], math.exp(-mean_extra), 0.0
    for k in range(max_draws - 1):
        acc += p
        cdf.append(acc)
        p *= mean_extra / (k + 1)
    counts = 1 + torch.searchsorted(torch.tensor(cdf, dtype=torch.float64), u).clamp(max=max_draws - 2)
    # Zipf by inversion of the exact cumulative weights
    w = torch.arange(1, L + 1, dtype=torch.float64).pow(-zipf_s)
    zc = torch.cumsum(w, 0)
    zc /= zc[-1].clone()
    ud = uniform01(seed, stream + 1, B * max_draws, "cpu").reshape(B, max_draws)
    ranks = torch.searchsorted(zc, ud).clamp(max=L - 1)
    perm = torch.argsort(hash64(seed, stream + 2, _counter(L, "cpu")))
    ids = perm[ranks]
    rows, row_ptr = [], [0]
    for b in range(B):
        lab = torch.unique(ids[b, : int(counts[b])])
        rows.append(lab)
        row_ptr.append(row_ptr[-1] + lab.numel())
    labels = torch.cat(rows).to(torch.int32)
    return torch.tensor(row_ptr, dtype=torch.int32).to(device), labels.to(device)
