"""CPU checks of the seeded synthetic input generators."""
import numpy as np
import torch

from ecml23_sparse_b200 import synth


def test_hash_stream_is_stable():
    h = synth.hash64(1, 2, torch.arange(4, dtype=torch.int64))
    assert h.tolist() == synth.hash64(1, 2, torch.arange(4, dtype=torch.int64)).tolist()
    assert len(set(h.tolist())) == 4
    assert synth.hash64(1, 3, torch.arange(4, dtype=torch.int64)).tolist() != h.tolist()


def test_indices_without_replacement_are_distinct_and_in_range():
    idx = synth.indices_without_replacement(5, 0, 300, 32, 768, rows_per_block=128)
    assert idx.dtype == torch.int32 and idx.shape == (300, 32)
    assert int(idx.min()) >= 0 and int(idx.max()) < 768
    assert all(len(set(r.tolist())) == 32 for r in idx)
    again = synth.indices_without_replacement(5, 0, 300, 32, 768, rows_per_block=77)
    assert torch.equal(idx, again), "result must not depend on the blocking"
    counts = np.bincount(idx.numpy().ravel(), minlength=768)
    assert counts.min() > 0 and counts.max() < 40  # roughly uniform: mean 12.5


def test_indices_with_replacement_range():
    idx = synth.indices_with_replacement(5, 1, 100, 7, 13)
    assert int(idx.min()) >= 0 and int(idx.max()) < 13


def test_normal_moments():
    x = synth.normal(9, 0, (200_000,), std=0.25)
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 0.25) < 5e-3


def test_multi_hot_targets_csr():
    B, L = 64, 10_000
    row_ptr, labels = synth.multi_hot_targets(3, 0, B, L)
    assert row_ptr.shape == (B + 1,) and int(row_ptr[0]) == 0 and int(row_ptr[-1]) == labels.numel()
    assert int(labels.min()) >= 0 and int(labels.max()) < L
    for b in range(B):
        row = labels[int(row_ptr[b]):int(row_ptr[b + 1])].tolist()
        assert len(row) >= 1 and row == sorted(set(row))
    mean = labels.numel() / B
    assert 3.0 < mean < 6.5  # 1 + Poisson(4), minus duplicates
