"""CPU tests of the layer's host-side logic (initialisation and rewiring); no kernels involved."""
import numpy as np
import torch

from ecml23_sparse_b200.layer import FFILayer


def test_layer_state_matches_reference_layout():
    layer = FFILayer(in_features=50, units=40, fan_in=6, seed=1)
    assert layer.kernel_indices.shape == (240,) and layer.kernel_indices.dtype == torch.int32
    assert layer.kernel_weights.shape == (240,)
    assert layer.lookup().shape == (40, 6) and layer.weights().shape == (40, 6)
    assert int(layer.kernel_indices.min()) >= 0 and int(layer.kernel_indices.max()) < 50
    assert torch.count_nonzero(layer.bias) == 0  # zeros initialiser (sparse/layer.py:112,199-207)
    limit = (6.0 / (2 * 240)) ** 0.5             # glorot_uniform over the flat [connections] variable
    assert float(layer.kernel_weights.abs().max()) <= limit


def test_rewire_candidates_follow_fixed_fraction_selector():
    # numpy restatement of FixedFractionSelector.select (sparse/layer.py:73-86)
    layer = FFILayer(in_features=30, units=100, fan_in=8, seed=2)
    w = layer.kernel_weights.detach().numpy()
    for fraction in (0.01, 0.1, 0.5):
        k = int(round(fraction * w.size))
        threshold = np.sort(np.abs(w))[k - 1]
        expected = np.nonzero(np.abs(w) < threshold)[0]
        got = layer.rewire_candidates(fraction).numpy()
        assert np.array_equal(got, expected)
        assert len(got) == k - 1  # strict "<": the threshold element itself stays
    assert layer.rewire_candidates(0.0).numel() == 0


def test_rewire_changes_only_selected_sources_and_zeroes_moments():
    class Moments:
        def __init__(self, n):
            self.m = [torch.ones(n)]
            self.v = [torch.ones(n)]

        def zero_moments(self, index, locations):
            self.m[index][locations] = 0
            self.v[index][locations] = 0

    layer = FFILayer(in_features=30, units=100, fan_in=8, seed=3)
    before_idx = layer.kernel_indices.clone()
    before_w = layer.kernel_weights.detach().clone()
    version = layer.kernel_indices._version
    opt = Moments(800)
    locs = layer.rewire_eager(0.1, optimizer=opt, seed=5)
    assert locs.numel() == 79
    untouched = torch.ones(800, dtype=torch.bool)
    untouched[locs] = False
    assert torch.equal(layer.kernel_indices[untouched], before_idx[untouched])
    assert int(layer.kernel_indices.min()) >= 0 and int(layer.kernel_indices.max()) < 30
    assert torch.equal(layer.kernel_weights.detach(), before_w)          # weights are kept
    assert layer.kernel_indices._version > version                        # cached plans become stale
    assert float(opt.m[0][locs].abs().sum()) == 0 and float(opt.v[0][locs].abs().sum()) == 0
    assert float(opt.m[0][untouched].min()) == 1
    # the device entry point refuses a layer that lives on the host: there is no CPU path
    import pytest
    with pytest.raises(ValueError, match="CUDA"):
        layer.rewire(0.1)
