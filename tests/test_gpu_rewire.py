"""GPU test of one rewiring step on the device (`ffi_rewire` through `FFILayer.rewire`) against the
numpy restatement of the reference's graph: FixedFractionSelector.select (sparse/layer.py:62-86),
StratifiedRewireLayerV2._rewire and _update_sparse_kernel (sparse/custom_layer.py:20-43).

Integer and index work: the selected set, the new index table, the zeroed moments and the transposed
index rebuilt afterwards are compared bit for bit.
"""
import numpy as np
import pytest
import torch

import oracle
import ecml23_sparse_b200 as ffi
from ecml23_sparse_b200 import synth
from ecml23_sparse_b200.layer import _num_selected

pytestmark = pytest.mark.gpu


def numpy_rewire(w, idx, m, v, n_in, fraction, seed):
    """The reference's rewiring step on host arrays; returns (threshold, selected positions)."""
    n = w.size
    k = _num_selected(fraction, n)
    if k < 1:
        return 0.0, np.empty(0, np.int64)
    a = np.abs(w)
    threshold = np.partition(a, k - 1)[k - 1]          # the k-th smallest |w| (top_k of -|w|, last value)
    sel = np.nonzero(a < threshold)[0]                  # tf.less: strict
    h = synth.hash64(seed, 0, torch.from_numpy(sel.astype(np.int64))).numpy()
    idx[sel] = (((h >> 1) & ((1 << 63) - 1)) % n_in).astype(np.int32)
    m[sel] = 0
    v[sel] = 0
    return float(threshold), sel


@pytest.mark.parametrize("shape,fraction", [((96, 500, 12), 0.1), ((768, 20_011, 32), 0.01), ((64, 1000, 8), 0.5),
                                            ((30, 100, 8), 0.0), ((768, 670_091, 32), 0.01)],
                         ids=["small", "headline-rows-20k", "half", "none", "headline-full"])
def test_rewire_step_matches_host_restatement(cuda_device, shape, fraction):
    dev = cuda_device
    n_in, units, fan_in = shape
    layer = ffi.FFILayer(in_features=n_in, units=units, fan_in=fan_in, device=dev, seed=7)
    n = units * fan_in
    with torch.no_grad():
        # weights with repeated magnitudes and exact zeros, so that ties at the threshold occur
        w0 = synth.normal(3, 1, (n,), std=0.05, device=dev)
        w0[::17] = 0.0
        twin = w0[2::13]
        w0[1::13][: twin.numel()] = twin.abs()[: w0[1::13].numel()]
        layer.kernel_weights.copy_(w0)
    opt = ffi.FusedAdam([layer.kernel_weights], lr=1e-3)
    opt.m[0].copy_(synth.normal(3, 2, (n,), device=dev))
    opt.v[0].copy_(synth.normal(3, 3, (n,), device=dev).abs())

    w_h = layer.kernel_weights.detach().cpu().numpy().copy()
    idx_h = layer.kernel_indices.cpu().numpy().copy()
    m_h, v_h = opt.m[0].cpu().numpy().copy(), opt.v[0].cpu().numpy().copy()
    version = layer.kernel_indices._version
    plan_before = layer.plan()
    plan_before.rebuild(layer.lookup())  # a first in-place rebuild allocates the plan's sort scratch

    thr, count = layer.rewire(fraction, optimizer=opt, seed=11)
    thr_ref, sel = numpy_rewire(w_h, idx_h, m_h, v_h, n_in, fraction, seed=11)

    assert int(count) == sel.size
    if sel.size or _num_selected(fraction, n) > 0:
        assert float(thr) == np.float32(thr_ref)
    assert np.array_equal(layer.kernel_indices.cpu().numpy(), idx_h)
    assert np.array_equal(opt.m[0].cpu().numpy(), m_h) and np.array_equal(opt.v[0].cpu().numpy(), v_h)
    assert np.array_equal(layer.kernel_weights.detach().cpu().numpy(), w_h)      # weights are kept
    if _num_selected(fraction, n) > 0:
        assert sel.size <= _num_selected(fraction, n) - 1 + 0                     # strict "<": the threshold stays
        assert layer.kernel_indices._version > version
        # the cached plan is stale now; the next one is rebuilt from the new table, bit-exact
        builds = plan_before.builds
        plan_after = layer.plan()
        assert plan_after is plan_before and plan_after.builds == builds + 1   # rebuilt in place
        rowptr, perm = plan_after.export()
        exp_rowptr, exp_perm = oracle.transpose_index(idx_h.reshape(units, fan_in), n_in)
        assert np.array_equal(rowptr.cpu().numpy(), exp_rowptr)
        assert np.array_equal(perm.cpu().numpy(), exp_perm)


def test_rewire_then_backward_uses_the_new_table(cuda_device):
    """After a rewiring step the layer's gradients follow the new index table."""
    dev = cuda_device
    layer = ffi.FFILayer(in_features=256, units=3_000, fan_in=16, device=dev, seed=9)
    with torch.no_grad():
        layer.kernel_weights.copy_(synth.normal(4, 1, (3_000 * 16,), std=0.1, device=dev))
    x = synth.normal(4, 0, (64, 256)).numpy()
    g = synth.normal(4, 5, (64, 3_000)).numpy()

    def grads():
        xt = torch.from_numpy(x).to(dev).requires_grad_()
        layer.zero_grad()
        layer(xt).backward(torch.from_numpy(g).to(dev))
        return xt.grad.cpu().numpy(), layer.kernel_weights.grad.view(3_000, 16).cpu().numpy()

    grads()  # builds and caches the plan of the old table
    layer.rewire(0.2, seed=1)
    gx, gw = grads()
    idx = layer.lookup().cpu().numpy()
    W = layer.weights().detach().cpu().numpy()
    from cases import ATOL, RTOL, assert_close, gx_atol
    assert_close(gx, oracle.grad_x_f64(idx, W, g, 256), RTOL, gx_atol(3_000, 16, 256), "grad_x after rewiring")
    assert_close(gw, oracle.grad_w_f64(x, idx, g), RTOL, ATOL, "grad_W after rewiring")
