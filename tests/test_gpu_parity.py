"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle, the golden
fixtures produced by the reference's own CPU kernels, and size-independent properties.

Tolerances: fp32 results within |d| <= 1e-5 + 1e-5*|ref| of the fp64 oracle; against the
reference's fp32 goldens the reference's own bounds apply (1e-5 forward, 1.5e-5 backward,
testing/test_case_templates.h:82,139-140) plus the same relative term.  The transposed index
is compared bit for bit.
"""
import numpy as np
import pytest
import torch

import oracle
import ecml23_sparse_b200 as ffi
from ecml23_sparse_b200 import _lib, synth
from cases import (ATOL, HUGE_SIZE, KAT_IDX, KAT_W, KAT_X, KAT_Y, RTOL, SMALL_SIZES, assert_close, config_style_inputs,
                   golden_path, gx_atol, reference_style_inputs, size_id, to_cuda)

pytestmark = pytest.mark.gpu

def run_forward(dev, x, idx, W, transposed, bias=None):
    xin = np.ascontiguousarray(x.T) if transposed else x
    fn = ffi.fan_in_sparse_matmul_tp if transposed else ffi.fan_in_sparse_matmul
    if bias is None:
        return fn(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev)).cpu().numpy()
    op = ffi.ffi_matmul_tp if transposed else ffi.ffi_matmul
    return op(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(bias, dev)).cpu().numpy()


def run_backward(dev, x, idx, W, g, transposed):
    xin = np.ascontiguousarray(x.T) if transposed else x
    fn = ffi.fan_in_sparse_matmul_grad_tp if transposed else ffi.fan_in_sparse_matmul_grad
    gx, gw = fn(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(g, dev))
    gx = gx.cpu().numpy()
    return (gx.T if transposed else gx), gw.cpu().numpy()


def check_against_oracle(dev, x, idx, W, g, transposed, what=""):
    B, N = x.shape
    y = run_forward(dev, x, idx, W, transposed)
    assert_close(y, oracle.forward_f64(x, idx, W), RTOL, ATOL, what + " y")
    gx, gw = run_backward(dev, x, idx, W, g, transposed)
    assert_close(gw, oracle.grad_w_f64(x, idx, g), RTOL, ATOL, what + " grad_W")
    L, K = idx.shape
    assert_close(gx, oracle.grad_x_f64(idx, W, g, N), RTOL, gx_atol(L, K, N), what + " grad_x")
    return y, gx, gw


@pytest.mark.parametrize("transposed", [False, True], ids=["plain", "tp"])
def test_known_answer_forward_exact(cuda_device, transposed):
    # testing/test.cpp:13-47: exact equality, both layouts
    y = run_forward(cuda_device, KAT_X, KAT_IDX, KAT_W, transposed)
    assert np.array_equal(y, KAT_Y)


@pytest.mark.parametrize("size", SMALL_SIZES, ids=size_id)
@pytest.mark.parametrize("transposed", [False, True], ids=["plain", "tp"])
def test_reference_fixtures(cuda_device, size, transposed):
    x, idx, W, g = reference_style_inputs(size)
    y, gx, gw = check_against_oracle(cuda_device, x, idx, W, g, transposed, size_id(size))
    gold = np.load(golden_path(size))
    assert_close(y, gold["y"], RTOL, 1e-5, "y vs reference golden")
    assert_close(gw, gold["grad_w"], RTOL, 1.5e-5, "grad_W vs reference golden")
    assert_close(gx, gold["grad_x"], 2e-5, 1.5e-5, "grad_x vs reference golden")


def test_reference_fixture_four_million_units(cuda_device):
    # (1, 32, 4,000,000, 4): the fixture on which the reference's clamped grid skips units
    # (tfsparse/cc/kernels/kernel_data.cu.h:125-143); every unit must be written here.
    x, idx, W, g = reference_style_inputs(HUGE_SIZE)
    B, N, L, K = HUGE_SIZE
    gold = np.load(golden_path(HUGE_SIZE))
    s = int(gold["sample_stride"])
    for transposed in (False, True):
        y = run_forward(cuda_device, x, idx, W, transposed)
        assert_close(y, oracle.forward_f64(x, idx, W), RTOL, ATOL, "y")
        assert_close(y.ravel()[::s], gold["y_sample"], RTOL, 1e-5, "y vs golden sample")
        gx, gw = run_backward(cuda_device, x, idx, W, g, transposed)
        assert_close(gw, oracle.grad_w_f64(x, idx, g), RTOL, ATOL, "grad_W")
        assert_close(gw.ravel()[::s], gold["grad_w_sample"], RTOL, 1.5e-5, "grad_W vs golden sample")
        gx64 = oracle.grad_x_f64(idx, W, g, N)
        assert_close(gx, gx64, RTOL, gx_atol(L, K, N), "grad_x")
        # the reference's own fp32 running sum of 500,000 terms carries ~1e-4 relative error ...
        assert_close(gx, gold["grad_x"], 5e-4, 1.5e-5, "grad_x vs golden")
        # ... and is further from the fp64 value than the CUDA result is
        assert np.abs(gx - gx64).max() <= np.abs(gold["grad_x"] - gx64).max()


EXTRA_SHAPES = [
    # (B, N, L, K)  fan-ins around the vector widths, odd sizes, batch tile edges
    (5, 7, 33, 1), (9, 10, 50, 3), (31, 129, 300, 32), (33, 130, 301, 33), (64, 64, 257, 64),
    (65, 255, 1000, 72), (128, 768, 2049, 32), (129, 100, 513, 5), (200, 37, 700, 12), (2, 2, 1, 2),
    (32, 768, 20_011, 32), (128, 768, 20_011, 32), (256, 512, 4_099, 32),
    # batch 65..128 takes the half-warp backward: partial last slice, many slices, long and short runs
    (100, 300, 5_000, 16), (96, 130, 777, 8), (128, 64, 4_000, 4), (127, 2_000, 3_000, 32), (66, 768, 511, 64),
]


@pytest.mark.parametrize("shape", EXTRA_SHAPES, ids=size_id)
@pytest.mark.parametrize("transposed", [False, True], ids=["plain", "tp"])
def test_extra_shapes(cuda_device, shape, transposed):
    x, idx, W, g = reference_style_inputs(shape, seed=sum(shape), relu_grad=False)
    check_against_oracle(cuda_device, x, idx, W, g, transposed, size_id(shape))


@pytest.mark.parametrize("shape", [(16, 5000, 3000, 8), (130, 3000, 2000, 16), (40, 2500, 1500, 7), (1, 60_000, 5, 4),
                                   (33, 7_000, 9, 36), (129, 2_500, 41, 8), (64, 3_300, 1_001, 72), (257, 1_200, 300, 12)],
                         ids=size_id)
@pytest.mark.parametrize("transposed", [False, True], ids=["plain", "tp"])
def test_wide_inputs(cuda_device, shape, transposed):
    # N too large for the shared-memory x tile / register accumulators: the global-memory paths
    x, idx, W, g = reference_style_inputs(shape, seed=11, relu_grad=False)
    check_against_oracle(cuda_device, x, idx, W, g, transposed, size_id(shape))


def test_benchmark_distribution_inputs(cuda_device):
    B, N, L, K = 128, 768, 30_000, 32
    x, idx, W, g = config_style_inputs(B, N, L, K)
    check_against_oracle(cuda_device, x, idx, W, g, True, "config-style")


def test_uint32_indices_and_duplicates(cuda_device):
    dev = cuda_device
    x, idx, W, g = reference_style_inputs((17, 12, 63, 44))
    idx[:, 1] = idx[:, 0]  # force duplicates inside every row
    y32 = ffi.fan_in_sparse_matmul(to_cuda(x, dev), to_cuda(idx, dev), to_cuda(W, dev))
    if hasattr(torch, "uint32"):
        yu = ffi.fan_in_sparse_matmul(to_cuda(x, dev), to_cuda(idx, dev).view(torch.uint32), to_cuda(W, dev))
        assert torch.equal(y32, yu)
    assert_close(y32.cpu().numpy(), oracle.forward_f64(x, idx, W), RTOL, ATOL, "y with duplicates")
    gx, gw = run_backward(dev, x, idx, W, g, False)
    assert_close(gx, oracle.grad_x_f64(idx, W, g, 12), RTOL, ATOL, "grad_x with duplicates")
    assert_close(gw, oracle.grad_w_f64(x, idx, g), RTOL, ATOL, "grad_W with duplicates")


def test_fused_bias_and_grad_bias(cuda_device):
    dev = cuda_device
    x, idx, W, g = reference_style_inputs((65, 255, 1000, 72), relu_grad=False)
    bias = np.linspace(-2, 2, 1000).astype(np.float32)
    for transposed in (False, True):
        y = run_forward(dev, x, idx, W, transposed, bias=bias)
        assert_close(y, oracle.forward_f64(x, idx, W, bias=bias), RTOL, ATOL, "y + bias")
    xt, it, wt, bt = to_cuda(x, dev).requires_grad_(), to_cuda(idx, dev), to_cuda(W, dev).requires_grad_(), \
        to_cuda(bias, dev).requires_grad_()
    out = ffi.ffi_matmul(xt, it, wt, bt)
    out.backward(to_cuda(g, dev))
    assert_close(bt.grad.cpu().numpy(), oracle.grad_bias_f64(g), RTOL, ATOL, "grad_bias")
    assert_close(wt.grad.cpu().numpy(), oracle.grad_w_f64(x, idx, g), RTOL, ATOL, "grad_W (autograd)")
    assert_close(xt.grad.cpu().numpy(), oracle.grad_x_f64(idx, W, g, 255), RTOL, ATOL, "grad_x (autograd)")


@pytest.mark.parametrize("shape", [(3, 5, 4, 2), (17, 12, 63, 44), (4, 300, 1000, 7), (8, 768, 5000, 32),
                                   (2, 70_000, 3000, 4)], ids=size_id)
def test_transposed_index_bit_exact(cuda_device, shape):
    B, N, L, K = shape
    idx = reference_style_inputs(shape)[1]
    plan = ffi.FFIPlan(to_cuda(idx, cuda_device), N)
    rowptr, perm = plan.export()
    exp_rowptr, exp_perm = oracle.transpose_index(idx, N)
    assert np.array_equal(rowptr.cpu().numpy(), exp_rowptr)
    assert np.array_equal(perm.cpu().numpy(), exp_perm)
    info = plan.info()
    assert (info["L"], info["K"], info["N"]) == (L, K, N)
    if info["chunk_rows"] > 0:
        rowptr_c, perm_c = plan.export(chunked=True)
        assert np.array_equal(rowptr_c.cpu().numpy(), exp_rowptr)
        assert np.array_equal(perm_c.cpu().numpy(), exp_perm)
    else:
        assert N > 2048
    plan.close()


def test_plan_rejects_out_of_range_index_and_stale_shape(cuda_device):
    dev = cuda_device
    bad = torch.tensor([[0, 9]], dtype=torch.int32, device=dev)
    with pytest.raises(_lib.FFIError) as e:
        ffi.FFIPlan(bad, 9)
    assert e.value.status == 6
    x, idx, W, g = reference_style_inputs((12, 8, 32, 16))
    plan = ffi.FFIPlan(to_cuda(idx, dev), 8)
    from ecml23_sparse_b200.ops import _backward
    with pytest.raises(_lib.FFIError) as e:
        _backward(to_cuda(x[:, :7].copy(), dev), to_cuda(idx % 7, dev), to_cuda(W, dev), to_cuda(g, dev), False, plan=plan)
    assert e.value.status == 5


def test_debug_bounds_mode_rejects_bad_indices_before_any_kernel_runs(cuda_device):
    """With debug bounds on, an index outside [0, N) makes forward / fused loss / backward return
    FFI_ERR_INDEX_RANGE without launching their kernels (the status-code counterpart of the reference's
    audit-mode index asserts, tfsparse/cc/kernels/kernel_data.cu.h:26-43,211)."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    lib = _lib.load()
    x, idx, W, g = reference_style_inputs((12, 8, 32, 16))
    good = to_cuda(idx, dev)
    bad = good.clone()
    bad[5, 3] = 8            # N = 8: one past the end
    row_ptr, labels = synth.multi_hot_targets(1, 2, 12, 32)
    plan = ffi.FFIPlan(good, 8)
    _lib.check(lib.ffi_set_debug_bounds(1))
    try:
        y = ops._forward(to_cuda(x, dev), good, to_cuda(W, dev), None, False)   # a valid table passes
        assert_close(y.cpu().numpy(), oracle.forward_f64(x, idx, W), RTOL, ATOL, "y with debug bounds on")
        for call in (lambda: ops._forward(to_cuda(x, dev), bad, to_cuda(W, dev), None, False),
                     lambda: ops.forward_bce(to_cuda(x, dev), bad, to_cuda(W, dev), None, row_ptr, labels, False),
                     lambda: ops._backward(to_cuda(x, dev), bad, to_cuda(W, dev), to_cuda(g, dev), False, plan=plan)):
            with pytest.raises(_lib.FFIError) as e:
                call()
            assert e.value.status == 6
    finally:
        _lib.check(lib.ffi_set_debug_bounds(0))


def test_plan_cache_follows_tensor_version(cuda_device):
    dev = cuda_device
    x, idx, W, g = reference_style_inputs((12, 8, 32, 16))
    it = to_cuda(idx, dev)
    p1 = ffi.get_plan(it, 8)
    assert ffi.get_plan(it, 8) is p1
    it[0, 0] = (it[0, 0] + 1) % 8  # rewiring: in-place update bumps the version
    p2 = ffi.get_plan(it, 8)
    assert p2 is p1 and p1.builds == 2  # rebuilt in place from the changed table
    gx, _ = ffi.fan_in_sparse_matmul_grad(to_cuda(x, dev), it, to_cuda(W, dev), to_cuda(g, dev))
    assert_close(gx.cpu().numpy(), oracle.grad_x_f64(it.cpu().numpy(), W, g, 8), RTOL, ATOL, "grad_x after rewiring")


def test_backward_is_bit_reproducible(cuda_device):
    dev = cuda_device
    x, idx, W, g = config_style_inputs(128, 768, 10_000, 32)
    args = [to_cuda(np.ascontiguousarray(x.T), dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(g, dev)]
    gx1, gw1 = ffi.fan_in_sparse_matmul_grad_tp(*args)
    gx2, gw2 = ffi.fan_in_sparse_matmul_grad_tp(*args)
    assert torch.equal(gx1, gx2) and torch.equal(gw1, gw2)


def test_sigmoid_bce_gradient(cuda_device):
    dev = cuda_device
    B, L = 37, 5003
    z = (synth.normal(5, 0, (B, L)) * 3).numpy()
    row_ptr, labels = synth.multi_hot_targets(5, 1, B, L)
    loss_ref, g_ref = oracle.bce_f64(z, row_ptr.numpy(), labels.numpy())
    loss, g = ffi.sparse_bce_with_logits(to_cuda(z, dev), row_ptr, labels)
    assert abs(float(loss) - loss_ref) <= 1e-5 * abs(loss_ref) + 1e-7
    assert_close(g.cpu().numpy(), g_ref, 2e-5, 1e-12, "bce grad")
    # label shard: columns [1000, 3000) of the same problem
    lo, hi = 1000, 3000
    zs = np.ascontiguousarray(z[:, lo:hi])
    loss_s, g_s = ffi.sparse_bce_with_logits(to_cuda(zs, dev), row_ptr, labels, total_labels=L, label_offset=lo)
    assert_close(g_s.cpu().numpy(), g_ref[:, lo:hi], 2e-5, 1e-12, "bce grad (shard)")
    # in place
    zt = to_cuda(z, dev)
    _, g_in = ffi.sparse_bce_with_logits(zt, row_ptr, labels, inplace=True)
    assert g_in.data_ptr() == zt.data_ptr() and torch.equal(g_in, g)


@pytest.mark.parametrize("n", [1, 7, 4096, 100_003])
def test_fused_adam_matches_oracle(cuda_device, n):
    dev = cuda_device
    w0 = synth.normal(1, 0, (n,)).numpy()
    w = to_cuda(w0.copy(), dev)
    opt = ffi.FusedAdam([w], lr=1e-3, beta_1=0.9, beta_2=0.999, epsilon=1e-7)
    # Keras holds the hyper-parameters in the variable's dtype: the oracle gets them rounded to fp32
    lr, b1, b2, eps = (float(np.float32(v)) for v in (1e-3, 0.9, 0.999, 1e-7))
    wr, mr, vr = w0.astype(np.float64), np.zeros(n), np.zeros(n)
    for step in range(1, 4):
        grad = synth.normal(2, step, (n,)).numpy()
        opt.step([to_cuda(grad, dev)])
        wr, mr, vr = oracle.adam_f64(wr, mr, vr, grad.astype(np.float64), lr, b1, b2, eps, step)
    assert opt.iterations == 3
    assert_close(w.cpu().numpy(), wr, 1e-5, 1e-6, "adam w")
    assert_close(opt.m[0].cpu().numpy(), mr, 1e-5, 1e-7, "adam m")
    assert_close(opt.v[0].cpu().numpy(), vr, 1e-5, 1e-9, "adam v")


@pytest.mark.parametrize("n", [5, 4096, 100_003])
def test_fused_adam_on_bf16_weights(cuda_device, n):
    """bf16 storage of W (benchmark configurations 2-4): m, v and the update are fp32, the new weight is rounded
    to bf16 once.  Against the fp64 oracle on the same bf16 starting point: m and v to fp32 accuracy, w within
    one bf16 rounding step (2^-8 relative) of the oracle's unrounded value."""
    dev = cuda_device
    w0 = synth.normal(1, 0, (n,)).to(torch.bfloat16)
    w = w0.clone().to(dev)
    opt = ffi.FusedAdam([w], lr=1e-3, beta_1=0.9, beta_2=0.999, epsilon=1e-7)
    lr, b1, b2, eps = (float(np.float32(v)) for v in (1e-3, 0.9, 0.999, 1e-7))
    wr, mr, vr = w0.double().numpy(), np.zeros(n), np.zeros(n)
    for step in range(1, 4):
        grad = synth.normal(2, step, (n,)).numpy()
        w_before = w.double().cpu().numpy()
        opt.step([to_cuda(grad, dev)])
        # the oracle restarts from the device's rounded weights, so that rounding does not accumulate between steps
        wr, mr, vr = oracle.adam_f64(w_before, mr, vr, grad.astype(np.float64), lr, b1, b2, eps, step)
        got = w.double().cpu().numpy()
        assert np.all(np.abs(got - wr) <= np.abs(wr) * 2.0 ** -8 + 1e-30), "bf16 weight further than one rounding step"
    assert w.dtype == torch.bfloat16
    assert_close(opt.m[0].cpu().numpy(), mr, 1e-5, 1e-7, "adam m (bf16 W)")
    assert_close(opt.v[0].cpu().numpy(), vr, 1e-5, 1e-9, "adam v (bf16 W)")


def test_layer_module_matches_oracle(cuda_device):
    dev = cuda_device
    layer = ffi.FFILayer(in_features=96, units=500, fan_in=12, device=dev, seed=3)
    with torch.no_grad():
        layer.bias.copy_(torch.linspace(-1, 1, 500, device=dev))
    x = synth.normal(4, 0, (20, 96)).numpy()
    xt = to_cuda(x, dev).requires_grad_()
    y = layer(xt)
    idx = layer.lookup().cpu().numpy()
    W = layer.weights().detach().cpu().numpy()
    bias = layer.bias.detach().cpu().numpy()
    assert_close(y.detach().cpu().numpy(), oracle.forward_f64(x, idx, W, bias=bias), RTOL, ATOL, "layer y")
    g = synth.normal(4, 1, (20, 500)).numpy()
    y.backward(to_cuda(g, dev))
    assert_close(xt.grad.cpu().numpy(), oracle.grad_x_f64(idx, W, g, 96), RTOL, ATOL, "layer grad_x")
    assert_close(layer.kernel_weights.grad.view(500, 12).cpu().numpy(), oracle.grad_w_f64(x, idx, g), RTOL, ATOL,
                 "layer grad_W")
    assert_close(layer.bias.grad.cpu().numpy(), oracle.grad_bias_f64(g), RTOL, ATOL, "layer grad_bias")


def test_two_layer_stack_with_fused_loss_and_adam(cuda_device):
    """The shape family of the benchmark configurations 1 and 2, scaled down: an FFI layer with ReLU
    feeding the FFI output layer, loss fused into the output layer's forward, one Adam step on the
    output weights; every gradient against the fp64 oracle chained by hand."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N0, N1, L, K = 128, 768, 512, 6_001, 32  # hidden width that keeps the output layer on the fused-loss path
    x0 = synth.normal(21, 0, (B, N0)).numpy()
    idx1 = synth.indices_without_replacement(21, 1, N1, K, N0).numpy()
    W1 = synth.normal(21, 2, (N1, K), std=(2.0 / K) ** 0.5).numpy()
    idx2 = synth.indices_without_replacement(21, 3, L, K, N1).numpy()
    W2 = synth.normal(21, 4, (L, K), std=(2.0 / K) ** 0.5).numpy()
    bias2 = np.zeros(L, np.float32)
    row_ptr, labels = synth.multi_hot_targets(21, 5, B, L)

    # device: hidden = relu(FFI1(x0)); (loss, gT) = FFI2 with the fused BCE; backward through both
    xd = to_cuda(x0, dev)
    h_pre = ops._forward(xd, to_cuda(idx1, dev), to_cuda(W1, dev), None, False)
    h = torch.relu(h_pre)
    loss, gT = ops.forward_bce(h, to_cuda(idx2, dev), to_cuda(W2, dev), to_cuda(bias2, dev), row_ptr, labels, False)
    gh, gW2, gb2 = ops._backward(h, to_cuda(idx2, dev), to_cuda(W2, dev), gT, False, want_bias_grad=True,
                                 grad_is_transposed=True)
    gh_pre = gh * (h_pre > 0)
    gx0, gW1, _ = ops._backward(xd, to_cuda(idx1, dev), to_cuda(W1, dev), gh_pre.contiguous(), False)

    # oracle chain in fp64 (the hidden activations the device produced are the second layer's input)
    h_ref = np.maximum(oracle.forward_f64(x0, idx1, W1), 0.0)
    assert_close(h.cpu().numpy(), h_ref, RTOL, ATOL, "hidden activations")
    h32 = h.cpu().numpy()
    z = oracle.forward_f64(h32, idx2, W2, bias=bias2).astype(np.float32)
    loss_ref, g_ref = oracle.bce_f64(z, row_ptr.numpy(), labels.numpy())
    assert abs(float(loss) - loss_ref) <= 2e-5 * abs(loss_ref) + 1e-7
    g32 = g_ref.astype(np.float32)
    scale = np.abs(g32).max()

    def close(name, got, want, rtol=2e-4):
        err = np.abs(got.cpu().numpy().astype(np.float64) - want).max()
        assert err <= rtol * np.abs(want).max() + 1e-12, f"{name}: {err:.3e} vs scale {np.abs(want).max():.3e}"

    close("grad_W2", gW2, oracle.grad_w_f64(h32, idx2, g32))
    close("grad_bias2", gb2, oracle.grad_bias_f64(g32))
    gh_ref = oracle.grad_x_f64(idx2, W2, g32, N1)
    close("grad_hidden", gh, gh_ref)
    ghp = (gh.cpu().numpy() * (h_pre.cpu().numpy() > 0)).astype(np.float32)
    close("grad_W1", gW1, oracle.grad_w_f64(x0, idx1, ghp))
    close("grad_x0", gx0, oracle.grad_x_f64(idx1, W1, ghp, N0))
    assert scale > 0

    # one Adam step on the output layer's weights (lr 1e-3, beta 0.9/0.999, eps 1e-7, as Keras)
    w = to_cuda(W2, dev).reshape(-1).clone()
    opt = ffi.FusedAdam([w], lr=1e-3)
    opt.step([gW2.reshape(-1)])
    w_ref, _, _ = oracle.adam_f64(W2.reshape(-1), np.zeros(L * K), np.zeros(L * K), gW2.cpu().numpy().reshape(-1),
                                  np.float32(1e-3), np.float32(0.9), np.float32(0.999), np.float32(1e-7), 1)
    assert_close(w.cpu().numpy(), w_ref, 1e-5, 1e-6, "Adam step")


def test_peer_sum_single_rank_and_argument_checks(cuda_device):
    """ffi_peer_sum with a world of one rank (the multi-GPU exchange needs several GPUs; here the
    kernel's flag protocol and the sum run against the rank's own buffers) and its argument checks."""
    import ctypes

    dev = cuda_device
    lib = _lib.load()
    n = 768 * 128 + 4
    buf = torch.zeros((2, n), device=dev)
    flags = torch.zeros((2, 1), dtype=torch.int32, device=dev)
    out = torch.empty(n, device=dev)
    bufs = (ctypes.c_void_p * 1)(buf.data_ptr())
    flgs = (ctypes.c_void_p * 1)(flags.data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream
    for step in range(1, 6):
        part = torch.randn(n, device=dev)
        buf[step & 1].copy_(part)
        _lib.check(lib.ffi_peer_sum(bufs, flgs, 0, 1, n, step, out.data_ptr(), stream))
        assert torch.equal(out, part)
        assert int(flags[step & 1, 0]) == step
    assert lib.ffi_peer_sum(bufs, flgs, 0, 1, n, 0, out.data_ptr(), stream) == 1      # steps count from 1
    assert lib.ffi_peer_sum(bufs, flgs, 1, 1, n, 1, out.data_ptr(), stream) == 1      # rank outside the world
    assert lib.ffi_peer_sum(bufs, flgs, 0, 1, n - 1, 1, out.data_ptr(), stream) == 1  # not a multiple of 4
    assert lib.ffi_peer_sum(None, flgs, 0, 1, n, 1, out.data_ptr(), stream) == 1
    count = ctypes.c_int(-1)
    _lib.check(lib.ffi_wait_timeouts(ctypes.byref(count)))
    import cases
    assert count.value == cases.EXPECTED_WAIT_TIMEOUTS


def test_bounded_peer_wait_gives_up_and_is_counted(cuda_device):
    """A wait on another GPU that nothing will ever satisfy: a world of two ranks of which only rank 0
    exists.  With the limit lowered to about a millisecond the kernel must return by itself, leave the
    context usable and be counted by ffi_wait_timeouts (the host-visible error status of the wait)."""
    import ctypes
    import time

    import cases

    dev = cuda_device
    lib = _lib.load()
    n = 1024
    bufs = [torch.zeros((2, n), device=dev) for _ in range(2)]
    flags = [torch.zeros((2, 2), dtype=torch.int32, device=dev) for _ in range(2)]
    out = torch.empty(n, device=dev)
    pb = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    pf = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    before = ctypes.c_int(-1)
    _lib.check(lib.ffi_wait_timeouts(ctypes.byref(before)))
    _lib.check(lib.ffi_set_wait_limit_ticks(2_000_000))  # about a millisecond
    try:
        t0 = time.perf_counter()
        _lib.check(lib.ffi_peer_sum(pb, pf, 0, 2, n, 1, out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
    finally:
        _lib.check(lib.ffi_set_wait_limit_ticks(4_000_000_000))
    after = ctypes.c_int(-1)
    _lib.check(lib.ffi_wait_timeouts(ctypes.byref(after)))
    assert after.value > before.value
    cases.EXPECTED_WAIT_TIMEOUTS += after.value - before.value
    # the context is still usable and rank 0's own flag went up
    assert int(flags[0][1, 0]) == 1 and int(flags[1][1, 0]) == 1
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
    assert lib.ffi_set_wait_limit_ticks(5) == 1


def _torch_reference(xT, idx, W, g, chunk=4096):
    """Plain PyTorch fp64 statement of the layer, chunked over the outputs: (y, grad_x[N,B], grad_W)."""
    N, B = xT.shape
    L, K = idx.shape
    x64 = xT.double()
    y = torch.empty((B, L), dtype=torch.float64, device=xT.device)
    gW = torch.empty((L, K), dtype=torch.float64, device=xT.device)
    gx = torch.zeros((N, B), dtype=torch.float64, device=xT.device)
    for o0 in range(0, L, chunk):
        o1 = min(L, o0 + chunk)
        ii = idx[o0:o1].long()
        gathered = x64[ii]                                    # [l, K, B]
        w = W[o0:o1].double()
        y[:, o0:o1] = torch.einsum("lk,lkb->bl", w, gathered)
        gc = g[:, o0:o1].double()                             # [B, l]
        gW[o0:o1] = torch.einsum("bl,lkb->lk", gc, gathered)
        contrib = w[:, :, None] * gc.t()[:, None, :]          # [l, K, B]
        gx.index_add_(0, ii.reshape(-1), contrib.reshape(-1, B))
    return y, gx, gW


def test_headline_shape_full_size(cuda_device):
    """B=128, N=768, L=670,091, K=32 (the benchmark shape) against a PyTorch fp64 reference on the
    device, a CPU-oracle check on a slice of the outputs, and linearity in x."""
    dev = cuda_device
    B, N, L, K = 128, 768, 670_091, 32
    xT = synth.normal(21, 0, (N, B), device=dev)
    idx = synth.indices_without_replacement(21, 1, L, K, N, device=dev)
    W = synth.normal(21, 2, (L, K), std=(1.0 / K) ** 0.5, device=dev)
    g = synth.normal(21, 3, (B, L), device=dev)
    y = ffi.fan_in_sparse_matmul_tp(xT, idx, W)
    gx, gW = ffi.fan_in_sparse_matmul_grad_tp(xT, idx, W, g)
    y_ref, gx_ref, gW_ref = _torch_reference(xT, idx, W, g)

    def close(a, b, what, atol=ATOL):
        err = (a.double() - b).abs()
        bound = atol + RTOL * b.abs()
        assert bool((err <= bound).all()), f"{what}: max excess {(err - bound).max().item():.3e}"

    close(y, y_ref, "y")
    close(gW, gW_ref, "grad_W")
    close(gx, gx_ref, "grad_x", atol=gx_atol(L, K, N))
    # CPU oracle on a slice of outputs (rows of idx/W are independent for y and grad_W)
    rows = np.r_[0:64, L // 2:L // 2 + 64, L - 64:L]
    x_np = xT.t().contiguous().cpu().numpy()
    idx_s, W_s = idx[rows].cpu().numpy(), W[rows].cpu().numpy()
    assert_close(y[:, rows].cpu().numpy(), oracle.forward_f64(x_np, idx_s, W_s), RTOL, ATOL, "y slice vs oracle")
    assert_close(gW[rows].cpu().numpy(), oracle.grad_w_f64(x_np, idx_s, g[:, rows].contiguous().cpu().numpy()),
                 RTOL, ATOL, "grad_W slice vs oracle")
    # linearity: FFI(2x) = 2 FFI(x) exactly in binary floating point
    assert torch.equal(ffi.fan_in_sparse_matmul_tp(xT * 2, idx, W), y * 2)
    # determinism at full size
    gx2, gW2 = ffi.fan_in_sparse_matmul_grad_tp(xT, idx, W, g)
    assert torch.equal(gx, gx2) and torch.equal(gW, gW2)


def test_transpose_gradient_and_backward_from_transposed(cuda_device):
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    # the last three take the tiled grad_W kernel (wide inputs, K not a multiple of 4), which reads either layout
    for shape in [(128, 768, 5_001, 32), (37, 254, 513, 16), (200, 100, 300, 8), (130, 3_000, 1_000, 16),
                  (70, 300, 500, 7), (128, 32_768, 2_001, 32)]:
        B, N, L, K = shape
        x, idx, W, g = reference_style_inputs(shape, seed=3, relu_grad=False)
        gT, gb = ops.transpose_gradient(to_cuda(g, dev), want_bias_grad=True)
        assert gT.shape[0] == L and gT.shape[1] >= B and gT.shape[1] % 32 == 0
        assert torch.equal(gT[:, :B], to_cuda(g, dev).t())
        assert not gT[:, B:].any()
        assert_close(gb.cpu().numpy(), oracle.grad_bias_f64(g), RTOL, ATOL, "grad_bias from transposition")
        args = (to_cuda(x, dev), to_cuda(idx, dev), to_cuda(W, dev))
        gx1, gw1, gb1 = ops._backward(*args, to_cuda(g, dev), False, want_bias_grad=True)
        gx2, gw2, gb2 = ops._backward(*args, gT, False, want_bias_grad=True, grad_is_transposed=True)
        assert torch.equal(gx1, gx2) and torch.equal(gw1, gw2)
        assert_close(gb2.cpu().numpy(), oracle.grad_bias_f64(g), RTOL, ATOL, "grad_bias from gT rows")


@pytest.mark.parametrize("shape,transposed", [((128, 768, 20_011, 32), True), ((37, 254, 513, 16), False),
                                              ((64, 100, 1000, 8), True)], ids=["headline-like", "small", "b64"])
def test_fused_forward_bce_matches_unfused(cuda_device, shape, transposed):
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N, L, K = shape
    x, idx, W, _ = config_style_inputs(B, N, L, K, seed=9)
    bias = synth.normal(9, 40, (L,), std=0.5).numpy()
    row_ptr, labels = synth.multi_hot_targets(9, 41, B, L)
    xin = np.ascontiguousarray(x.T) if transposed else x
    loss, gT = ops.forward_bce(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(bias, dev), row_ptr,
                               labels, transposed)
    z = oracle.forward_f64(x, idx, W, bias=bias).astype(np.float32)
    loss_ref, g_ref = oracle.bce_f64(z, row_ptr.numpy(), labels.numpy())
    assert abs(float(loss) - loss_ref) <= 2e-5 * abs(loss_ref) + 1e-7
    assert_close(gT[:, :B].t().cpu().numpy(), g_ref, 5e-5, 1e-12, "fused BCE gradient")
    assert not gT[:, B:].any()
    # label shard [lo, hi) of the same problem
    lo, hi = L // 4, L // 4 + (L // 2) // 4 * 4
    loss_s, gT_s = ops.forward_bce(to_cuda(xin, dev), to_cuda(idx[lo:hi], dev), to_cuda(W[lo:hi], dev),
                                   to_cuda(bias[lo:hi], dev), row_ptr, labels, transposed, total_labels=L,
                                   label_offset=lo)
    assert_close(gT_s[:, :B].t().cpu().numpy(), g_ref[:, lo:hi], 5e-5, 1e-12, "fused BCE gradient (shard)")


@pytest.mark.parametrize("loss_name", ["squared_hinge", "hinge"])
@pytest.mark.parametrize("shape,transposed", [((128, 768, 20_011, 32), True), ((37, 254, 513, 16), False)],
                         ids=["headline-like", "small"])
def test_fused_forward_hinge_losses(cuda_device, shape, transposed, loss_name):
    """The reference's default loss (squared hinge) and the plain hinge, fused into the forward pass."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N, L, K = shape
    x, idx, W, _ = config_style_inputs(B, N, L, K, seed=11)
    W = W * 8  # spread the logits over both sides of the hinge
    bias = synth.normal(11, 40, (L,), std=0.5).numpy()
    row_ptr, labels = synth.multi_hot_targets(11, 41, B, L)
    xin = np.ascontiguousarray(x.T) if transposed else x
    loss, gT = ops.forward_bce(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(bias, dev), row_ptr,
                               labels, transposed, loss=loss_name)
    z64 = oracle.forward_f64(x, idx, W, bias=bias)
    z = z64.astype(np.float32)
    squared = loss_name == "squared_hinge"
    loss_ref, g_ref = oracle.hinge_f64(z, row_ptr.numpy(), labels.numpy(), squared=squared)
    assert abs(float(loss) - loss_ref) <= 2e-5 * abs(loss_ref) + 1e-7
    got = gT[:, :B].t().cpu().numpy()
    scale = 1.0 / (B * L)
    assert (g_ref != 0).mean() > 0.05 and (g_ref == 0).mean() > 0.05, "test inputs must exercise both branches"
    if squared:
        # continuous in z: an fp32 logit within 1e-5 of the fp64 one moves the gradient by 2e-5 * scale
        assert np.abs(got - g_ref).max() <= 4e-5 * scale * max(1.0, np.abs(z).max())
    else:
        # a step function of z: compare away from the kink at |z| = 1
        away = np.abs(np.abs(z64) - 1.0) > 1e-4
        assert away.mean() > 0.99
        assert np.array_equal(got[away], g_ref[away].astype(np.float32))
    assert not gT[:, B:].any()
    lo, hi = L // 4, L // 4 + (L // 2) // 4 * 4
    loss_s, gT_s = ops.forward_bce(to_cuda(xin, dev), to_cuda(idx[lo:hi], dev), to_cuda(W[lo:hi], dev),
                                   to_cuda(bias[lo:hi], dev), row_ptr, labels, transposed, total_labels=L,
                                   label_offset=lo, loss=loss_name)
    assert torch.equal(gT_s[:, :B], gT[lo:hi, :B])


@pytest.mark.parametrize("shape,transposed", [((128, 768, 20_011, 32), True), ((37, 254, 513, 16), False),
                                              ((64, 100, 7, 8), True), ((128, 32_768, 5_003, 32), False),
                                              ((33, 40_000, 2_000, 72), True), ((70, 300, 1_500, 7), False),
                                              ((200, 500, 900, 5), True)],
                         ids=["headline-like", "small", "few-rows", "wide-N", "wide-N-K72", "odd-K", "odd-K-two-batch-tiles"])
def test_fused_forward_topk_and_precision_at_k(cuda_device, shape, transposed):
    """Top-k of the logits from the forward kernel's epilogue (the logits are never written) against a
    stable sort of the oracle's logits; P@k as the reference's PrecisionAtK accumulates it."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N, L, K = shape
    x, idx, W, _ = config_style_inputs(B, N, L, K, seed=13)
    bias = synth.normal(13, 40, (L,), std=0.5).numpy()
    row_ptr, labels = synth.multi_hot_targets(13, 41, B, L)
    xin = np.ascontiguousarray(x.T) if transposed else x
    k = 5
    vals, lab = ops.forward_topk(to_cuda(xin, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(bias, dev), k, transposed)
    z64 = oracle.forward_f64(x, idx, W, bias=bias)
    order = np.argsort(-z64, axis=1, kind="stable")[:, :k]
    want_vals = np.take_along_axis(z64, order, axis=1)
    got_vals, got_lab = vals.cpu().numpy(), lab.cpu().numpy()
    assert_close(got_vals, want_vals, RTOL, ATOL, "top-k values")
    # labels must agree wherever the ranking is not decided by less than the fp32 tolerance
    full = np.sort(z64, axis=1)[:, ::-1][:, :k + 1]
    decided = np.abs(np.diff(full, axis=1)) > 1e-4
    decided = decided[:, :k] & np.concatenate([np.ones((B, 1), bool), decided[:, :k - 1]], axis=1)
    assert decided.mean() > 0.9
    assert np.array_equal(got_lab[decided], order[decided])
    # every returned label carries its own logit
    assert_close(got_vals, np.take_along_axis(z64, got_lab.astype(np.int64), axis=1), RTOL, ATOL, "value of label")
    # two shards merged give the same candidates
    half = (L // 2) // 4 * 4
    if half > 0:
        c0 = ops.forward_topk(to_cuda(xin, dev), to_cuda(idx[:half], dev), to_cuda(W[:half], dev),
                              to_cuda(bias[:half], dev), min(k, half), transposed, label_offset=0)
        c1 = ops.forward_topk(to_cuda(xin, dev), to_cuda(idx[half:], dev), to_cuda(W[half:], dev),
                              to_cuda(bias[half:], dev), min(k, L - half), transposed, label_offset=half)
        mv, ml = ops.merge_topk([c0, c1], k)
        assert torch.equal(ml, lab) and torch.equal(mv, vals)
    # P@k against a direct count on the oracle's ranking
    for kk in (1, 3, 5):
        hits = sum(len(set(order[b, :kk].tolist()) & set(labels[row_ptr[b]:row_ptr[b + 1]].tolist())) for b in range(B))
        want = hits / (B * kk)
        got = ops.precision_at_k(lab, row_ptr, labels, kk)
        assert abs(got - want) <= (1.0 - decided.mean()) + 1e-12


@pytest.mark.parametrize("shape", [(17, 64, 63, 45), (70, 300, 500, 7), (130, 3_000, 1_000, 16), (128, 32_768, 3_001, 32)],
                         ids=["K45", "K7_B70", "wide_N3000_B130", "wide_N32768"])
@pytest.mark.parametrize("loss_name", ["bce", "squared_hinge"])
def test_fused_forward_loss_on_tiled_kernel_shapes(cuda_device, shape, loss_name):
    """Shapes the barrier-free forward does not take (K not a multiple of 4, x too wide for shared memory):
    the tiled forward kernel carries the same loss epilogue."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N, L, K = shape
    x, idx, W, _ = config_style_inputs(B, N, L, K, seed=19)
    W = W * 4
    bias = synth.normal(19, 40, (L,), std=0.5).numpy()
    row_ptr, labels = synth.multi_hot_targets(19, 41, B, L)
    loss, gT = ops.forward_bce(to_cuda(x, dev), to_cuda(idx, dev), to_cuda(W, dev), to_cuda(bias, dev), row_ptr, labels,
                               False, loss=loss_name)
    z = oracle.forward_f64(x, idx, W, bias=bias).astype(np.float32)
    if loss_name == "bce":
        loss_ref, g_ref = oracle.bce_f64(z, row_ptr.numpy(), labels.numpy())
        # positives with a large logit: sigmoid(z) - 1 cancels, so the floor is relative to the scale 1/(B*L)
        assert_close(gT[:, :B].t().cpu().numpy(), g_ref, 5e-5, 2e-7 / (B * L), "fused BCE gradient (tiled kernel)")
    else:
        loss_ref, g_ref = oracle.hinge_f64(z, row_ptr.numpy(), labels.numpy(), squared=True)
        assert np.abs(gT[:, :B].t().cpu().numpy() - g_ref).max() <= 4e-5 / (B * L) * max(1.0, np.abs(z).max())
    assert abs(float(loss) - loss_ref) <= 2e-5 * abs(loss_ref) + 1e-7
    assert gT.shape[1] >= B and not gT[:, B:].any()


@pytest.mark.parametrize("shape,transposed", [((64, 512, 3_001, 32), True), ((37, 254, 513, 16), False),
                                              ((130, 100, 600, 73), False), ((128, 768, 20_011, 32), True),
                                              ((100, 300, 2_001, 64), False), ((128, 32_768, 1_001, 32), True),
                                              ((256, 40_000, 1_501, 32), True), ((300, 33_000, 777, 64), False),
                                              ((512, 34_000, 515, 72), False)],
                         ids=["wiki-like", "small", "odd", "headline-like", "K64-staged-x", "wide", "wide-B256",
                              "wide-B300", "wide-B512-K72"])
def test_bf16_storage_of_x_and_w(cuda_device, shape, transposed):
    """x and W stored as bf16, fp32 accumulation (benchmark configurations 2-4; the reference is fp32
    only, tfsparse/cc/kernels/register.cpp:79-109).  Inputs are rounded to bf16 once; the CUDA result
    must match the fp64 oracle evaluated on the rounded values to fp32 accuracy, and stay within
    rel 2e-2 (of the output scale) of the result for the unrounded fp32 inputs."""
    dev = cuda_device
    from ecml23_sparse_b200 import ops
    B, N, L, K = shape
    x, idx, W, g = config_style_inputs(B, N, L, K, seed=17)
    xb = torch.from_numpy(x).to(torch.bfloat16)
    Wb = torch.from_numpy(W).to(torch.bfloat16)
    xr, Wr = xb.float().numpy(), Wb.float().numpy()          # the rounded values, exactly
    xin = (xb.t().contiguous() if transposed else xb).to(dev)
    y = ops._forward(xin, to_cuda(idx, dev), Wb.to(dev), None, transposed).cpu().numpy()
    gx, gw, _ = ops._backward(xin, to_cuda(idx, dev), Wb.to(dev), to_cuda(g, dev), transposed)
    assert gx.dtype == torch.float32 and gw.dtype == torch.float32
    gx = gx.cpu().numpy().T if transposed else gx.cpu().numpy()
    gw = gw.cpu().numpy()
    assert_close(y, oracle.forward_f64(xr, idx, Wr), RTOL, ATOL, "bf16 y vs oracle on rounded inputs")
    assert_close(gw, oracle.grad_w_f64(xr, idx, g), RTOL, ATOL, "bf16 grad_W vs oracle on rounded inputs")
    assert_close(gx, oracle.grad_x_f64(idx, Wr, g, N), RTOL, gx_atol(L, K, N), "bf16 grad_x vs oracle on rounded inputs")
    for got, ref, what in ((y, oracle.forward_f64(x, idx, W), "y"), (gw, oracle.grad_w_f64(x, idx, g), "grad_W"),
                           (gx, oracle.grad_x_f64(idx, W, g, N), "grad_x")):
        scale = np.abs(ref).max()
        assert np.abs(got - ref).max() <= 2e-2 * scale, f"bf16 {what} further than 2e-2 from the fp32-input result"
    with pytest.raises(TypeError):
        ops._forward(xin, to_cuda(idx, dev), to_cuda(W, dev), None, transposed)  # mixed storage types
    # the fused loss on bf16 storage: same logits, so the same gradient as the oracle's on the rounded inputs
    bias = synth.normal(17, 40, (L,), std=0.5).numpy()
    row_ptr, labels = synth.multi_hot_targets(17, 41, B, L)
    loss, gT = ops.forward_bce(xin, to_cuda(idx, dev), Wb.to(dev), to_cuda(bias, dev), row_ptr, labels, transposed)
    z = oracle.forward_f64(xr, idx, Wr, bias=bias).astype(np.float32)
    loss_ref, g_ref = oracle.bce_f64(z, row_ptr.numpy(), labels.numpy())
    assert abs(float(loss) - loss_ref) <= 2e-5 * abs(loss_ref) + 1e-7
    assert_close(gT[:, :B].t().cpu().numpy(), g_ref, 5e-5, 2e-7 / (B * L), "fused BCE gradient on bf16 storage")
    assert not gT[:, B:].any()
    # top-k on bf16 storage: values of the oracle's logits on the rounded inputs, every label carries its logit
    k = 5
    vals, lab = ops.forward_topk(xin, to_cuda(idx, dev), Wb.to(dev), to_cuda(bias, dev), k, transposed)
    z64 = oracle.forward_f64(xr, idx, Wr, bias=bias)
    want = -np.sort(-z64, axis=1)[:, :k]
    assert_close(vals.cpu().numpy(), want, RTOL, ATOL, "bf16 top-k values")
    assert_close(vals.cpu().numpy(), np.take_along_axis(z64, lab.cpu().numpy().astype(np.int64), axis=1), RTOL, ATOL,
                 "bf16 top-k: value of label")
