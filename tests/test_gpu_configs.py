"""GPU parity on the shapes the benchmark configurations name: the batch sizes, fan-ins and input
widths of configurations 0-4, at full size where a reference finishes in seconds and at a reduced
number of outputs L otherwise (rows of idx/W are independent for y and grad_W, and grad_x is a sum
over rows, so a smaller L exercises the same kernels, tilings and index arithmetic).

Checker: a plain PyTorch fp64 statement of the layer evaluated on the device in chunks of outputs
(`torch_reference_chunks`), cross-checked against the CPU oracle on row slices.  Tolerance as in
test_gpu_parity.py: |d| <= 1e-5 + 1e-5*|ref|, with the grad_x floor widened for long sums (gx_atol).
"""
import numpy as np
import pytest
import torch

import oracle
import ecml23_sparse_b200 as ffi
from ecml23_sparse_b200 import ops, synth
from cases import ATOL, RTOL, assert_close, gx_atol

pytestmark = pytest.mark.gpu


def make_inputs(dev, B, N, L, K, seed, w_var=1.0):
    """Benchmark-style inputs on the device: x ~ N(0,1) as [N,B], K distinct inputs per row, W ~ N(0, w_var/K)."""
    xT = synth.normal(seed, 0, (N, B), device=dev)
    idx = synth.indices_without_replacement(seed, 1, L, K, N, device=dev)
    W = synth.normal(seed, 2, (L, K), std=(w_var / K) ** 0.5, device=dev)
    g = synth.normal(seed, 3, (B, L), device=dev)
    return xT, idx, W, g


def torch_reference_chunks(xT, idx, W, g, bias=None, chunk=2048):
    """Yields (o0, o1, y[B,l] fp64, grad_W[l,K] fp64) per chunk of outputs and accumulates grad_x[N,B] fp64
    into the returned holder's `.gx` (complete once the generator is exhausted)."""
    N, B = xT.shape
    L, K = idx.shape
    x64 = xT.double()

    class Holder:
        gx = torch.zeros((N, B), dtype=torch.float64, device=xT.device)

    def gen():
        for o0 in range(0, L, chunk):
            o1 = min(L, o0 + chunk)
            ii = idx[o0:o1].long()
            gathered = x64[ii]                                    # [l, K, B]
            w = W[o0:o1].double()
            y = torch.einsum("lk,lkb->bl", w, gathered)
            if bias is not None:
                y = y + bias[o0:o1].double()
            gc = g[:, o0:o1].double()                             # [B, l]
            gW = torch.einsum("bl,lkb->lk", gc, gathered)
            contrib = w[:, :, None] * gc.t()[:, None, :]          # [l, K, B]
            Holder.gx.index_add_(0, ii.reshape(-1), contrib.reshape(-1, B))
            yield o0, o1, y, gW

    return Holder, gen()


def bias_atol(B):
    """Absolute floor for grad_bias[o] = sum_b g[b,o]: an fp32 sum of B values of unit scale passes through
    partial sums of size sqrt(B), whose rounding (half an ulp each) the 1e-5 floor does not cover for
    B in the hundreds; the floor grows like sqrt(B)/4 beyond B = 16 (8e-5 at B = 1024)."""
    return ATOL * max(1.0, B ** 0.5 / 4)


def excess(a, ref, atol):
    err = (a.double() - ref).abs()
    return float((err - (atol + RTOL * ref.abs())).max())


def check_layer(dev, xT, idx, W, g, bias=None, chunk=2048, transposed=True, oracle_rows=48):
    """forward (+bias), grad_x, grad_W (+grad_bias) of one layer against the chunked fp64 reference and,
    on a few rows, the CPU oracle."""
    N, B = xT.shape
    L, K = idx.shape
    xin = xT if transposed else xT.t().contiguous()
    y = ops._forward(xin, idx, W, bias, transposed)
    gx, gW, gb = ops._backward(xin, idx, W, g, transposed, want_bias_grad=bias is not None)
    holder, chunks = torch_reference_chunks(xT, idx, W, g, bias=bias, chunk=chunk)
    worst_y = worst_w = -1.0
    for o0, o1, y_ref, gW_ref in chunks:
        worst_y = max(worst_y, excess(y[:, o0:o1], y_ref, ATOL))
        worst_w = max(worst_w, excess(gW[o0:o1], gW_ref, ATOL))
    assert worst_y <= 0, f"y exceeds the tolerance by {worst_y:.3e}"
    assert worst_w <= 0, f"grad_W exceeds the tolerance by {worst_w:.3e}"
    gx_nb = gx if transposed else gx.t()
    ex = excess(gx_nb, holder.gx, gx_atol(L, K, N))
    assert ex <= 0, f"grad_x exceeds the tolerance by {ex:.3e}"
    if bias is not None:
        exb = excess(gb, g.double().sum(0), bias_atol(B))
        assert exb <= 0, f"grad_bias exceeds the tolerance by {exb:.3e}"
    # the CPU oracle on a slice of the rows (y and grad_W rows are independent)
    rows = np.unique(np.r_[0:oracle_rows, L // 2:L // 2 + oracle_rows, L - oracle_rows:L].clip(0, L - 1))
    x_np = xT.t().contiguous().cpu().numpy()
    idx_s, W_s = idx[rows].cpu().numpy(), W[rows].cpu().numpy()
    b_s = bias[rows].cpu().numpy() if bias is not None else None
    assert_close(y[:, rows].cpu().numpy(), oracle.forward_f64(x_np, idx_s, W_s, bias=b_s), RTOL, ATOL, "y rows vs oracle")
    assert_close(gW[rows].cpu().numpy(), oracle.grad_w_f64(x_np, idx_s, g[:, rows].contiguous().cpu().numpy()),
                 RTOL, ATOL, "grad_W rows vs oracle")
    return y, gx, gW, gb


def test_config0_full_size_with_grad_bias(cuda_device):
    """Configuration 0 at full size: B=32, N=768, L=670,091, K=32, fp32, y / grad_W / grad_x / grad_bias."""
    dev = cuda_device
    B, N, L, K = 32, 768, 670_091, 32
    xT, idx, W, g = make_inputs(dev, B, N, L, K, seed=100)
    bias = synth.normal(100, 9, (L,), std=0.1, device=dev)
    check_layer(dev, xT, idx, W, g, bias=bias, chunk=8192)
    # grad_x of the whole layer against the CPU oracle (fp64), the configuration's own comparison
    gx, _, _ = ops._backward(xT, idx, W, g, True, want_weight_grad=False)
    ref = oracle.grad_x_f64(idx.cpu().numpy(), W.cpu().numpy(), g.cpu().numpy(), N)
    assert_close(gx.t().cpu().numpy(), ref, RTOL, gx_atol(L, K, N), "grad_x vs CPU oracle, full size")


@pytest.mark.parametrize("B", [512, 1024])
@pytest.mark.parametrize("transposed", [True, False], ids=["tp", "plain"])
def test_large_batches_of_configs_3_and_4(cuda_device, B, transposed):
    """Batch 512 (configuration 3) and 1024 (configuration 4): several batch tiles per kernel."""
    dev = cuda_device
    N, L, K = 768, 12_011, 32
    xT, idx, W, g = make_inputs(dev, B, N, L, K, seed=200 + B)
    bias = synth.normal(200, 9, (L,), std=0.1, device=dev)
    check_layer(dev, xT, idx, W, g, bias=bias, chunk=1024, transposed=transposed)


@pytest.mark.parametrize("shape", [(512, 100_000, 3_001, 72), (1024, 65_536, 2_003, 64), (128, 32_768, 6_007, 32),
                                   (256, 65_536, 4_001, 32)],
                         ids=["config3_N100000_K72", "config4_N65536_K64", "config1_N32768_K32", "config2_N65536_K32"])
def test_wide_output_layers_of_configs_1_to_4(cuda_device, shape):
    """The output layers of the stacked configurations: inputs N = 32,768 ... 100,000 (the hidden width),
    fan-in 32 / 64 / 72, batch 128 ... 1024; forward, both gradients, grad_bias and the unfused
    sigmoid-BCE gradient on the logits."""
    dev = cuda_device
    B, N, L, K = shape
    xT, idx, W, g = make_inputs(dev, B, N, L, K, seed=300 + K, w_var=2.0)
    xT = torch.relu(xT)  # hidden activations after the ReLU: half of them exactly zero
    bias = synth.normal(300, 9, (L,), std=0.1, device=dev)
    y, _, _, _ = check_layer(dev, xT, idx, W, g, bias=bias, chunk=256)
    row_ptr, labels = synth.multi_hot_targets(300, 5, B, L)
    loss, gz = ffi.sparse_bce_with_logits(y, row_ptr, labels)
    loss_ref, g_ref = oracle.bce_f64(y.cpu().numpy(), row_ptr.numpy(), labels.numpy())
    assert abs(float(loss) - loss_ref) <= 1e-5 * abs(loss_ref) + 1e-7
    assert_close(gz.cpu().numpy(), g_ref, 2e-5, 1e-12, "BCE gradient on the wide layer's logits")


def test_offsets_beyond_two_to_the_31(cuda_device):
    """B*L >= 2^31 elements in y and g (the reference indexes batch*L+unit in int32,
    tfsparse/cc/kernels/kernel_data.cu.h:221-225): B=1024, N=512, L=2,100,000, K=4."""
    dev = cuda_device
    B, N, L, K = 1024, 512, 2_100_000, 4
    assert B * L >= 2 ** 31
    xT, idx, W, _ = make_inputs(dev, B, N, 1, K, seed=400)
    idx = synth.indices_without_replacement(400, 1, L, K, N, device=dev)
    W = synth.normal(400, 2, (L, K), std=0.5, device=dev)
    # upstream gradient generated in slabs (one call would need a 2^31-element temporary)
    g = torch.empty((B, L), dtype=torch.float32, device=dev)
    for b0 in range(0, B, 128):
        g[b0:b0 + 128] = synth.normal(400, 10 + b0, (128, L), device=dev)
    y = ops._forward(xT, idx, W, None, True)
    gx, gW, gb = ops._backward(xT, idx, W, g, True, want_bias_grad=True)
    holder, chunks = torch_reference_chunks(xT, idx, W, g, chunk=65_536)
    worst_y = worst_w = worst_b = -1.0
    for o0, o1, y_ref, gW_ref in chunks:
        worst_y = max(worst_y, excess(y[:, o0:o1], y_ref, ATOL))
        worst_w = max(worst_w, excess(gW[o0:o1], gW_ref, ATOL * 4))  # sums of 1024 products
        worst_b = max(worst_b, excess(gb[o0:o1], g[:, o0:o1].double().sum(0), bias_atol(B)))
    assert worst_y <= 0 and worst_w <= 0 and worst_b <= 0, (worst_y, worst_w, worst_b)
    ex = excess(gx, holder.gx, gx_atol(L, K, N, term_rms=0.5))  # W ~ N(0, 1/K) with K = 4: summands of scale 0.5
    assert ex <= 0, f"grad_x exceeds the tolerance by {ex:.3e}"
    # the last rows and the last batch element live beyond the 2^31-th element
    rows = np.r_[L - 32:L]
    x_np = xT.t().contiguous().cpu().numpy()
    assert_close(y[:, rows].cpu().numpy(), oracle.forward_f64(x_np, idx[rows].cpu().numpy(), W[rows].cpu().numpy()),
                 RTOL, ATOL, "y tail vs oracle")


def test_two_layer_stack_at_real_hidden_width(cuda_device):
    """Configuration 1's stack at its real hidden width: 768 -> 32,768 (K=32, ReLU) -> L (K=32), B=128,
    sigmoid-BCE on the logits, backward through both layers; L reduced to 20,011 rows."""
    dev = cuda_device
    B, N0, N1, L, K = 128, 768, 32_768, 20_011, 32
    x0T = synth.normal(500, 0, (N0, B), device=dev)
    idx1 = synth.indices_without_replacement(500, 1, N1, K, N0, device=dev)
    W1 = synth.normal(500, 2, (N1, K), std=(2.0 / K) ** 0.5, device=dev)
    idx2 = synth.indices_without_replacement(500, 3, L, K, N1, device=dev)
    W2 = synth.normal(500, 4, (L, K), std=(2.0 / K) ** 0.5, device=dev)
    bias2 = torch.zeros(L, device=dev)
    row_ptr, labels = synth.multi_hot_targets(500, 5, B, L)

    h_pre = ops._forward(x0T, idx1, W1, None, True)                    # [B, N1]
    h = torch.relu(h_pre)
    z = ops._forward(h, idx2, W2, bias2, False)                        # [B, L]
    loss, gz = ffi.sparse_bce_with_logits(z, row_ptr, labels)
    gh, gW2, gb2 = ops._backward(h, idx2, W2, gz, False, want_bias_grad=True)
    gh_pre = (gh * (h_pre > 0)).contiguous()
    gx0, gW1, _ = ops._backward(x0T, idx1, W1, gh_pre, True)

    # layer 1 forward against the fp64 reference
    hold1, ch1 = torch_reference_chunks(x0T, idx1, W1, gh_pre, chunk=4096)
    for o0, o1, y_ref, gW_ref in ch1:
        assert excess(h_pre[:, o0:o1], y_ref, ATOL) <= 0
        assert excess(gW1[o0:o1], gW_ref, 1e-9) <= 0 or \
            float((gW1[o0:o1].double() - gW_ref).abs().max()) <= 2e-5 * float(gW_ref.abs().max())
    assert float((gx0.double() - hold1.gx).abs().max()) <= 2e-5 * float(hold1.gx.abs().max())
    # layer 2 (the wide output layer) on the activations the device produced
    hT = h.t().contiguous()
    hold2, ch2 = torch_reference_chunks(hT, idx2, W2, gz, bias=bias2, chunk=1024)
    for o0, o1, y_ref, gW_ref in ch2:
        assert excess(z[:, o0:o1], y_ref, ATOL) <= 0
        assert float((gW2[o0:o1].double() - gW_ref).abs().max()) <= 2e-5 * float(gW_ref.abs().max()) + 1e-12
    assert float((gh.t().double() - hold2.gx).abs().max()) <= 2e-5 * float(hold2.gx.abs().max())
    loss_ref, g_ref = oracle.bce_f64(z.cpu().numpy(), row_ptr.numpy(), labels.numpy())
    assert abs(float(loss) - loss_ref) <= 1e-5 * abs(loss_ref) + 1e-7
    assert_close(gz.cpu().numpy(), g_ref, 2e-5, 1e-12, "BCE gradient")
    assert float((gb2.double() - gz.double().sum(0)).abs().max()) <= 1e-5 * float(gz.abs().max()) * 8
