"""GPU test of ffi_grad_x_static, the grad_x entry point for callers that may not allocate.

Framework op kernels and steady-state serving loops cannot call cudaMalloc where they call this
library; ffi_grad_x_static therefore keeps its scratch in a fixed array inside the library.  The
test drives it through the C ABI exactly as such a caller would (raw pointers, no workspace) and
compares with grad_x of the regular entry point ffi_backward, twice in a row with different data
so that the second call runs on top of the first call's leftovers in the shared array.

Collected last (file name), so a run that stops at the first failure has run everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import ecml23_sparse_b200 as ffi
from ecml23_sparse_b200 import _lib, synth
from ecml23_sparse_b200.ops import _backward, _stream_ptr
from cases import RTOL, assert_close, gx_atol

pytestmark = pytest.mark.gpu


def _transposed_gradient(g: torch.Tensor) -> torch.Tensor:
    """[B,L] -> [L][ldg] with the batch zero padded to a multiple of 32 (what the entry point takes)."""
    B, L = g.shape
    ldg = 32 if B <= 32 else (64 if B <= 64 else -(-B // 128) * 128)
    gT = torch.zeros((L, ldg), dtype=torch.float32, device=g.device)
    gT[:, :B] = g.t()
    return gT


def _static_grad_x(W, gT, plan, B, N, L, K, transposed):
    out = torch.empty((N, B) if transposed else (B, N), dtype=torch.float32, device=W.device)
    lib = _lib.load()
    with torch.cuda.device(W.device):
        _lib.check(lib.ffi_grad_x_static(W.data_ptr(), gT.data_ptr(), gT.shape[1], plan.handle, out.data_ptr(),
                                         B, N, L, K, int(transposed), _stream_ptr(W.device)))
    return out


@pytest.mark.parametrize("shape,transposed", [((128, 768, 20_011, 32), True), ((37, 254, 513, 16), False),
                                              ((16, 5_000, 3_000, 8), False), ((200, 300, 2_000, 12), True)],
                         ids=["headline-like", "small", "wide-inputs", "two-batch-tiles"])
def test_static_scratch_grad_x_matches_regular_entry_point_twice(cuda_device, shape, transposed):
    dev = cuda_device
    B, N, L, K = shape
    idx = synth.indices_without_replacement(31, 0, L, K, N, device=dev)
    plan = ffi.FFIPlan(idx, N)
    x = synth.normal(31, 1, (N, B) if transposed else (B, N), device=dev)
    for call in range(2):
        W = synth.normal(31, 10 + call, (L, K), std=0.2, device=dev)
        g = synth.normal(31, 20 + call, (B, L), device=dev)
        expected, _, _ = _backward(x, idx, W, g, transposed, plan=plan, want_weight_grad=False)
        got = _static_grad_x(W, _transposed_gradient(g), plan, B, N, L, K, transposed)
        torch.cuda.synchronize()
        # same kernel; the regular entry point cuts its fp32 sums into shorter segments when its workspace
        # allows, so the two agree within the grad_x tolerance of the other tests rather than bit for bit
        assert torch.allclose(got, expected, rtol=RTOL, atol=gx_atol(L, K, N))
        # and the numbers themselves against the CPU oracle (fp64), independent of any CUDA kernel
        want = oracle.grad_x_f64(idx.cpu().numpy(), W.cpu().numpy(), g.cpu().numpy(), N)
        got_bn = got.t() if transposed else got
        assert_close(got_bn.cpu().numpy(), want, RTOL, gx_atol(L, K, N), "static-scratch grad_x vs oracle")


def test_static_scratch_rejects_oversize_and_bad_arguments(cuda_device):
    dev = cuda_device
    lib = _lib.load()
    limit = lib.ffi_grad_x_static_max_scratch_bytes()
    assert limit == 20 << 20
    B, N, L, K = 4096, 2048, 512, 8  # one range of partial sums alone is 2048*4096*4 = 32 MiB
    idx = synth.indices_without_replacement(5, 0, L, K, N, device=dev)
    plan = ffi.FFIPlan(idx, N)
    W = torch.zeros((L, K), device=dev)
    gT = torch.zeros((L, 4096), device=dev)
    out = torch.empty((B, N), device=dev)
    rc = lib.ffi_grad_x_static(W.data_ptr(), gT.data_ptr(), 4096, plan.handle, out.data_ptr(), B, N, L, K, 0,
                               _stream_ptr(dev))
    assert rc == 3 and b"scratch" in lib.ffi_last_error()
    assert lib.ffi_grad_x_static(None, gT.data_ptr(), 4096, plan.handle, out.data_ptr(), B, N, L, K, 0, None) == 1
    assert lib.ffi_grad_x_static(W.data_ptr(), gT.data_ptr(), 4000, plan.handle, out.data_ptr(), B, N, L, K, 0,
                                 None) == 1
    assert lib.ffi_grad_x_static(W.data_ptr(), gT.data_ptr(), 4096, plan.handle, out.data_ptr(), B, N, L + 1, K, 0,
                                 None) == 5


def test_no_device_wait_gave_up(cuda_device):
    """Collected last: after every backward call of the session, no bounded device-side wait (the
    bulk copies of the fused backward) may have run out."""
    import ctypes

    # one more fused backward at a batch that takes the bulk-copy path
    B, N, L, K = 128, 256, 4099, 32
    dev = cuda_device
    x = torch.randn(B, N, device=dev)
    idx = torch.stack([torch.randperm(N, device=dev)[:K] for _ in range(L)]).to(torch.int32)
    W = torch.randn(L, K, device=dev) * 0.1
    g = torch.randn(B, L, device=dev)
    gx, gw, _ = _backward(x, idx, W, g, False)
    ref_gw = torch.einsum("bl,blk->lk", g, x[:, idx.long()])
    assert torch.allclose(gw, ref_gw, rtol=1e-4, atol=1e-4)
    count = ctypes.c_int(-1)
    _lib.check(_lib.load().ffi_wait_timeouts(ctypes.byref(count)))
    import cases
    assert count.value == cases.EXPECTED_WAIT_TIMEOUTS  # only the waits a test made run out on purpose
