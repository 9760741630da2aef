"""CPU tests that pin the parity oracle: known-answer vector, golden fixtures produced by the
reference's own CPU kernels, the compiled reference itself when it is present, and the dense
restatement of the reference's test oracle."""
import hashlib

import numpy as np
import pytest

import oracle
from cases import (HUGE_SIZE, KAT_IDX, KAT_W, KAT_X, KAT_Y, REFERENCE_SIZES, SMALL_SIZES, assert_close,
                   golden_path, reference_style_inputs, size_id)


def _digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("transposed", [False, True])
def test_known_answer_forward_exact(transposed):
    # testing/test.cpp:13-47 demands exact equality in both layouts
    x = np.ascontiguousarray(KAT_X.T) if transposed else KAT_X
    assert np.array_equal(oracle.forward_f32(x, KAT_IDX, KAT_W, transposed=transposed), KAT_Y)
    assert np.array_equal(oracle.forward_f64(x, KAT_IDX, KAT_W, transposed=transposed), KAT_Y)
    assert np.array_equal(oracle.dense_forward(x, KAT_IDX, KAT_W, transposed=transposed), KAT_Y)


@pytest.mark.parametrize("size", REFERENCE_SIZES, ids=size_id)
def test_oracle_matches_golden_from_reference(size):
    gold = np.load(golden_path(size))
    x, idx, W, g = reference_style_inputs(size)
    assert str(gold["digest"]) == _digest(x, idx, W, g), "input recipe drifted from the golden fixtures"
    B, N, L, K = size
    y32 = oracle.forward_f32(x, idx, W)
    y64 = oracle.forward_f64(x, idx, W)
    gx32 = oracle.grad_x_f32(idx, W, g, N)
    gx64 = oracle.grad_x_f64(idx, W, g, N)
    gw32 = oracle.grad_w_f32(x, idx, g)
    gw64 = oracle.grad_w_f64(x, idx, g)
    if size == HUGE_SIZE:
        s = int(gold["sample_stride"])
        ys, gws = gold["y_sample"], gold["grad_w_sample"]
        assert_close(y32.ravel()[::s], ys, what="y f32")
        assert_close(y64.ravel()[::s], ys, what="y f64")
        assert_close(gw32.ravel()[::s], gws, what="gW f32")
        assert_close(gw64.ravel()[::s], gws, what="gW f64")
    else:
        assert_close(y32, gold["y"], what="y f32")
        assert_close(y64, gold["y"], what="y f64")
        assert_close(gw32, gold["grad_w"], what="gW f32")
        assert_close(gw64, gold["grad_w"], what="gW f64")
    # grad_x sums L*K/N terms; the reference's own bound is absolute 1.5e-5 on O(1) values and
    # the huge fixture sums 500,000 terms per input in fp32, hence the relative term.
    # (sequential fp32 sums of that length differ by a few 1e-4 between two builds of the same loop).
    loose = 5e-4 if size == HUGE_SIZE else 2e-5
    assert_close(gx32, gold["grad_x"], rtol=loose, atol=1.5e-5, what="gx f32")
    assert_close(gx64, gold["grad_x"], rtol=loose, atol=1.5e-5, what="gx f64")


@pytest.mark.parametrize("size", SMALL_SIZES, ids=size_id)
@pytest.mark.parametrize("transposed", [False, True])
def test_oracle_matches_dense_reference(size, transposed):
    # the reference's own acceptance test: CPU kernels vs dense GEMM oracle
    # (testing/test_case_templates.h:82,139-140), here two-sided
    x, idx, W, g = reference_style_inputs(size)
    B, N, L, K = size
    xin = np.ascontiguousarray(x.T) if transposed else x
    assert_close(oracle.forward_f32(xin, idx, W, transposed=transposed),
                 oracle.dense_forward(xin, idx, W, transposed=transposed), atol=1e-5, rtol=1e-5, what="y")
    dgx, dgw = oracle.dense_backward(xin, idx, W, g, transposed=transposed)
    assert_close(oracle.grad_x_f32(idx, W, g, N, transposed=transposed), dgx, atol=1.5e-5, rtol=1e-5, what="gx")
    assert_close(oracle.grad_w_f32(xin, idx, g, transposed=transposed), dgw, atol=1.5e-5, rtol=1e-5, what="gW")
    assert_close(oracle.grad_x_f64(idx, W, g, N, transposed=transposed), dgx, atol=1e-9, rtol=1e-9, what="gx64")
    assert_close(oracle.grad_w_f64(xin, idx, g, transposed=transposed), dgw, atol=1e-9, rtol=1e-9, what="gW64")


@pytest.mark.skipif(not oracle.ref_available(), reason="compiled reference kernels not present")
@pytest.mark.parametrize("size", SMALL_SIZES, ids=size_id)
@pytest.mark.parametrize("transposed", [False, True])
def test_oracle_matches_compiled_reference(size, transposed):
    x, idx, W, g = reference_style_inputs(size, seed=123, relu_grad=False)
    B, N, L, K = size
    xin = np.ascontiguousarray(x.T) if transposed else x
    for threads in (1, 3):
        y = oracle.ref_forward(xin, idx, W, transposed=transposed, threads=threads)
        gx, gw = oracle.ref_backward(xin, idx, W, g, transposed=transposed, threads=threads)
        assert_close(oracle.forward_f32(xin, idx, W, transposed=transposed, threads=threads), y, atol=2e-6, rtol=2e-6)
        assert_close(oracle.grad_x_f32(idx, W, g, N, transposed=transposed, threads=threads), gx, atol=4e-6, rtol=4e-6)
        assert_close(oracle.grad_w_f32(xin, idx, g, transposed=transposed, threads=threads), gw, atol=4e-6, rtol=4e-6)


def test_duplicate_indices_in_a_row_add():
    x = np.array([[1.0, 10.0]], np.float32)
    idx = np.array([[1, 1, 0]], np.int32)
    W = np.array([[2.0, 3.0, 5.0]], np.float32)
    assert oracle.forward_f32(x, idx, W)[0, 0] == 55.0
    g = np.array([[2.0]], np.float32)
    assert np.array_equal(oracle.grad_x_f32(idx, W, g, 2), [[10.0, 10.0]])
    assert np.array_equal(oracle.grad_w_f32(x, idx, g), [[20.0, 20.0, 2.0]])


def test_bias_and_grad_bias():
    x, idx, W, g = reference_style_inputs((12, 8, 32, 16))
    bias = np.linspace(-1, 1, 32).astype(np.float32)
    assert_close(oracle.forward_f32(x, idx, W, bias=bias), oracle.forward_f32(x, idx, W) + bias[None, :], atol=1e-6)
    assert_close(oracle.grad_bias_f64(g), g.astype(np.float64).sum(0), atol=1e-12)


@pytest.mark.parametrize("size", [(3, 5, 4, 2), (17, 12, 63, 44), (4, 300, 1000, 7)], ids=size_id)
def test_transposed_index_definition(size):
    B, N, L, K = size
    idx = reference_style_inputs(size)[1]
    rowptr, perm = oracle.transpose_index(idx, N)
    rp2, perm2 = oracle.transpose_index_np(idx, N)
    assert np.array_equal(rowptr, rp2) and np.array_equal(perm, perm2)
    flat = idx.ravel()
    assert rowptr[0] == 0 and rowptr[-1] == L * K
    assert np.array_equal(np.sort(perm), np.arange(L * K))
    keys = flat[perm]
    assert (np.diff(keys) >= 0).all()
    same = np.diff(keys) == 0
    assert (np.diff(perm)[same] > 0).all(), "ties must keep ascending positions"
    for i in range(N):
        assert (keys[rowptr[i]:rowptr[i + 1]] == i).all()


def test_transposed_index_rejects_out_of_range():
    with pytest.raises(ValueError):
        oracle.transpose_index(np.array([[0, 5]], np.int32), 5)


def test_bce_matches_closed_form():
    rng = np.random.default_rng(0)
    B, L = 5, 37
    z = (rng.standard_normal((B, L)) * 3).astype(np.float32)
    rows = [np.sort(rng.choice(L, size=rng.integers(0, 4), replace=False)) for _ in range(B)]
    row_ptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    labels = np.concatenate(rows).astype(np.int32) if row_ptr[-1] else np.zeros(0, np.int32)
    t = np.zeros((B, L))
    for b, r in enumerate(rows):
        t[b, r] = 1
    zd = z.astype(np.float64)
    elem = np.maximum(zd, 0) - zd * t + np.log1p(np.exp(-np.abs(zd)))
    loss, g = oracle.bce_f64(z, row_ptr, labels)
    assert abs(loss - elem.mean(axis=1).mean()) < 1e-12
    assert_close(g, (1 / (1 + np.exp(-zd)) - t) / (B * L), atol=1e-15, rtol=1e-12)


@pytest.mark.parametrize("squared", [True, False])
def test_hinge_losses_match_closed_form(squared):
    rng = np.random.default_rng(3)
    B, L = 6, 41
    z = (rng.standard_normal((B, L)) * 2).astype(np.float32)
    rows = [np.sort(rng.choice(L, size=rng.integers(0, 5), replace=False)) for _ in range(B)]
    row_ptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    labels = np.concatenate(rows).astype(np.int32)
    t = np.zeros((B, L))
    for b, r in enumerate(rows):
        t[b, r] = 1
    zd = z.astype(np.float64)
    sign = 2 * t - 1
    h = np.maximum(1 - sign * zd, 0)
    elem = h * h if squared else h
    grad = (-sign * 2 * h if squared else -sign * (h > 0)) / (B * L)
    loss, g = oracle.hinge_f64(z, row_ptr, labels, squared=squared)
    assert abs(loss - elem.mean(axis=1).mean()) < 1e-12
    assert_close(g, grad, atol=1e-15, rtol=1e-12)
    # finite differences of the loss in a few coordinates away from the kink
    eps = 1e-3
    for (b, o) in [(0, 0), (2, 17), (5, 40)] + [(b, int(r[0])) for b, r in enumerate(rows) if len(r)][:2]:
        if abs(h[b, o]) < 10 * eps:
            continue
        zp, zm = z.copy(), z.copy()
        zp[b, o] += eps
        zm[b, o] -= eps
        fd = (oracle.hinge_f64(zp, row_ptr, labels, squared, False)[0]
              - oracle.hinge_f64(zm, row_ptr, labels, squared, False)[0]) / (float(zp[b, o]) - float(zm[b, o]))
        assert abs(fd - g[b, o]) < 1e-6 * max(1.0, abs(g[b, o]) * B * L) / (B * L) + 1e-9


def test_adam_matches_textbook_form():
    rng = np.random.default_rng(1)
    n = 50
    w0 = rng.standard_normal(n)
    w, m, v = w0.copy(), np.zeros(n), np.zeros(n)
    wr, mr, vr = w0.copy(), np.zeros(n), np.zeros(n)
    lr, b1, b2, eps = 1e-3, 0.9, 0.999, 1e-7
    for step in range(1, 6):
        grad = rng.standard_normal(n)
        w, m, v = oracle.adam_f64(w, m, v, grad, lr, b1, b2, eps, step)
        mr = b1 * mr + (1 - b1) * grad
        vr = b2 * vr + (1 - b2) * grad * grad
        wr = wr - lr * np.sqrt(1 - b2 ** step) / (1 - b1 ** step) * mr / (np.sqrt(vr) + eps)
        assert_close(w, wr, atol=1e-14, rtol=1e-12)
        assert_close(m, mr, atol=1e-14, rtol=1e-12)
        assert_close(v, vr, atol=1e-14, rtol=1e-12)
