"""Generates the golden fixtures in this directory from the reference's own CPU kernels.

Needs a checkout of the reference (``$FFI_REFERENCE_ROOT``; a built-in default location is tried when it is unset):
``oracle/build_oracle.py`` compiles its tfsparse/cc/kernels/forward.cpp and backward.cpp
into ``oracle/_ref/libffi_ref.so`` and this script runs them (single thread) on the seeded
inputs of ``tests/cases.py`` for each size fixture of testing/test.cpp:50-59.

Per fixture ``B*_N*_L*_K*.npz`` holds the reference outputs for the plain layout
(y, grad_x, grad_W), the largest difference the transposed-layout kernels showed against
them (the reference's own transpose-consistency bound is 1.5e-5, testing/test.cpp:125,164),
and a SHA-256 of the inputs, so that a drift of the input recipe is detected.
The 4,000,000-unit fixture stores strided samples of y and grad_W instead of the full arrays.

Run:  python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from cases import REFERENCE_SIZES, HUGE_SIZE, golden_path, reference_style_inputs  # noqa: E402

SAMPLE_STRIDE = 4001


def input_digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    if not oracle.ref_available():
        raise SystemExit("reference checkout not found: cannot generate golden fixtures")
    for size in REFERENCE_SIZES:
        x, idx, W, g = reference_style_inputs(size)
        y = oracle.ref_forward(x, idx, W, transposed=False, threads=1)
        gx, gW = oracle.ref_backward(x, idx, W, g, transposed=False, threads=1)
        xt = np.ascontiguousarray(x.T)
        y_tp = oracle.ref_forward(xt, idx, W, transposed=True, threads=1)
        gx_tp, gW_tp = oracle.ref_backward(xt, idx, W, g, transposed=True, threads=1)
        tp_diff = max(float(np.abs(y - y_tp).max()), float(np.abs(gx - gx_tp.T).max()),
                      float(np.abs(gW - gW_tp).max()))
        assert tp_diff < 1.5e-5, tp_diff
        out = dict(size=np.array(size, np.int64), digest=np.array(input_digest(x, idx, W, g)),
                   tp_max_diff=np.array(tp_diff), grad_x=gx)
        if size == HUGE_SIZE:
            out.update(y_sample=y.ravel()[::SAMPLE_STRIDE], grad_w_sample=gW.ravel()[::SAMPLE_STRIDE],
                       sample_stride=np.array(SAMPLE_STRIDE))
        else:
            out.update(y=y, grad_w=gW)
        np.savez_compressed(golden_path(size), **out)
        print(size, "tp_max_diff", tp_diff, os.path.getsize(golden_path(size)), "bytes")


if __name__ == "__main__":
    main()
