"""Generates tests/golden/refconv_*.npz from the reference's own CPU convolution.

Run in a container that has the reference checkout (it compiles
test/ReferenceConvolutions.cpp from there through oracle/Makefile):

    python tests/golden/make_golden.py

Each fixture stores the inputs and what the three reference functions returned
(fp32, single thread).  The deterministic inputs follow the reference's own
fixture generator (value = sum of factor_d * index_d, test/TestUtils.cpp:92-112,
factors at test/ConvolutionTest.cpp:79-87); the random ones are seeded numpy.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def factor_tensor(shape, factors):
    idx = np.indices(shape, dtype=np.float32)
    out = np.zeros(shape, np.float32)
    for d, f in enumerate(factors):
        out += np.float32(f) * idx[d]
    return out


def emit(name, s, x, w, go, scale):
    out = oracle.reference_update_output(s, x, w)
    gi = oracle.reference_update_grad_input(s, go, w)
    gw = oracle.reference_acc_grad_weight(s, x, go, scale)
    np.savez_compressed(
        os.path.join(HERE, f"refconv_{name}.npz"),
        shape=np.array([s.B, s.P, s.F, s.iH, s.iW, s.kH, s.kW, s.padH, s.padW], np.int64),
        input=x, weight=w, grad_output=go, scale=np.float32(scale),
        output=out, grad_input=gi, grad_weight=gw)
    print(name, out.shape, gi.shape, gw.shape)


def main():
    assert oracle.reference_available(), "needs the reference checkout"
    # kCuFFTParams(16, 8, 8, 8, 16, 4, 1) = {batch, inputPlanes, inputRow, inputCol,
    # outputPlanes, filterSize, filterStride}  (test/ConvolutionTest.cpp:1213)
    s = oracle.Shape(B=16, P=8, F=16, iH=8, iW=8, kH=4, kW=4)
    x = factor_tensor((s.B, s.P, s.iH, s.iW), (0.1, 0.3, 0.4, 0.5)) * np.float32(0.01)
    w = factor_tensor((s.F, s.P, s.kH, s.kW), (0.2, 0.3, 0.8, 0.9)) * np.float32(0.01)
    go = factor_tensor((s.B, s.F, s.oH, s.oW), (0.1, 0.2, 0.6, 0.7)) * np.float32(0.01)
    emit("cufftparams_factors", s, x, w, go, 1.0)

    rng = np.random.default_rng(20241)
    # padded, rectangular image and kernel (shape family of test/test_FFT.lua:257-293)
    s = oracle.Shape(B=3, P=5, F=4, iH=13, iW=14, kH=7, kW=5, padH=2, padW=1)
    emit("rect_padded_random", s,
         rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32),
         rng.uniform(-0.1, 0.1, (s.F, s.P, s.kH, s.kW)).astype(np.float32),
         rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32), 0.37)
    # kernel as large as the image, 1x1 output
    s = oracle.Shape(B=2, P=3, F=2, iH=5, iW=5, kH=5, kW=5)
    emit("kernel_equals_image", s,
         rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32),
         rng.uniform(-0.2, 0.2, (s.F, s.P, s.kH, s.kW)).astype(np.float32),
         rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32), 1.0)
    # a slice of the first benchmark configuration (test/benchmark_fft.lua:42)
    s = oracle.Shape(B=2, P=16, F=16, iH=32, iW=32, kH=5, kW=5)
    emit("config1_slice", s,
         rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32),
         rng.uniform(-0.05, 0.05, (s.F, s.P, s.kH, s.kW)).astype(np.float32),
         rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32), 1.0)


if __name__ == "__main__":
    main()
