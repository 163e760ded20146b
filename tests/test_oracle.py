"""Pins the CPU oracle: against the reference's known-answer vectors, against the
committed outputs of the reference's own CPU convolution, and (where the compiled
reference is present) against that code run live."""
import glob
import json
import os

import numpy as np
import pytest

import oracle
from oracle import spectral


def _load(path):
    z = np.load(path)
    s = oracle.Shape(*[int(v) for v in z["shape"]])
    return s, z


def _fixtures(golden_dir=None):
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    return sorted(glob.glob(os.path.join(here, "refconv_*.npz")))


def _rel_linf(a, ref):
    return np.abs(a - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.mark.parametrize("path", _fixtures(), ids=lambda p: os.path.basename(p)[8:-4])
def test_restatement_matches_committed_reference_outputs(path):
    """fp64 restatement vs what test/ReferenceConvolutions.cpp returned (fp32 sums)."""
    s, z = _load(path)
    scale = float(z["scale"])
    assert _rel_linf(oracle.update_output(s, z["input"], z["weight"]), z["output"]) < 2e-5
    assert _rel_linf(oracle.update_grad_input(s, z["grad_output"], z["weight"]), z["grad_input"]) < 2e-5
    assert _rel_linf(oracle.acc_grad_weight(s, z["input"], z["grad_output"], scale), z["grad_weight"]) < 2e-5


@pytest.mark.parametrize("path", _fixtures(), ids=lambda p: os.path.basename(p)[8:-4])
def test_spectral_restatement_matches_spatial(path):
    """The frequency-domain algorithm (FFT -> per-bin product -> inverse, crop) equals
    the direct definition: this is the identity the whole path rests on."""
    s, z = _load(path)
    scale = float(z["scale"])
    x, w, go = z["input"], z["weight"], z["grad_output"]
    assert _rel_linf(spectral.update_output(x, w, None, s.padH, s.padW), oracle.update_output(s, x, w)) < 1e-12
    assert _rel_linf(spectral.update_grad_input(go, w, s.iH, s.iW, s.padH, s.padW),
                     oracle.update_grad_input(s, go, w)) < 1e-12
    assert _rel_linf(spectral.acc_grad_weight(x, go, s.kH, s.kW, s.padH, s.padW, scale),
                     oracle.acc_grad_weight(s, x, go, scale)) < 1e-12


def test_full_convolution_border_pattern():
    """Known answer of test/ConvolutionTest.cpp:1316-1374: a 7x7 plane of ones
    back-propagated through a 3x3 kernel of ones gives the 1-2-3 / 2-4-6 / 3-6-9
    border pattern on a 9x9 plane."""
    s = oracle.Shape(B=1, P=1, F=1, iH=9, iW=9, kH=3, kW=3)
    go = np.ones((1, 1, 7, 7), np.float32)
    w = np.ones((1, 1, 3, 3), np.float32)
    ramp = np.minimum(np.minimum(np.arange(9) + 1, 9 - np.arange(9)), 3)
    expected = np.outer(ramp, ramp).astype(np.float64)
    assert expected[0, 0] == 1 and expected[1, 1] == 4 and expected[4, 4] == 9 and expected[0, 4] == 3
    got = oracle.update_grad_input(s, go, w)[0, 0]
    np.testing.assert_array_equal(got, expected)
    got_f = spectral.update_grad_input(go, w, 9, 9, 0, 0)[0, 0]
    np.testing.assert_allclose(got_f, expected, atol=1e-12)


def test_fft_known_answers(golden_dir):
    """Literal spectra of test/FFTTest.cpp against the DFT restatement."""
    with open(os.path.join(golden_dir, "fft_known_answers.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) >= 6
    for c in cases:
        b0, b1 = c["batch"]
        shape = (b0, b1, c["rows"], c["cols"])
        if c["input_kind"] == "constant":
            x = np.ones(shape)
        else:
            idx = np.indices(shape)
            x = 0.1 * idx[0] + 0.2 * idx[1] + 0.3 * idx[2] + 0.4 * idx[3]
        got = spectral.rfft2_padded(x, c["fft_rows"], c["fft_cols"])
        exp = np.zeros((c["fft_rows"], c["fft_cols"] // 2 + 1), np.complex128)
        for r, col, re, im in c["nonzero"]:
            exp[r, col] = re + 1j * im
        tol = max(c["tol"], 1e-6) * max(1.0, np.abs(exp).max())
        if c["input_kind"] == "constant":
            for i in range(b0):
                for j in range(b1):
                    assert np.abs(got[i, j] - exp).max() <= tol, c["name"]
        else:
            assert np.abs(got[0, 0] - exp).max() <= tol, c["name"]


def test_transform_contract():
    """Padding offset, Hermitian half, un-normalised inverse (src/fft/FFTWrapperLua.cpp:235-237)."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 3, 5, 6))
    got = spectral.rfft2_padded(x, 8, 8, 1, 2)
    ref = np.fft.rfft2(np.pad(x, ((0, 0), (0, 0), (1, 2), (2, 0))), s=(8, 8))
    assert np.abs(got - ref).max() < 1e-12
    back = spectral.irfft2_unnormalised(spectral.rfft2_padded(x, 8), 8)
    assert np.abs(back[..., :5, :6] - 64 * x).max() < 1e-11
    assert np.abs(back[..., 5:, :]).max() < 1e-11


def test_bias_and_planes():
    rng = np.random.default_rng(7)
    s = oracle.Shape(B=3, P=2, F=4, iH=6, iW=7, kH=3, kW=2, padH=1, padW=1)
    x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
    w = rng.standard_normal((s.F, s.P, s.kH, s.kW)).astype(np.float32)
    b = rng.standard_normal(s.F).astype(np.float32)
    go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
    full = oracle.update_output(s, x, w, b)
    nob = oracle.update_output(s, x, w)
    np.testing.assert_allclose(full - nob, np.broadcast_to(b[None, :, None, None].astype(np.float64), full.shape), atol=1e-12)
    np.testing.assert_allclose(oracle.acc_grad_bias(s, go, 0.5), 0.5 * go.astype(np.float64).sum((0, 2, 3)), rtol=1e-12)
    bi, fi = np.array([2, 0]), np.array([1, 3])
    np.testing.assert_array_equal(oracle.update_output_planes(s, x, w, b, bi, fi), full[bi, fi])
    gi = oracle.update_grad_input(s, go, w)
    np.testing.assert_array_equal(oracle.update_grad_input_planes(s, go, w, bi, np.array([1, 0])), gi[bi, [1, 0]])
    gw = oracle.acc_grad_weight(s, x, go, 0.25)
    np.testing.assert_array_equal(oracle.acc_grad_weight_planes(s, x, go, 0.25, fi, np.array([0, 1])), gw[fi, [0, 1]])


@pytest.mark.skipif(not oracle.reference_available(), reason="compiled reference not present")
def test_restatement_matches_live_reference():
    rng = np.random.default_rng(11)
    for s in (oracle.Shape(2, 3, 4, 8, 8, 3, 3), oracle.Shape(2, 2, 3, 9, 7, 4, 2, 3, 1),
              oracle.Shape(1, 1, 1, 1, 1, 1, 1)):
        x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
        w = rng.standard_normal((s.F, s.P, s.kH, s.kW)).astype(np.float32)
        go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
        assert _rel_linf(oracle.update_output(s, x, w), oracle.reference_update_output(s, x, w, threads=2)) < 1e-5
        assert _rel_linf(oracle.update_grad_input(s, go, w), oracle.reference_update_grad_input(s, go, w)) < 1e-5
        assert _rel_linf(oracle.acc_grad_weight(s, x, go, 0.6),
                         oracle.reference_acc_grad_weight(s, x, go, 0.6, threads=2)) < 1e-5
