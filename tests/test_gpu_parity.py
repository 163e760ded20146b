"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Tolerances (written where used):
  * transforms: 5e-6 * max|spectrum| (the reference's own FFT test allows 4e-7 of the
    maximum against cuFFT, test/test_FFTModule.lua:13, at sizes where both are fp32;
    here the yardstick is fp64);
  * the three passes: max|x - ref| <= 1e-4 * max|ref| against the fp64 oracle, the bar
    of the benchmark definition (the reference's own module test uses a relative L2 of
    1e-4, test/test_FFT.lua:15,239-250).
"""
import ctypes
import glob
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import spectral
from fbcunn_b200 import FFTWrapper, SpatialConvolutionFBFFT, capi

pytestmark = pytest.mark.gpu

PASS_TOL = 1e-4
FFT_TOL = 5e-6
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _rel(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def _module(s: oracle.Shape, weight, bias=None, **kw):
    m = SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, **kw)
    m.weight.copy_(_dev(weight))
    if bias is None:
        m.bias.zero_()
    else:
        m.bias.copy_(_dev(bias))
    return m


def _data(s: oracle.Shape, seed, bias=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
    bound = 1.0 / np.sqrt(s.kH * s.kW * s.P)
    w = rng.uniform(-bound, bound, (s.F, s.P, s.kH, s.kW)).astype(np.float32)
    go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
    b = rng.uniform(-0.01, 0.01, s.F).astype(np.float32) if bias else None
    return x, w, go, b


def _check_three_passes(s, x, w, go, b, scale=1.0, **kw):
    m = _module(s, w, b, **kw)
    dx, dgo = _dev(x), _dev(go)
    out = m.updateOutput(dx).cpu().numpy()
    gi = m.updateGradInput(dx, dgo).cpu().numpy()
    m.accGradParameters(dx, dgo, scale)
    gw, gb = m.gradWeight.cpu().numpy(), m.gradBias.cpu().numpy()
    assert _rel(out, oracle.update_output(s, x, w, b)) <= PASS_TOL
    assert _rel(gi, oracle.update_grad_input(s, go, w)) <= PASS_TOL
    assert _rel(gw, oracle.acc_grad_weight(s, x, go, scale)) <= PASS_TOL
    assert _rel(gb, oracle.acc_grad_bias(s, go, scale)) <= PASS_TOL
    return m


# ---------------------------------------------------------------------------
# transforms
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("N", [8, 16, 32, 64, 128])
def test_fft2d_matches_dft(N):
    rng = np.random.default_rng(N)
    for (d1, d2, h, w, pu, pl) in [(3, 5, N, N, 0, 0), (2, 20, 3, 3, 0, 0), (4, 7, N - 3, N - 5, 1, 2),
                                   (1, 1, 1, 1, 0, 0), (5, 33, max(1, N // 2), max(1, N // 2 + 1), 0, 1)]:
        x = rng.standard_normal((d1, d2, h, w)).astype(np.float32)
        ref = spectral.rfft2_padded(x, N, N, pu, pl)
        for transposed in (False, True):
            wr = FFTWrapper("fbfft", pl, pu)
            freq = FFTWrapper.frequency_tensor(d1, d2, N, transposed=transposed)
            freq.fill_(float("nan"))
            wr.fft(_dev(x), freq, N, transposed=transposed)
            inner = d1 if transposed else d2
            got = FFTWrapper.to_plane_major(freq, inner, N, transposed).cpu().numpy()
            assert np.abs(got - ref).max() <= FFT_TOL * np.abs(ref).max(), (N, d1, d2, h, w, transposed)
            assert torch.all(freq[:, :, inner:] == 0), "padding planes are written as zero"


def test_fft2d_known_answers_of_the_reference():
    """Spectra held by test/FFTTest.cpp whose transform size this library supports are
    power-of-two squares only, so the literal vectors are checked through the oracle
    (tests/test_oracle.py) and here the same inputs are pushed through size 8."""
    ones = np.ones((1, 1, 2, 2), np.float32)
    var = np.array([[[[0.0, 0.4], [0.3, 0.7]]]], np.float32)  # 0.3*row + 0.4*col, test/TestUtils.cpp:92-112
    for x in (ones, var):
        freq = FFTWrapper.frequency_tensor(1, 1, 8)
        FFTWrapper().fft(_dev(x), freq, 8)
        got = FFTWrapper.to_plane_major(freq, 1, 8).cpu().numpy()[0, 0]
        ref = spectral.rfft2_padded(x, 8)[0, 0]
        assert np.abs(got - ref).max() <= 1e-6
        assert abs(got[0, 0] - x.sum()) <= 1e-6  # DC term: 4.0 resp. 1.4 (test/FFTTest.cpp:212-219,280-289)


@pytest.mark.parametrize("N", [8, 16, 32, 64, 128])
def test_ifft2d_crop_bias_and_round_trip(N):
    rng = np.random.default_rng(100 + N)
    for (d1, d2, oh, ow, oy, ox) in [(3, 5, N, N, 0, 0), (2, 18, 3, 3, 0, 0), (2, 7, N - 3, N - 5, 1, 2),
                                     (1, 1, 1, 1, 2, 3), (4, 9, N - 4, N - 4, 0, 0)]:
        full = rng.standard_normal((d1, d2, N, N))
        spec = torch.from_numpy(np.fft.rfft2(full).astype(np.complex64)).cuda()
        freq = FFTWrapper.from_plane_major(spec, N)
        bias = rng.standard_normal(d2).astype(np.float32)
        out = torch.full((d1, d2, oh, ow), float("nan"), device="cuda")
        FFTWrapper("fbfft", ox, oy).ffti(out, freq, N, bias=_dev(bias))
        ref = N * N * full[:, :, oy:oy + oh, ox:ox + ow] + bias[None, :, None, None]
        assert _rel(out.cpu().numpy(), ref) <= FFT_TOL * 4
    # fft then ffti gives N^2 times the input (un-normalised inverse, src/fft/FFTWrapperLua.cpp:235-237)
    x = rng.standard_normal((3, 6, N - 2, N - 1)).astype(np.float32)
    freq = FFTWrapper.frequency_tensor(3, 6, N)
    w = FFTWrapper("fbfft", 1, 2)
    w.fft(_dev(x), freq, N)
    back = torch.empty(3, 6, N - 2, N - 1, device="cuda")
    w.ffti(back, freq, N)
    assert _rel(back.cpu().numpy() / (N * N), x.astype(np.float64)) <= FFT_TOL * 4


# ---------------------------------------------------------------------------
# contraction and bias kernels
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("use_simt", [1, 0])
@pytest.mark.parametrize("mn_a,mn_b", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("conj_a,conj_b", [(0, 1), (0, 0), (1, 0)])
def test_transpose_mm(use_simt, conj_a, conj_b, mn_a, mn_b):
    """mn_x: the operand is handed over stored [bins][k][rows] (contraction index as the row
    index), the way updateGradInput reads the weight spectrum and accGradParameters both of its
    operands."""
    rng = np.random.default_rng(3)
    for (bins, m, n, k) in [(5, 7, 9, 3), (3, 64, 64, 8), (2, 130, 70, 21), (1, 1, 1, 1), (4, 16, 128, 128),
                            (3, 130, 3, 96), (2, 96, 4, 128), (3, 128, 384, 384), (2, 300, 200, 77),
                            # tiles of 16 / 32 / 64 complex columns (batch shards on the column side)
                            (4, 384, 16, 384), (3, 200, 24, 40), (2, 384, 48, 64), (2, 129, 33, 17)]:
        kp, npad = (k + 3) // 4 * 4, (n + 3) // 4 * 4
        a = np.zeros((bins, m, kp), np.complex64)
        b = np.zeros((bins, n, kp), np.complex64)
        a[:, :, :k] = rng.standard_normal((bins, m, k)) + 1j * rng.standard_normal((bins, m, k))
        b[:, :, :k] = rng.standard_normal((bins, n, k)) + 1j * rng.standard_normal((bins, n, k))
        c = torch.full((bins, m, npad), float("nan"), dtype=torch.complex64, device="cuda")

        def stored(x, rows, mn):
            if not mn:
                return torch.from_numpy(x).cuda()
            t = np.zeros((bins, k, (rows + 3) // 4 * 4), np.complex64)
            t[:, :, :rows] = x[:, :, :k].transpose(0, 2, 1)
            return torch.from_numpy(t).cuda()

        da, db = stored(a, m, mn_a), stored(b, n, mn_b)
        capi.check(capi.lib().fbfftconv_transpose_mm(
            ctypes.c_void_p(da.data_ptr()), ctypes.c_void_p(db.data_ptr()), ctypes.c_void_p(c.data_ptr()),
            bins, m, n, k, ctypes.c_float(0.25), conj_a | (mn_a << 1), conj_b | (mn_b << 1), use_simt,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        a64 = a.astype(np.complex128).conj() if conj_a else a.astype(np.complex128)
        b64 = b.astype(np.complex128).conj() if conj_b else b.astype(np.complex128)
        ref = 0.25 * np.einsum("zmk,znk->zmn", a64, b64)
        got = c.cpu().numpy()[:, :, :n]
        # exact-fp32 CUDA-core kernel: 2e-6; tensor cores with the 3xTF32 split (each product
        # good to about 2^-21): 1e-5, still ten times inside the 1e-4 bar of the passes
        tol = 2e-6 if use_simt else 1e-5
        assert capi.lib().fbfftconv_tensor_core_status(1) == 0, "a bounded wait ran out on the device"
        assert np.abs(got - ref).max() <= tol * np.abs(ref).max(), (bins, m, n, k)
        assert np.all(c.cpu().numpy()[:, :, n:] == 0), "the padding columns of C are written as zero"


def test_bias_kernels():
    rng = np.random.default_rng(9)
    B, F, h, w = 5, 7, 6, 9
    out = rng.standard_normal((B, F, h, w)).astype(np.float32)
    bias = rng.standard_normal(F).astype(np.float32)
    d = _dev(out)
    s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.check(capi.lib().fbfftconv_update_output_bias(ctypes.c_void_p(d.data_ptr()), ctypes.c_void_p(_dev(bias).data_ptr()), B, F, h, w, s))
    np.testing.assert_allclose(d.cpu().numpy(), out + bias[None, :, None, None], rtol=0, atol=1e-6)
    gb = torch.full((F,), 2.0, device="cuda")
    scratch = torch.empty(B * F, device="cuda")
    go = _dev(out)
    sh = oracle.Shape(B, 1, F, h, w, 1, 1)
    capi.check(capi.lib().fbfftconv_acc_grad_parameters_bias(ctypes.c_void_p(go.data_ptr()), ctypes.c_void_p(gb.data_ptr()),
                                                            ctypes.c_void_p(scratch.data_ptr()), B, F, h, w, ctypes.c_float(0.5), 0, s))
    ref = oracle.acc_grad_bias(sh, out, 0.5)
    assert _rel(gb.cpu().numpy(), ref) <= 1e-5   # overwrite (src/ConvolutionBias.cu:95)
    capi.check(capi.lib().fbfftconv_acc_grad_parameters_bias(ctypes.c_void_p(go.data_ptr()), ctypes.c_void_p(gb.data_ptr()),
                                                            ctypes.c_void_p(scratch.data_ptr()), B, F, h, w, ctypes.c_float(0.5), 1, s))
    assert _rel(gb.cpu().numpy(), 2 * ref) <= 1e-5


# ---------------------------------------------------------------------------
# the three passes
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "refconv_*.npz"))),
                         ids=lambda p: os.path.basename(p)[8:-4])
def test_passes_match_committed_reference_outputs(path):
    """Against what the reference's own CPU convolution returned (fp32 sums there, so
    the bound is the looser of the two error budgets)."""
    z = np.load(path)
    s = oracle.Shape(*[int(v) for v in z["shape"]])
    scale = float(z["scale"])
    m = _check_three_passes(s, z["input"], z["weight"], z["grad_output"], None, scale)
    assert _rel(m.output.cpu().numpy(), z["output"].astype(np.float64)) <= PASS_TOL
    assert _rel(m.gradInput.cpu().numpy(), z["grad_input"].astype(np.float64)) <= PASS_TOL
    assert _rel(m.gradWeight.cpu().numpy(), z["grad_weight"].astype(np.float64)) <= PASS_TOL


def test_full_convolution_border_pattern():
    """Known answer of test/ConvolutionTest.cpp:1316-1374."""
    s = oracle.Shape(1, 1, 1, 9, 9, 3, 3)
    m = _module(s, np.ones((1, 1, 3, 3), np.float32))
    gi = m.updateGradInput(torch.zeros(1, 1, 9, 9, device="cuda"), torch.ones(1, 1, 7, 7, device="cuda"))
    ramp = np.minimum(np.minimum(np.arange(9) + 1, 9 - np.arange(9)), 3)
    np.testing.assert_allclose(gi.cpu().numpy()[0, 0], np.outer(ramp, ramp), atol=2e-5)


def test_config1_all_passes():
    """The benchmark's first configuration in full: 16 x 16 planes x 32x32, 16 filters, 5x5."""
    s = oracle.Shape(16, 16, 16, 32, 32, 5, 5)
    x, w, go, _ = _data(s, 1000)
    m = _check_three_passes(s, x, w, go, None)
    assert m.fftSize == 32


# shapes of test/test_FFT.lua:257-293 and test/test_SpatialConvolutionTuned.lua:88-125:
# {B, P, F, kH, kW, iH, iW, padH, padW}
REGRESSION_SHAPES = [
    (1, 1, 1, 1, 1, 1, 1, 0, 0), (1, 1, 1, 1, 1, 1, 13, 0, 0), (2, 3, 4, 3, 3, 3, 3, 0, 0),
    (2, 2, 2, 5, 5, 5, 5, 0, 0), (2, 3, 2, 7, 5, 13, 14, 0, 0), (2, 3, 2, 7, 5, 13, 14, 2, 1),
    (1, 2, 3, 3, 4, 19, 23, 1, 2), (128, 64, 64, 1, 1, 3, 3, 0, 0), (128, 64, 64, 3, 3, 3, 3, 0, 0),
    (1, 3, 16, 3, 3, 8, 8, 0, 0), (64, 16, 16, 3, 3, 16, 16, 1, 1), (1, 128, 128, 3, 3, 32, 32, 0, 0),
    (2, 3, 5, 8, 8, 11, 11, 0, 0), (2, 2, 3, 13, 14, 20, 17, 0, 0), (1, 2, 2, 3, 3, 128, 128, 0, 0),
    (3, 5, 6, 9, 9, 64, 64, 0, 0), (2, 3, 96, 11, 11, 128, 128, 0, 0), (2, 5, 3, 3, 3, 33, 40, 2, 2),
    (2, 4, 4, 3, 3, 126, 126, 1, 1), (2, 3, 5, 9, 9, 64, 64, 0, 0), (3, 1, 2, 5, 5, 40, 50, 2, 1),
    (5, 2, 7, 3, 5, 70, 33, 0, 2),
]


@pytest.mark.parametrize("shape", REGRESSION_SHAPES, ids=lambda t: "x".join(map(str, t)))
def test_regression_shapes(shape):
    B, P, F, kH, kW, iH, iW, padH, padW = shape
    s = oracle.Shape(B, P, F, iH, iW, kH, kW, padH, padW)
    x, w, go, b = _data(s, hash(shape) % 10000, bias=True)
    _check_three_passes(s, x, w, go, b, scale=0.7)


def test_thin_layers_in_both_frequency_layouts():
    """Layers with <= 4 input planes use plane-major buffers and the streaming contraction at
    transform sizes 64 / 128; the bin-major path must give the same result."""
    s = oracle.Shape(6, 3, 10, 60, 57, 7, 4, 1, 2)
    x, w, go, b = _data(s, 4242, bias=True)
    a = _check_three_passes(s, x, w, go, b, scale=1.3)
    c = _check_three_passes(s, x, w, go, b, scale=1.3, contraction="bin_major")
    for name in ("output", "gradInput", "gradWeight", "gradBias"):
        ta, tc = getattr(a, name), getattr(c, name)
        assert float((ta - tc).abs().max()) <= 2e-5 * float(tc.abs().max()), name


def _stage_launches(m):
    """(pass, stage) -> number of timed launches since profiling was switched on."""
    lib = capi.lib()
    out = {}
    for pi in range(3):
        for si in range(6):
            ms, n = ctypes.c_double(), ctypes.c_int()
            capi.check(lib.fbfftconv_profile_read(m._handle, pi, si, ctypes.byref(ms), ctypes.byref(n)))
            out[(pi, si)] = n.value
    return out


@pytest.mark.parametrize("plane_major", [True, False])
def test_spectrum_reuse_across_the_passes_of_a_step(plane_major):
    """memoryReusePolicy of the reference (fbcunn/SpatialConvolutionFFT.lua:405-416): the backward
    passes take over spectra of the earlier passes.  Results must not change, and the transforms
    are really skipped in both frequency layouts (a spectrum is written once and every pass reads
    it whichever way its sum runs)."""
    s = oracle.Shape(4, 3, 6, 50, 44, 5, 6, 1, 0) if plane_major else oracle.Shape(4, 8, 6, 20, 18, 3, 4, 1, 0)
    x, w, go, b = _data(s, 991, bias=True)
    m = SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, "all")
    m.weight.copy_(_dev(w))
    m.bias.copy_(_dev(b))
    dx, dgo = _dev(x), _dev(go)
    m.updateOutput(dx)
    lib = capi.lib()
    capi.check(lib.fbfftconv_profile_enable(m._handle, 1))
    capi.check(lib.fbfftconv_profile_reset(m._handle))
    for _ in range(2):  # a second step must find the buffers in a usable state again
        out = m.updateOutput(dx).cpu().numpy()
        gi = m.updateGradInput(dx, dgo).cpu().numpy()
        m.accGradParameters(dx, dgo, 0.8)
        assert _rel(out, oracle.update_output(s, x, w, b)) <= PASS_TOL
        assert _rel(gi, oracle.update_grad_input(s, go, w)) <= PASS_TOL
        assert _rel(m.gradWeight.cpu().numpy(), oracle.acc_grad_weight(s, x, go, 0.8)) <= PASS_TOL
        assert _rel(m.gradBias.cpu().numpy(), oracle.acc_grad_bias(s, go, 0.8)) <= PASS_TOL
    torch.cuda.synchronize()
    n = _stage_launches(m)
    FFT_A, FFT_B = 0, 1
    assert n[(0, FFT_A)] == 2 and n[(0, FFT_B)] == 2 and n[(1, FFT_A)] == 2
    assert n[(1, FFT_B)] == 0, "weight spectrum of updateOutput"
    assert n[(2, FFT_A)] == 0, "gradOutput spectrum of updateGradInput"
    assert n[(2, FFT_B)] == 0, "input spectrum of updateOutput"
    # accGradParameters on its own (nothing to take over) still transforms what it needs
    m2 = SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, "all")
    m2.accGradParameters(dx, dgo, 0.8)
    assert _rel(m2.gradWeight.cpu().numpy(), oracle.acc_grad_weight(s, x, go, 0.8)) <= PASS_TOL


@pytest.mark.parametrize("shape", [oracle.Shape(4, 8, 12, 14, 14, 3, 3, 1, 1), oracle.Shape(2, 3, 4, 40, 40, 5, 5, 0, 0)])
def test_passes_replay_from_a_cuda_graph(shape):
    """After the first call a pass allocates nothing and only enqueues work on the caller's stream,
    so a training step can be captured once and replayed: small layers are bound by launch gaps."""
    s = shape
    x, w, go, b = _data(s, 31, bias=True)
    m = _module(s, w, b)
    dx, dgo = _dev(x), _dev(go)
    m.updateOutput(dx)
    m.updateGradInput(dx, dgo)
    m.accGradParameters(dx, dgo, 1.0)          # warm: workspace and staging exist now
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        m.updateOutput(dx)
        m.updateGradInput(dx, dgo)
        m.accGradParameters(dx, dgo, 1.0)
    x2, _, go2, _ = _data(s, 32, bias=True)     # new contents in the captured buffers
    dx.copy_(_dev(x2))
    dgo.copy_(_dev(go2))
    m.output.zero_()
    m.gradInput.zero_()
    m.gradWeight.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert _rel(m.output.cpu().numpy(), oracle.update_output(s, x2, w, b)) <= PASS_TOL
    assert _rel(m.gradInput.cpu().numpy(), oracle.update_grad_input(s, go2, w)) <= PASS_TOL
    assert _rel(m.gradWeight.cpu().numpy(), oracle.acc_grad_weight(s, x2, go2, 1.0)) <= PASS_TOL
    assert _rel(m.gradBias.cpu().numpy(), oracle.acc_grad_bias(s, go2, 1.0)) <= PASS_TOL


@pytest.mark.parametrize("shape", [
    oracle.Shape(1, 1, 1, 8, 8, 1, 1, 0, 0),          # 1x1 kernel, one plane of each kind
    oracle.Shape(2, 1, 1, 5, 7, 5, 7, 0, 0),          # kernel as large as the image: 1x1 output
    oracle.Shape(1, 2, 3, 128, 128, 3, 3, 0, 0),      # the largest transform exactly filled
    oracle.Shape(1, 2, 3, 126, 120, 3, 5, 1, 2),      # padded image reaches 128 in one direction
    oracle.Shape(2, 130, 70, 9, 9, 3, 3, 1, 1),       # more than 128 input planes: K and M tails on the tensor cores
    oracle.Shape(3, 40, 260, 6, 6, 2, 2, 0, 0),       # more than 256 filters: several column tiles
    oracle.Shape(130, 5, 6, 4, 4, 2, 2, 1, 1),        # batch above one 128-row tile
])
def test_edge_shapes(shape):
    x, w, go, b = _data(shape, 1234, bias=True)
    _check_three_passes(shape, x, w, go, b, scale=0.9)


def test_random_sweep():
    """Recipe of test/test_FFT.lua:82-107: B = 4*rand(4), planes <= 13, k <= 7, pad <= min(4, k-1)."""
    rng = np.random.default_rng(424242)
    for _ in range(25):
        B = 4 * int(rng.integers(1, 5))
        P, F = int(rng.integers(1, 14)), int(rng.integers(1, 14))
        kH, kW = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        padH, padW = int(rng.integers(0, min(4, kH - 1) + 1)), int(rng.integers(0, min(4, kW - 1) + 1))
        iH, iW = int(rng.integers(kH, 41)), int(rng.integers(kW, 41))
        s = oracle.Shape(B, P, F, iH, iW, kH, kW, padH, padW)
        x, w, go, b = _data(s, int(rng.integers(1 << 30)), bias=True)
        _check_three_passes(s, x, w, go, b, scale=float(rng.uniform(0.1, 2.0)))


def test_reference_semantics_of_gradients_and_skip_bias():
    s = oracle.Shape(4, 3, 5, 12, 12, 3, 3, 1, 1)
    x, w, go, b = _data(s, 77, bias=True)
    dx, dgo = _dev(x), _dev(go)
    ref_w, ref_b = oracle.acc_grad_weight(s, x, go, 1.0), oracle.acc_grad_bias(s, go, 1.0)
    m = _module(s, w, b)
    m.gradWeight.fill_(5.0)
    m.gradBias.fill_(5.0)
    m.accGradParameters(dx, dgo)  # overwrites, as the reference does
    assert _rel(m.gradWeight.cpu().numpy(), ref_w) <= PASS_TOL
    assert _rel(m.gradBias.cpu().numpy(), ref_b) <= PASS_TOL
    m.gradBias.fill_(3.0)
    m.accGradParameters(dx, dgo, skipBias=True)
    assert torch.all(m.gradBias == 3.0)
    acc = _module(s, w, b, accumulate=True)  # nn contract: +=
    acc.accGradParameters(dx, dgo)
    acc.accGradParameters(dx, dgo, 0.5)
    assert _rel(acc.gradWeight.cpu().numpy(), 1.5 * ref_w) <= PASS_TOL
    assert _rel(acc.gradBias.cpu().numpy(), 1.5 * ref_b) <= PASS_TOL
    out_nb = m.updateOutput(dx, skipBias=True).cpu().numpy()
    assert _rel(out_nb, oracle.update_output(s, x, w, None)) <= PASS_TOL
    # the batch may change between calls: buffers follow (superset of the reference)
    x2 = x[:2].copy()
    assert _rel(m.updateOutput(_dev(x2)).cpu().numpy(), oracle.update_output(oracle.Shape(2, 3, 5, 12, 12, 3, 3, 1, 1), x2, w, b)) <= PASS_TOL


def test_host_buffer_entry_points():
    s = oracle.Shape(3, 4, 5, 10, 9, 3, 2, 1, 0)
    x, w, go, b = _data(s, 5, bias=True)
    lib = capi.lib()
    desc = capi.Desc(s.B, s.P, s.F, s.iH, s.iW, s.kH, s.kW, 1, 1, s.padH, s.padW, 0, 0)
    h = ctypes.c_void_p()
    capi.check(lib.fbfftconv_create(ctypes.byref(desc), ctypes.byref(h)))
    out = torch.empty((s.B, s.F, s.oH, s.oW)).pin_memory()
    gi = torch.empty((s.B, s.P, s.iH, s.iW)).pin_memory()
    gw = torch.empty((s.F, s.P, s.kH, s.kW)).pin_memory()
    gb = torch.empty((s.F,)).pin_memory()
    tx, tw, tgo, tb = (torch.from_numpy(a).pin_memory() for a in (x, w, go, b))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    capi.check(lib.fbfftconv_update_output_host(h, p(tx), p(tw), p(tb), p(out), st))
    capi.check(lib.fbfftconv_update_grad_input_host(h, p(tgo), p(tw), p(gi), st))
    capi.check(lib.fbfftconv_acc_grad_parameters_host(h, p(tx), p(tgo), p(gw), p(gb), ctypes.c_float(0.5), st))
    assert _rel(out.numpy(), oracle.update_output(s, x, w, b)) <= PASS_TOL
    assert _rel(gi.numpy(), oracle.update_grad_input(s, go, w)) <= PASS_TOL
    assert _rel(gw.numpy(), oracle.acc_grad_weight(s, x, go, 0.5)) <= PASS_TOL
    assert _rel(gb.numpy(), oracle.acc_grad_bias(s, go, 0.5)) <= PASS_TOL
    lib.fbfftconv_destroy(h)


# bin-major on CUDA cores; plane-major (three input planes, 64-point transform); tensor cores with the
# batch on the MMA's column side; tensor cores with the batch on its rows
@pytest.mark.parametrize("s", [oracle.Shape(6, 4, 5, 30, 29, 3, 2, 1, 0), oracle.Shape(4, 3, 6, 60, 50, 5, 5, 0, 0),
                               oracle.Shape(8, 16, 24, 20, 20, 5, 5, 0, 0), oracle.Shape(72, 16, 16, 12, 12, 3, 3, 1, 1)],
                         ids=["simt", "plane_major", "tc_batch_on_columns", "tc"])
def test_asynchronous_host_buffer_entry_points(s):
    """Three passes enqueued without waiting, results read after one fbfftconv_host_sync; repeated with
    new data so that the staging buffers of a pass are reused while the previous step is in flight.
    The middle step is one backward call, whose two passes share the spectrum of gradOutput."""
    lib = capi.lib()
    desc = capi.Desc(s.B, s.P, s.F, s.iH, s.iW, s.kH, s.kW, 1, 1, s.padH, s.padW, 0, 0)
    h = ctypes.c_void_p()
    capi.check(lib.fbfftconv_create(ctypes.byref(desc), ctypes.byref(h)))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    steps = []
    for step in range(3):
        x, w, go, b = _data(s, 50 + step, bias=True)
        host = dict(x=x, w=w, go=go, b=b,
                    out=torch.empty((s.B, s.F, s.oH, s.oW)).pin_memory(), gi=torch.empty((s.B, s.P, s.iH, s.iW)).pin_memory(),
                    gw=torch.empty((s.F, s.P, s.kH, s.kW)).pin_memory(), gb=torch.empty((s.F,)).pin_memory(),
                    tx=torch.from_numpy(x).pin_memory(), tw=torch.from_numpy(w).pin_memory(),
                    tgo=torch.from_numpy(go).pin_memory(), tb=torch.from_numpy(b).pin_memory())
        steps.append(host)
        capi.check(lib.fbfftconv_update_output_host_async(h, p(host["tx"]), p(host["tw"]), p(host["tb"]), p(host["out"]), st))
        if step == 1:   # nn.Module:backward in one call
            capi.check(lib.fbfftconv_backward_host_async(h, p(host["tx"]), p(host["tgo"]), p(host["tw"]), p(host["gi"]),
                                                         p(host["gw"]), p(host["gb"]), ctypes.c_float(0.5), st))
        else:
            capi.check(lib.fbfftconv_update_grad_input_host_async(h, p(host["tgo"]), p(host["tw"]), p(host["gi"]), st))
            capi.check(lib.fbfftconv_acc_grad_parameters_host_async(h, p(host["tx"]), p(host["tgo"]), p(host["gw"]),
                                                                    p(host["gb"]), ctypes.c_float(0.5), st))
    capi.check(lib.fbfftconv_host_sync(h))   # one wait for all three steps
    for host in steps:
        x, w, go, b = host["x"], host["w"], host["go"], host["b"]
        assert _rel(host["out"].numpy(), oracle.update_output(s, x, w, b)) <= PASS_TOL
        assert _rel(host["gi"].numpy(), oracle.update_grad_input(s, go, w)) <= PASS_TOL
        assert _rel(host["gw"].numpy(), oracle.acc_grad_weight(s, x, go, 0.5)) <= PASS_TOL
        assert _rel(host["gb"].numpy(), oracle.acc_grad_bias(s, go, 0.5)) <= PASS_TOL
    lib.fbfftconv_destroy(h)



# ---------------------------------------------------------------------------
# the benchmark's full-size layers: sampled planes against the oracle, plus
# size-independent properties
# ---------------------------------------------------------------------------
FULL_LAYERS = {
    "C2": oracle.Shape(128, 3, 96, 128, 128, 11, 11),
    "C3": oracle.Shape(128, 64, 128, 64, 64, 9, 9),
    "C4a": oracle.Shape(128, 128, 128, 32, 32, 9, 9),
    "C4b": oracle.Shape(128, 128, 128, 16, 16, 7, 7),
    "C5": oracle.Shape(128, 384, 384, 13, 13, 3, 3, 1, 1),
}


def _gen(shape, seed, kind="normal", bound=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = torch.empty(shape, device="cuda")
    return t.normal_(generator=g) if kind == "normal" else t.uniform_(-bound, bound, generator=g)


@pytest.mark.parametrize("name", list(FULL_LAYERS))
def test_full_size_layers(name):
    s = FULL_LAYERS[name]
    cfg = list(FULL_LAYERS).index(name) + 2
    bound = 1.0 / np.sqrt(s.kH * s.kW * s.P)
    x = _gen((s.B, s.P, s.iH, s.iW), 1000 * cfg)
    go = _gen((s.B, s.F, s.oH, s.oW), 1000 * cfg + 1)
    w = _gen((s.F, s.P, s.kH, s.kW), 1000 * cfg + 2, "uniform", bound)
    b = _gen((s.F,), 1000 * cfg + 3, "uniform", 0.01) if name == "C2" else torch.zeros(s.F, device="cuda")
    m = SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH)
    m.weight.copy_(w)
    m.bias.copy_(b)
    out = m.updateOutput(x)
    gi = m.updateGradInput(x, go)
    m.accGradParameters(x, go, 1.0)
    torch.cuda.synchronize()
    hx, hw, hgo, hb = x.cpu().numpy(), w.cpu().numpy(), go.cpu().numpy(), b.cpu().numpy()
    rng = np.random.default_rng(cfg)
    n = 24
    bi, fi, pi = rng.integers(0, s.B, n), rng.integers(0, s.F, n), rng.integers(0, s.P, n)
    ref = oracle.update_output_planes(s, hx, hw, hb, bi, fi)
    got = out[torch.from_numpy(bi).cuda(), torch.from_numpy(fi).cuda()].cpu().numpy()
    assert _rel(got, ref) <= PASS_TOL
    ref = oracle.update_grad_input_planes(s, hgo, hw, bi, pi)
    got = gi[torch.from_numpy(bi).cuda(), torch.from_numpy(pi).cuda()].cpu().numpy()
    assert _rel(got, ref) <= PASS_TOL
    ref = oracle.acc_grad_weight_planes(s, hx, hgo, 1.0, fi, pi)
    got = m.gradWeight[torch.from_numpy(fi).cuda(), torch.from_numpy(pi).cuda()].cpu().numpy()
    assert _rel(got, ref) <= PASS_TOL
    assert _rel(m.gradBias.cpu().numpy(), oracle.acc_grad_bias(s, hgo, 1.0)) <= PASS_TOL
    # properties that need no oracle: linearity in the input, and the adjoint identity
    # <conv(x), go> == <x, convT(go)> == <w, gradWeight> (bias removed)
    out0 = m.updateOutput(x, skipBias=True).clone()
    out2 = m.updateOutput(2.0 * x, skipBias=True)
    assert float((out2 - 2.0 * out0).abs().max()) <= 1e-4 * float(out0.abs().max())
    lhs = float((out0.double() * go.double()).sum())
    assert abs(lhs - float((x.double() * gi.double()).sum())) <= 1e-4 * abs(lhs) + 1e-3
    assert abs(lhs - float((w.double() * m.gradWeight.double()).sum())) <= 1e-4 * abs(lhs) + 1e-3
