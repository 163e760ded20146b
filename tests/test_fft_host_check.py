"""Runs the FFT kernels' phase functions on the host (threads as loops, shared memory
pre-filled with NaN) and checks them against the DFT restatement of the oracle: the
index arithmetic of every size / tile combination is verified without a GPU."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from oracle import spectral

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "host_check", "fft_host_check.cpp")
LIB = os.path.join(ROOT, "tests", "host_check", "libfft_host_check.so")
CORE = os.path.join(ROOT, "fbcunn_b200", "csrc", "fft_core.cuh")
LL = ctypes.c_longlong


@pytest.fixture(scope="module")
def hc():
    newest = max(os.path.getmtime(SRC), os.path.getmtime(CORE))
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-o", LIB, SRC])
    return ctypes.CDLL(LIB)


def _bin_major(spec_plane_major):
    """(d1, d2, ky, kx) -> (ky*(N/2+1)+kx, d1, d2)."""
    d1, d2, n, half = spec_plane_major.shape
    return spec_plane_major.transpose(2, 3, 0, 1).reshape(half * n, d1, d2)


CASES = [(N, T) for N in (2, 4, 8, 16, 32, 64, 128) for T in (1, 2, 4, 8, 16)
         if (T <= (8 if N == 64 else 2) if N > 32 else (N // 2 + 1) * T <= 512)]


@pytest.mark.parametrize("N,T", CASES)
def test_forward(hc, N, T):
    rng = np.random.default_rng(N * 100 + T)
    ran = 0
    for (h, w, pu, pl) in [(N, N, 0, 0), (3, 3, 0, 0), (N - 3, N - 5, 1, 2), (1, 1, 0, 0), (N - 1, N - 1, 1, 0)]:
        if h < 1 or w < 1 or h + pu > N or w + pl > N:
            continue  # the two smallest sizes cannot hold every window
        if hc.hostcheck_forward_smem_bytes(N, T, h, w, pu, pl) > 227 * 1024:
            continue
        assert hc.hostcheck_forward_threads(N, T, h, w, pu, pl) > 0
        ran += 1
        for transposed in (False, True):
            d1, d2 = (2, 5) if not transposed else (5, 2)
            x = rng.standard_normal((d1, d2, h, w)).astype(np.float32)
            rows, inner = (d2, d1) if transposed else (d1, d2)
            rs, is_ = (1, d2) if transposed else (d2, 1)
            kc = (inner + 3) // 4 * 4
            spec = np.full(((N // 2 + 1) * N, rows, kc, 2), np.nan, np.float32)
            rc = hc.hostcheck_fft_forward(x.ctypes.data_as(ctypes.c_void_p), spec.ctypes.data_as(ctypes.c_void_p),
                                          N, T, h, w, pu, pl, rows, inner, kc, LL(rs), LL(is_), 0)
            assert rc == 0
            ref = _bin_major(spectral.rfft2_padded(x, N, N, pu, pl))
            if transposed:
                ref = ref.transpose(0, 2, 1)
            got = spec[..., 0] + 1j * spec[..., 1]
            assert np.abs(got[:, :, :inner] - ref).max() <= 3e-6 * np.abs(ref).max()
            assert np.all(got[:, :, inner:] == 0), "padding planes must be written as zero"
    assert ran > 0


@pytest.mark.parametrize("N,T", CASES)
def test_inverse(hc, N, T):
    rng = np.random.default_rng(N * 100 + T + 7)
    for (oh, ow, oy, ox) in [(N, N, 0, 0), (3, 3, 0, 0), (N - 3, N - 5, 1, 2), (N - 4, N - 4, 0, 0), (1, 1, 2, 3),
                             (N - 1, N - 1, 1, 0), (1, 1, 1, 1)]:
        if oh < 1 or ow < 1 or oh + oy > N or ow + ox > N:
            continue
        if hc.hostcheck_inverse_smem_bytes(N, T, oh, ow) > 227 * 1024:
            continue
        assert hc.hostcheck_inverse_threads(N, T, oh, ow) > 0
        rows, inner, kc = 2, 5, 8
        full = rng.standard_normal((rows, inner, N, N))
        sb = _bin_major(np.fft.rfft2(full))
        spec = np.full(((N // 2 + 1) * N, rows, kc, 2), np.nan, np.float32)  # padding must not be read
        spec[:, :, :inner, 0] = sb.real
        spec[:, :, :inner, 1] = sb.imag
        bias = rng.standard_normal(inner).astype(np.float32)
        out = np.full((rows, inner, oh, ow), np.nan, np.float32)
        rc = hc.hostcheck_fft_inverse(spec.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                      bias.ctypes.data_as(ctypes.c_void_p), N, T, oh, ow, oy, ox, rows, inner, kc,
                                      LL(inner), LL(1), 0, 0)
        assert rc == 0
        # un-normalised inverse (src/fft/FFTWrapperLua.cpp:235-237), cropped, bias added
        ref = spectral.irfft2_unnormalised(np.fft.rfft2(full), N)[:, :, oy:oy + oh, ox:ox + ow] + bias[None, :, None, None]
        assert np.abs(out - ref).max() <= 3e-6 * np.abs(ref).max()
        init = rng.standard_normal((rows, inner, oh, ow)).astype(np.float32)
        acc = init.copy()
        hc.hostcheck_fft_inverse(spec.ctypes.data_as(ctypes.c_void_p), acc.ctypes.data_as(ctypes.c_void_p), None,
                                 N, T, oh, ow, oy, ox, rows, inner, kc, LL(inner), LL(1), 1, 0)
        assert np.abs(acc - (ref - bias[None, :, None, None] + init)).max() <= 3e-6 * np.abs(ref).max()


@pytest.mark.parametrize("N,T", [(64, 1), (64, 4), (128, 1), (16, 1), (32, 2)])
def test_plane_major_layout(hc, N, T):
    """Spectrum stored [row][inner][bin] (bins contiguous): forward then inverse."""
    rng = np.random.default_rng(N + T)
    d1, d2, h, w, pu, pl = 3, 5, N - 6, N - 9, 1, 2
    x = rng.standard_normal((d1, d2, h, w)).astype(np.float32)
    bins = (N // 2 + 1) * N
    spec = np.full((d1, d2, bins, 2), np.nan, np.float32)
    rc = hc.hostcheck_fft_forward(x.ctypes.data_as(ctypes.c_void_p), spec.ctypes.data_as(ctypes.c_void_p),
                                  N, T, h, w, pu, pl, d1, d2, d2, LL(d2), LL(1), 1)
    assert rc == 0
    ref = spectral.rfft2_padded(x, N, N, pu, pl).reshape(d1, d2, bins)   # bin = ky*(N/2+1) + kx
    got = spec[..., 0] + 1j * spec[..., 1]
    assert np.abs(got - ref).max() <= 3e-6 * np.abs(ref).max()
    out = np.full((d1, d2, h, w), np.nan, np.float32)
    rc = hc.hostcheck_fft_inverse(spec.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), None,
                                  N, T, h, w, pu, pl, d1, d2, d2, LL(d2), LL(1), 0, 1)
    assert rc == 0
    assert np.abs(out / (N * N) - x).max() <= 5e-6 * np.abs(x).max()


# (sizes above 32 have kernels of their own, which only the GPU tests reach)
@pytest.mark.parametrize("N,T", [(2, 16), (4, 16), (4, 2), (8, 16), (16, 4), (32, 16), (32, 2)])
def test_1d_transforms(hc, N, T):
    """The batched 1-D kernels (row phases + plain store / load of the column buffer) against numpy."""
    rng = np.random.default_rng(N + T)
    for (h, n, off, planes) in [(N, N, 0, 3), (5, N - 3, 2, 2), (1, 1, 0, 1), (N, 7, 0, 5), (N, N - 1, 1, 4)]:
        if h > N or n < 1 or n + off > N:
            continue
        if hc.hostcheck_forward_smem_bytes(N, T, h, n, 0, off) > 227 * 1024:
            continue
        x = rng.standard_normal((planes * h, n)).astype(np.float32)
        spec = np.full((planes * h, N // 2 + 1, 2), np.nan, np.float32)
        assert hc.hostcheck_fft1d(0, x.ctypes.data_as(ctypes.c_void_p), spec.ctypes.data_as(ctypes.c_void_p),
                                  N, T, h, n, off, planes) == 0
        padded = np.zeros((planes * h, N))
        padded[:, off:off + n] = x
        ref = np.fft.rfft(padded, axis=1)
        got = spec[..., 0] + 1j * spec[..., 1]
        assert np.abs(got - ref).max() <= 3e-6 * max(np.abs(ref).max(), 1.0)
        # inverse: un-normalised, cropped to [off, off + n)
        full = rng.standard_normal((planes * h, N))
        sp = np.fft.rfft(full, axis=1)
        spec2 = np.stack([sp.real, sp.imag], axis=-1).astype(np.float32)
        out = np.full((planes * h, n), np.nan, np.float32)
        assert hc.hostcheck_fft1d(1, out.ctypes.data_as(ctypes.c_void_p), spec2.ctypes.data_as(ctypes.c_void_p),
                                  N, T, h, n, off, planes) == 0
        ref_t = N * full[:, off:off + n]
        assert np.abs(out - ref_t).max() <= 3e-6 * np.abs(ref_t).max() * N
