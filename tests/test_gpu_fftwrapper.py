"""nn.FFTWrapper with the reference's tensor contract (fbcunn/FFTWrapper.lua:53-132,
test/test_FFTModule.lua:310-355): 1-D and 2-D transforms, one or two batch dimensions,
frequency tensors shaped like the reference's.  Yardstick: numpy's fp64 FFT; tolerance
5e-6 * max|spectrum| forward (the reference allows 4e-7 * max against cuFFT in fp32,
test/test_FFTModule.lua:13), and the same relative bound on the un-normalised inverse."""
import numpy as np
import pytest
import torch

from fbcunn_b200 import FFTWrapper

pytestmark = pytest.mark.gpu
TOL = 5e-6


def _complex(t):
    a = t.cpu().numpy().astype(np.float64)
    return a[..., 0] + 1j * a[..., 1]


# the sizes of the reference's own test list (test/test_FFTModule.lua:170-260)
SIZES = [2, 4, 8, 16, 32, 64, 128]


# 256 points exist for the 1-D transform only, as in the reference's list
@pytest.mark.parametrize("n", SIZES + [256])
@pytest.mark.parametrize("batch", [(1,), (4,), (3, 5), (127,), (437,), (1000,)])
def test_1d(n, batch):
    rng = np.random.default_rng(n + len(batch))
    x = rng.standard_normal(batch + (n,)).astype(np.float32)
    time = torch.from_numpy(x).cuda()
    freq = torch.full(batch + (n // 2 + 1, 2), float("nan"), device="cuda")
    w = FFTWrapper("fbfft", 0, 0)
    w.fft_reference_layout(time, freq, len(batch))
    ref = np.fft.rfft(x.astype(np.float64), axis=-1)
    assert np.abs(_complex(freq) - ref).max() <= TOL * np.abs(ref).max()
    back = torch.full_like(time, float("nan"))
    w.ffti_reference_layout(back, freq, len(batch))
    assert np.abs(back.cpu().numpy() / n - x).max() <= TOL * n * np.abs(x).max()


@pytest.mark.parametrize("n,rows,width,pad", [(32, 70, 20, 5), (256, 33, 200, 17), (256, 64, 129, 127)])
def test_1d_short_rows_are_zero_padded(n, rows, width, pad):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((rows, width)).astype(np.float32)
    freq = torch.empty((rows, n // 2 + 1, 2), device="cuda")
    FFTWrapper("fbfft", pad, 0).fft_reference_layout(torch.from_numpy(x).cuda(), freq, 1)
    padded = np.zeros((rows, n))
    padded[:, pad:pad + width] = x
    ref = np.fft.rfft(padded, axis=-1)
    assert np.abs(_complex(freq) - ref).max() <= TOL * np.abs(ref).max()


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("batch", [(1,), (3,), (9,), (2, 3), (128,)])
def test_2d_reference_layout(n, batch):
    rng = np.random.default_rng(10 * n + len(batch))
    x = rng.standard_normal(batch + (n, n)).astype(np.float32)
    time = torch.from_numpy(x).cuda()
    freq = torch.full(batch + (n // 2 + 1, n, 2), float("nan"), device="cuda")
    w = FFTWrapper("fbfft", 0, 0)
    w.fft_reference_layout(time, freq, len(batch))
    full = np.fft.fft2(x.astype(np.float64), axes=(-2, -1))          # [ky][kx]
    if 8 <= n <= 32:
        ref = full[..., :n // 2 + 1, :]                               # half along the first FFT dim
    else:
        ref = np.swapaxes(full[..., :, :n // 2 + 1], -1, -2)          # half along the second, transposed
    assert np.abs(_complex(freq) - ref).max() <= TOL * np.abs(ref).max()
    back = torch.full_like(time, float("nan"))
    w.ffti_reference_layout(back, freq, len(batch))
    assert np.abs(back.cpu().numpy() / (n * n) - x).max() <= TOL * n * np.abs(x).max()
