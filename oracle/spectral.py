"""Frequency-domain restatement of the path in numpy fp64 -- TEST INFRASTRUCTURE ONLY.

Follows, in the reference checkout:
  * the transform contract of nn.FFTWrapper / fbfft (fbcunn/FFTWrapper.lua:53-132,
    src/fft/FFTWrapperLua.cpp:209-272, src/fft/FBFFTHost.cpp:39-116): a real plane of
    h x w is placed at (padU, padL) of a zero N x N square, transformed with the
    forward sign convention exp(-2 pi i ...), only the Hermitian half is kept, and
    the inverse is NOT normalised (src/fft/FFTWrapperLua.cpp:235-237);
  * the per-bin products spelled out by the single-thread spec kernels
    src/fft/CuFFTConvolution_UpdateOutput.cu:25-59, _UpdateGradInput.cu:24-59 and
    _AccGradParameters.cu:25-64, with the conjugation flags and the 1/N^2 (times
    scale) factor the Lua module passes at
    fbcunn/SpatialConvolutionFBFFT.lua:157-164, :244-251, :337-344.

The transforms are written from the DFT definition (dense DFT matrices), not through
a library FFT, so that they are an independent statement of the arithmetic.
Spectra here are complex128 arrays shaped (..., N, N//2 + 1): all ky, half of kx.
"""
from __future__ import annotations

import numpy as np


def next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def fft_size(iH, iW, kH, kW, padH, padW) -> int:
    """Square transform size the module picks: next power of two that holds the
    padded input, the kernel and the output (fbcunn/SpatialConvolutionFFT.lua:875-882,
    :947-964)."""
    oH, oW = iH + 2 * padH - kH + 1, iW + 2 * padW - kW + 1
    return next_pow2(max(iH + 2 * padH, iW + 2 * padW, kH, kW, oH, oW))


def _dft_matrix(rows: int, n: int, sign: float) -> np.ndarray:
    k = np.arange(rows)[:, None]
    j = np.arange(n)[None, :]
    return np.exp(sign * 2j * np.pi * ((k * j) % n) / n)


def rfft2_padded(x: np.ndarray, rows: int, cols: int | None = None, pad_u: int = 0, pad_l: int = 0) -> np.ndarray:
    """Forward 2-D real-to-complex DFT of x[..., h, w] zero-extended to rows x cols
    with its origin at (pad_u, pad_l).  Returns (..., rows, cols//2 + 1)."""
    cols = rows if cols is None else cols
    x = np.asarray(x, dtype=np.float64)
    h, w = x.shape[-2:]
    assert pad_u + h <= rows and pad_l + w <= cols
    # sum_y sum_x x[y,x] e^{-2pi i ky (y+pad_u)/rows} e^{-2pi i kx (x+pad_l)/cols}
    fy = _dft_matrix(rows, rows, -1.0)[:, pad_u:pad_u + h]            # (ky, y)
    fx = _dft_matrix(cols // 2 + 1, cols, -1.0)[:, pad_l:pad_l + w]   # (kx, x)
    return np.einsum("ky,...yx,lx->...kl", fy, x, fx, optimize=True)


def irfft2_unnormalised(spec: np.ndarray, rows: int, cols: int | None = None) -> np.ndarray:
    """Un-normalised inverse of rfft2_padded: returns the real (..., rows, cols) array
    sum_{ky,kx} S[ky,kx] e^{+2 pi i (...)} with the missing half restored by
    Hermitian symmetry.  irfft2(rfft2(x)) == rows*cols*x."""
    cols = rows if cols is None else cols
    spec = np.asarray(spec, dtype=np.complex128)
    half = cols // 2 + 1
    assert spec.shape[-2:] == (rows, half)
    full = np.zeros(spec.shape[:-1] + (cols,), np.complex128)
    full[..., :half] = spec
    for kx in range(half, cols):
        src = spec[..., (-np.arange(rows)) % rows, cols - kx]
        full[..., kx] = np.conj(src)
    gy = _dft_matrix(rows, rows, +1.0)   # (y, ky)
    gx = _dft_matrix(cols, cols, +1.0)   # (x, kx)
    out = np.einsum("yk,...kl,xl->...yx", gy, full, gx, optimize=True)
    return out.real


def contract_update_output(i_hat, w_hat, norm):
    """O[b,f] = norm * sum_p I[b,p] conj(W[f,p])  (spec kernel _UpdateOutput.cu:25-59)."""
    return norm * np.einsum("bp...,fp...->bf...", i_hat, np.conj(w_hat), optimize=True)


def contract_update_grad_input(o_hat, w_hat, norm):
    """I'[b,p] = norm * sum_f O'[b,f] W[f,p]  (spec kernel _UpdateGradInput.cu:24-59)."""
    return norm * np.einsum("bf...,fp...->bp...", o_hat, w_hat, optimize=True)


def contract_acc_grad_parameters(o_hat, i_hat, norm):
    """W'[f,p] = norm * sum_b conj(O'[b,f]) I[b,p]  (spec kernel _AccGradParameters.cu:25-64)."""
    return norm * np.einsum("bf...,bp...->fp...", np.conj(o_hat), i_hat, optimize=True)


def update_output(x, weight, bias, padH, padW):
    """The module's forward pass carried out in the frequency domain (fp64)."""
    B, P, iH, iW = x.shape
    F, _, kH, kW = weight.shape
    N = fft_size(iH, iW, kH, kW, padH, padW)
    oH, oW = iH + 2 * padH - kH + 1, iW + 2 * padW - kW + 1
    i_hat = rfft2_padded(x, N, N, padH, padW)
    w_hat = rfft2_padded(weight, N)
    o_hat = contract_update_output(i_hat, w_hat, 1.0 / (N * N))
    out = irfft2_unnormalised(o_hat, N)[..., :oH, :oW]
    if bias is not None:
        out = out + np.asarray(bias, np.float64)[None, :, None, None]
    return out


def update_grad_input(grad_output, weight, iH, iW, padH, padW):
    F, P, kH, kW = weight.shape
    N = fft_size(iH, iW, kH, kW, padH, padW)
    o_hat = rfft2_padded(grad_output, N)
    w_hat = rfft2_padded(weight, N)
    i_hat = contract_update_grad_input(o_hat, w_hat, 1.0 / (N * N))
    return irfft2_unnormalised(i_hat, N)[..., padH:padH + iH, padW:padW + iW]


def acc_grad_weight(x, grad_output, kH, kW, padH, padW, scale=1.0):
    B, P, iH, iW = x.shape
    N = fft_size(iH, iW, kH, kW, padH, padW)
    i_hat = rfft2_padded(x, N, N, padH, padW)
    o_hat = rfft2_padded(grad_output, N)
    w_hat = contract_acc_grad_parameters(o_hat, i_hat, scale / (N * N))
    return irfft2_unnormalised(w_hat, N)[..., :kH, :kW]
