"""CPU-side checks of the boundary: the C-ABI library loads, exports every symbol the
header declares, validates its arguments without touching a GPU, and refuses to
compute without one (no fallback)."""
import ctypes
import os
import re

import pytest

from fbcunn_b200 import build as fb_build
from fbcunn_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    fb_build.build()
    return capi.lib()


def _declared():
    with open(os.path.join(ROOT, "include", "fbfftconv.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbfftconv_[a-z0-9_]+)\s*\(", text)))


def test_exports_match_header(lib):
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fbfftconv.h but not exported"
    assert sorted(capi.EXPORTS) == names


def _desc(**kw):
    base = dict(batch=2, n_input_plane=3, n_output_plane=4, input_h=8, input_w=8, kernel_h=3,
                kernel_w=3, stride_h=1, stride_w=1, pad_h=0, pad_w=0, device=0, flags=0)
    base.update(kw)
    return capi.Desc(**base)


def _create(lib, **kw):
    h = ctypes.c_void_p()
    rc = lib.fbfftconv_create(ctypes.byref(_desc(**kw)), ctypes.byref(h))
    return rc, h


def test_create_validates_like_the_lua_constructor(lib):
    rc, h = _create(lib)
    assert rc == capi.OK and h.value
    assert lib.fbfftconv_fft_size(h) == 8
    assert lib.fbfftconv_workspace_bytes(h) > 0
    assert lib.fbfftconv_destroy(h) == capi.OK
    # stride must be 1 (fbcunn/SpatialConvolutionFBFFT.lua:60-61)
    rc, _ = _create(lib, stride_w=2)
    assert rc == capi.ERR_INVALID_ARGUMENT and "stride" in capi.last_error()
    # padding smaller than the kernel (fbcunn/SpatialConvolutionFBFFT.lua:93-95)
    rc, _ = _create(lib, pad_h=3)
    assert rc == capi.ERR_INVALID_ARGUMENT and "padding" in capi.last_error()
    rc, _ = _create(lib, kernel_h=9, kernel_w=9)
    assert rc == capi.ERR_INVALID_ARGUMENT
    rc, _ = _create(lib, batch=0)
    assert rc == capi.ERR_INVALID_ARGUMENT
    # transforms above 128 are not supported (src/fft/FBFFTHost.cpp:96-98)
    rc, _ = _create(lib, input_h=129, input_w=10)
    assert rc == capi.ERR_UNSUPPORTED_SIZE
    assert lib.fbfftconv_create(None, None) == capi.ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("shape,n", [((32, 32, 5, 5, 0), 32), ((128, 128, 11, 11, 0), 128),
                                     ((64, 64, 9, 9, 0), 64), ((16, 16, 7, 7, 0), 16),
                                     ((13, 13, 3, 3, 1), 16), ((3, 3, 3, 3, 0), 8), ((30, 33, 3, 3, 0), 64)])
def test_fft_size_rule(lib, shape, n):
    """Next power of two holding the padded input (fbcunn/SpatialConvolutionFFT.lua:875-882)."""
    ih, iw, kh, kw, pad = shape
    rc, h = _create(lib, input_h=ih, input_w=iw, kernel_h=kh, kernel_w=kw, pad_h=pad, pad_w=pad)
    assert rc == capi.OK
    assert lib.fbfftconv_fft_size(h) == n
    lib.fbfftconv_destroy(h)


def test_workspace_accounting(lib):
    rc, h = _create(lib, batch=128, n_input_plane=384, n_output_plane=384, input_h=13, input_w=13,
                    kernel_h=3, kernel_w=3, pad_h=1, pad_w=1)
    assert rc == capi.OK
    bins = 9 * 16
    expect = bins * 8 * (128 * 384 + 128 * 384 + 384 * 384)
    got = lib.fbfftconv_workspace_bytes(h)
    # three spectra, the bias partial sums (B*F + F floats), the weight and bias gradient in the spatial
    # domain for the sums across ranks, once as each rank's contribution and once as the delivered sum
    # (2 x (F*P*kH*kW + F) floats, + F behind the spectrum), and alignment
    small = (128 * 384 + 384) * 4 + 2 * (384 * 384 * 9 + 2 * 384) * 4
    assert expect <= got <= expect + small + 8 * 256
    assert lib.fbfftconv_spectrum_bytes(16, 128, 384) == bins * 128 * 384 * 8
    assert lib.fbfftconv_spectrum_bytes(16, 128, 3) == bins * 128 * 4 * 8
    assert lib.fbfftconv_spectrum_bytes(12, 1, 1) == 0
    assert lib.fbfftconv_set_workspace(h, None, 0) == capi.ERR_INVALID_ARGUMENT
    lib.fbfftconv_destroy(h)


def test_substeps_reject_bad_arguments(lib):
    assert lib.fbfftconv_fft2d(None, None, 1, 1, 4, 4, 8, 0, 0, 0, None) == capi.ERR_INVALID_ARGUMENT
    one = ctypes.c_void_p(16)
    assert lib.fbfftconv_fft2d(one, one, 1, 1, 4, 4, 12, 0, 0, 0, None) == capi.ERR_UNSUPPORTED_SIZE
    assert lib.fbfftconv_fft2d(one, one, 1, 1, 9, 4, 8, 0, 0, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_ifft2d(one, one, None, 1, 1, 4, 4, 8, 5, 0, 0, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_transpose_mm(one, one, one, 0, 1, 1, 1, 1.0, 0, 0, 0, None) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_status_string(capi.ERR_NOMEM) == b"out of device memory"


def test_no_fallback_without_a_gpu(lib):
    """The product path must fail loudly where CUDA is missing, never compute elsewhere."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    rc, h = _create(lib)
    assert rc == capi.OK
    buf = (ctypes.c_float * 4096)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    rc = lib.fbfftconv_update_output(h, p, p, None, p, None)
    assert rc in (capi.ERR_CUDA, capi.ERR_NOMEM)
    assert capi.last_error()
    lib.fbfftconv_destroy(h)
