"""Tile geometry of the native tiled passes on the CPU (creating a tiled handle touches no GPU):
the tiles the library will cut must cover the output exactly once and the padded input completely,
and the untiled layer of the tiles must have the tile's transform size.  The kernels that cut,
assemble and overlap-add are checked on the GPU against the oracle (tests/test_gpu_tiled.py)."""
import ctypes

import pytest

from fbcunn_b200 import build as fb_build
from fbcunn_b200 import capi


@pytest.fixture(scope="module")
def lib():
    fb_build.build()
    return capi.lib()


def _tiled(lib, B, P, Fo, iH, iW, kH, kW, padH, padW, tH, tW):
    desc = capi.Desc(B, P, Fo, iH, iW, kH, kW, 1, 1, padH, padW, 0, 0)
    t = ctypes.c_void_p()
    rc = lib.fbfftconv_tiled_create(ctypes.byref(desc), tH, tW, ctypes.byref(t))
    return rc, t


@pytest.mark.parametrize("case", [
    (2, 3, 4, 70, 61, 5, 4, 2, 1, 16, 16),
    (1, 2, 2, 33, 40, 3, 3, 0, 0, 8, 8),
    (1, 1, 2, 150, 140, 3, 3, 1, 1, 32, 32),     # beyond the 128-pixel limit of the untiled layer
    (2, 2, 2, 12, 12, 3, 3, 0, 0, 16, 16),        # tile larger than the image: one tile
    (1, 2, 1, 20, 31, 7, 2, 3, 1, 16, 32),
    (1, 1, 1, 20, 20, 7, 7, 0, 0, 8, 8),          # a tile reaches beyond its neighbour (step 2, extent 8)
    (32, 64, 64, 224, 224, 3, 3, 1, 1, 16, 16),
])
def test_tiles_cover_the_layer(lib, case):
    B, P, Fo, iH, iW, kH, kW, padH, padW, tH, tW = case
    rc, t = _tiled(lib, *case)
    assert rc == capi.OK, capi.last_error()
    geo = (ctypes.c_int32 * 6)()
    assert lib.fbfftconv_tiled_geometry(t, geo) == capi.OK
    th, tw, sh, sw, nh, nw = list(geo)
    oH, oW = iH + 2 * padH - kH + 1, iW + 2 * padW - kW + 1
    assert th == min(tH, iH + 2 * padH) and tw == min(tW, iW + 2 * padW)
    assert sh == th - kH + 1 and sw == tw - kW + 1 and sh >= 1 and sw >= 1
    # disjoint output tiles cover the output, the last one possibly hanging over
    assert (nh - 1) * sh < oH <= nh * sh and (nw - 1) * sw < oW <= nw * sw
    # the overlapping input tiles cover the padded input
    assert (nh - 1) * sh + th >= iH + 2 * padH and (nw - 1) * sw + tw >= iW + 2 * padW
    # every padded input pixel is covered by at most ceil(th/sh) * ceil(tw/sw) tiles, at least one
    for extent, tile, step, n in ((iH + 2 * padH, th, sh, nh), (iW + 2 * padW, tw, sw, nw)):
        for pos in range(extent):
            covering = [i for i in range(n) if i * step <= pos < i * step + tile]
            assert 1 <= len(covering) <= -(-tile // step)
    # the untiled layer of the tiles: batch * tiles images, transform size of the tile
    inner = ctypes.c_void_p(lib.fbfftconv_tiled_inner(t))
    n_fft = lib.fbfftconv_fft_size(inner)
    need = max(th, tw)
    assert n_fft >= need and (n_fft == 8 or n_fft // 2 < need)
    assert lib.fbfftconv_tiled_destroy(t) == capi.OK


def test_tiled_create_validates(lib):
    # tile size must exceed the kernel size minus one (fbcunn/SpatialConvolutionFFTTiled.lua:300-303)
    rc, _ = _tiled(lib, 1, 1, 1, 20, 20, 7, 7, 0, 0, 6, 8)
    assert rc == capi.ERR_INVALID_ARGUMENT and "tile size" in capi.last_error()
    rc, _ = _tiled(lib, 1, 1, 1, 20, 20, 3, 3, 3, 0, 8, 8)
    assert rc == capi.ERR_INVALID_ARGUMENT and "padding" in capi.last_error()
    # too many tiles for one untiled pass
    rc, _ = _tiled(lib, 128, 1, 1, 512, 512, 3, 3, 1, 1, 8, 8)
    assert rc == capi.ERR_INVALID_ARGUMENT and "65535" in capi.last_error()
    # tiles of 256 pixels would need a 256-point transform
    rc, _ = _tiled(lib, 1, 1, 1, 300, 300, 3, 3, 1, 1, 256, 256)
    assert rc == capi.ERR_UNSUPPORTED_SIZE
    # without a CUDA device the passes refuse to compute (no fallback)
    import torch
    if not torch.cuda.is_available():
        rc, t = _tiled(lib, 1, 1, 1, 20, 20, 3, 3, 1, 1, 8, 8)
        assert rc == capi.OK
        one = ctypes.c_void_p(256)
        assert lib.fbfftconv_tiled_update_output(t, one, one, None, one, None) == capi.ERR_CUDA
        lib.fbfftconv_tiled_destroy(t)
