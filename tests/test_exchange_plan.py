"""CPU checks of how accGradParameters cuts the weight-gradient sum into per-rank shares.

fbfftconv_exchange_plan reports the arithmetic the pass itself uses (which sum, this rank's share of
the spectrum, what is cleared before the inverse transform, this rank's filters in gradWeight).  Here:
the choice of sum for divisible and non-divisible rank counts, that the shares of all ranks tile the
spectrum in whole 16-byte units, and -- by replaying the steps on numpy arrays with a linear map in the
transform's place -- that share-wise sum, clearing, transform and final sum give the transform of the
total.  The reference's counterpart is the gather / add / broadcast of nn.DataParallel
(fbcunn/DataParallel.lua:105-131), whose result the multi-GPU test checks on hardware.
"""
import ctypes

import numpy as np
import pytest

from fbcunn_b200 import build as fb_build
from fbcunn_b200 import capi

SUM_NONE, BY_FILTERS, BY_BINS, WHOLE, SPATIAL = 0, 1, 2, 3, 4
ALLREDUCE_SPATIAL = 8

# (batch, P, F, h, w, k, pad): a thin plane-major layer (transform 128), its 64-point sibling, the
# bin-major 16-point layer of the benchmark, a 32-point layer (544 bins) and an 8-point one (40 bins)
SHAPES = {
    "thin128": (8, 3, 96, 128, 128, 11, 0),
    "thin64": (4, 2, 12, 60, 60, 5, 0),
    "deep16": (16, 384, 384, 13, 13, 3, 1),
    "mid32": (8, 20, 24, 27, 27, 5, 2),
    "small8": (2, 5, 6, 6, 6, 3, 0),
}


@pytest.fixture(scope="module")
def lib():
    fb_build.build()
    return capi.lib()


def _handle(lib, shape, flags=0):
    b, p, f, h, w, k, pad = SHAPES[shape]
    desc = capi.Desc(batch=b, n_input_plane=p, n_output_plane=f, input_h=h, input_w=w, kernel_h=k, kernel_w=k,
                     stride_h=1, stride_w=1, pad_h=pad, pad_w=pad, device=0, flags=flags)
    out = ctypes.c_void_p()
    assert lib.fbfftconv_create(ctypes.byref(desc), ctypes.byref(out)) == capi.OK
    return out


def _plan(lib, h, rank, nranks):
    out = (ctypes.c_longlong * 10)()
    assert lib.fbfftconv_exchange_plan(h, rank, nranks, out) == capi.OK, capi.last_error()
    keys = ("mode", "spec", "chunk", "first", "zero_before", "zero_after", "n_weight", "slice", "slice_first", "vec4")
    return dict(zip(keys, list(out)))


def _expected_mode(shape, nranks, n):
    _, p, f, _, _, _, _ = SHAPES[shape]
    bins = (n // 2 + 1) * n
    plane_major = p <= 4 and n >= 64
    if nranks == 0:
        return SUM_NONE
    if plane_major:
        return BY_FILTERS if f % nranks == 0 else WHOLE
    return BY_BINS if nranks > 1 and bins % nranks == 0 else WHOLE


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_choice_of_sum_and_tiling_of_the_shares(lib, shape):
    h = _handle(lib, shape)
    n = lib.fbfftconv_fft_size(h)
    _, p, f, _, _, k, _ = SHAPES[shape]
    for nranks in range(0, 9):
        plans = [_plan(lib, h, r, nranks) for r in range(max(nranks, 1))]
        for x in plans:
            assert x["mode"] == _expected_mode(shape, nranks, n), (shape, nranks, x)
            assert x["n_weight"] == f * p * k * k
            assert 4 * x["vec4"] >= x["n_weight"] + f > 4 * (x["vec4"] - 1)
            assert x["spec"] % 4 == 0 and x["spec"] == plans[0]["spec"]
        mode = plans[0]["mode"]
        if mode in (BY_FILTERS, BY_BINS):
            # the shares tile the spectrum, in rank order, in whole 16-byte units
            assert [x["first"] for x in plans] == [r * plans[0]["chunk"] for r in range(nranks)]
            assert sum(x["chunk"] for x in plans) == plans[0]["spec"]
            for x in plans:
                assert x["chunk"] % 4 == 0 and x["first"] % 4 == 0 and x["chunk"] > 0
        if mode == BY_BINS:
            for x in plans:
                assert x["zero_before"] == x["first"]
                assert x["zero_before"] + x["chunk"] + x["zero_after"] == x["spec"]
                assert x["slice"] == 0
        elif mode == BY_FILTERS:
            assert [x["slice_first"] for x in plans] == [r * plans[0]["slice"] for r in range(nranks)]
            assert sum(x["slice"] for x in plans) == plans[0]["n_weight"]
            for x in plans:
                assert x["zero_before"] == 0 and x["zero_after"] == 0
                # a share holds whole filters: spectrum floats per filter x filters per rank
                assert x["chunk"] * f == x["spec"] * (f // nranks)
        else:
            for x in plans:
                assert x["chunk"] == 0 and x["slice"] == 0 and x["zero_before"] == 0 and x["zero_after"] == 0
    lib.fbfftconv_destroy(h)


def test_ranks_that_divide_neither_filters_nor_bins_sum_the_whole_spectrum(lib):
    # 96 filters / 5 or 7 ranks, 144 bins / 5 or 7 ranks, 544 bins / 3 ranks
    for shape, nranks in (("thin128", 5), ("thin128", 7), ("deep16", 5), ("deep16", 7), ("mid32", 3)):
        h = _handle(lib, shape)
        assert _plan(lib, h, nranks - 1, nranks)["mode"] == WHOLE
        lib.fbfftconv_destroy(h)
    # ... and ranks that do divide them take shares: 96 / 3, 144 / 3, 544 / 8
    for shape, nranks, mode in (("thin128", 3, BY_FILTERS), ("deep16", 3, BY_BINS), ("mid32", 8, BY_BINS)):
        h = _handle(lib, shape)
        assert _plan(lib, h, 0, nranks)["mode"] == mode
        lib.fbfftconv_destroy(h)


def test_spatial_flag_and_argument_checks(lib):
    h = _handle(lib, "deep16", flags=ALLREDUCE_SPATIAL)
    assert _plan(lib, h, 1, 4)["mode"] == SPATIAL
    assert _plan(lib, h, 0, 0)["mode"] == SUM_NONE  # no communicator: the flag has nothing to act on
    out = (ctypes.c_longlong * 10)()
    assert lib.fbfftconv_exchange_plan(h, 4, 4, out) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_exchange_plan(h, -1, 2, out) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_exchange_plan(None, 0, 1, out) == capi.ERR_INVALID_ARGUMENT
    assert lib.fbfftconv_exchange_plan(h, 0, 1, None) == capi.ERR_INVALID_ARGUMENT
    lib.fbfftconv_destroy(h)


@pytest.mark.parametrize("shape,nranks", [("small8", 2), ("small8", 4), ("small8", 5), ("small8", 8),
                                          ("thin64", 2), ("thin64", 3), ("thin64", 4), ("thin64", 6)])
def test_replay_of_the_steps_gives_the_transform_of_the_total(lib, shape, nranks):
    """Each rank holds a partial spectrum; a fixed linear map stands for the inverse transform.  The
    steps of the pass, replayed with the plan's offsets: share-wise sum in rank order, clearing of
    the other ranks' bins (by bins) or transform of the own filters into their slice (by filters),
    then the sum / gather of the spatial vectors.  Every rank must end with map(sum of spectra)."""
    h = _handle(lib, shape)
    plans = [_plan(lib, h, r, nranks) for r in range(nranks)]
    mode, spec, n_weight = plans[0]["mode"], plans[0]["spec"], plans[0]["n_weight"]
    rng = np.random.default_rng(17 + nranks)
    partial = [rng.standard_normal(spec) for _ in range(nranks)]
    total = np.sum(partial, axis=0)
    _, p, f, _, _, k, _ = SHAPES[shape]
    if mode == BY_FILTERS:
        # plane-major: the transform acts filter by filter ([f][rest] -> [f][p*k*k])
        per_f_in, per_f_out = spec // f, n_weight // f
        m = rng.standard_normal((per_f_out, per_f_in))
        transform = lambda s: (s.reshape(-1, per_f_in) @ m.T).reshape(-1)
        want = transform(total)
        vec = [np.zeros(n_weight) for _ in range(nranks)]
        for r, x in enumerate(plans):
            share = slice(x["first"], x["first"] + x["chunk"])
            summed = np.sum([partial[q][share] for q in range(nranks)], axis=0)
            vec[r][x["slice_first"]:x["slice_first"] + x["slice"]] = transform(summed)
        got = np.sum(vec, axis=0)  # the other ranks' slices are zero: the sum is a gather
    elif mode == BY_BINS:
        m = rng.standard_normal((n_weight, spec)) / np.sqrt(spec)
        want = m @ total
        vec = []
        for r, x in enumerate(plans):
            work = partial[r].copy()
            share = slice(x["first"], x["first"] + x["chunk"])
            work[share] = np.sum([partial[q][share] for q in range(nranks)], axis=0)
            work[:x["zero_before"]] = 0.0
            if x["zero_after"]:
                work[x["first"] + x["chunk"]:x["first"] + x["chunk"] + x["zero_after"]] = 0.0
            vec.append(m @ work)
        got = np.sum(vec, axis=0)
    else:
        assert mode == WHOLE
        m = rng.standard_normal((n_weight, spec)) / np.sqrt(spec)
        want = m @ total
        got = m @ np.sum(partial, axis=0)
    np.testing.assert_allclose(got, want, rtol=1e-10, atol=1e-10)
    lib.fbfftconv_destroy(h)
