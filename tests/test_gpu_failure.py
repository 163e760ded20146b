"""Failure paths on the GPU that need no fault: a bounded device wait that runs out on
purpose, and pointers the boundary must refuse before anything is launched.

The tensor-core contraction bounds every wait on an mbarrier; fbfftconv_tensor_core_wait_selftest
runs that same wait on a barrier nothing completes (limit: a few microseconds).  The kernel
returns normally, the sticky code is what the host reads, and the context stays usable.
"""
import ctypes

import numpy as np
import pytest
import torch

from fbcunn_b200 import SpatialConvolutionFBFFT, capi

pytestmark = pytest.mark.gpu


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _contraction_error():
    rng = np.random.default_rng(11)
    bins, m, n, k = 3, 128, 96, 64
    a = (rng.standard_normal((bins, m, k)) + 1j * rng.standard_normal((bins, m, k))).astype(np.complex64)
    b = (rng.standard_normal((bins, n, k)) + 1j * rng.standard_normal((bins, n, k))).astype(np.complex64)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.empty((bins, m, n), dtype=torch.complex64, device="cuda")
    capi.check(capi.lib().fbfftconv_transpose_mm(
        ctypes.c_void_p(da.data_ptr()), ctypes.c_void_p(db.data_ptr()), ctypes.c_void_p(c.data_ptr()),
        bins, m, n, k, ctypes.c_float(1.0), 0, 1, 0, _stream()))
    torch.cuda.synchronize()
    ref = np.einsum("bmk,bnk->bmn", a.astype(np.complex128), np.conj(b.astype(np.complex128)))
    return float(np.abs(c.cpu().numpy() - ref).max() / np.abs(ref).max())


def test_bounded_wait_gives_up_and_the_context_survives():
    lib = capi.lib()
    lib.fbfftconv_tensor_core_status(1)
    assert lib.fbfftconv_tensor_core_status(0) == 0
    capi.check(lib.fbfftconv_tensor_core_wait_selftest(_stream()))
    assert lib.fbfftconv_tensor_core_status(0) == 99
    # an entry point that waits for the device reports the code instead of returning OK
    m = SpatialConvolutionFBFFT(4, 4, 3, 3)
    x = torch.randn(2, 4, 8, 8, device="cuda")
    m.updateOutput(x)
    hx, hw, hb = x.cpu().pin_memory(), m.weight.cpu().pin_memory(), m.bias.cpu().pin_memory()
    hout = torch.empty(2, 4, 6, 6).pin_memory()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.fbfftconv_update_output_host(m._handle, p(hx), p(hw), p(hb), p(hout), _stream())
    assert rc == capi.ERR_CUDA and "bounded wait" in capi.last_error()
    assert lib.fbfftconv_tensor_core_status(1) == 99  # read and reset
    assert lib.fbfftconv_tensor_core_status(0) == 0
    rc = lib.fbfftconv_update_output_host(m._handle, p(hx), p(hw), p(hb), p(hout), _stream())
    assert rc == capi.OK
    np.testing.assert_allclose(hout.numpy(), m.output.cpu().numpy(), rtol=0, atol=1e-6)
    # and the tensor cores still answer
    assert _contraction_error() <= 1e-5


def test_peer_flag_wait_gives_up():
    """The flag barriers of the weight-gradient exchange over peer memory bound their waits the same
    way; one rank, a flag nothing sets, a limit of a few polls."""
    lib = capi.lib()
    capi.check(lib.fbfftconv_peer_exchange_wait_selftest(_stream()))
    assert _contraction_error() <= 1e-5


def test_host_and_foreign_pointers_are_refused():
    """THCudaTensor_checkGPU of the reference's bindings (src/fft/SpatialConvolutionCuFFTHost.cpp:33-66)."""
    lib = capi.lib()
    m = SpatialConvolutionFBFFT(3, 5, 3, 3)
    x = torch.randn(2, 3, 9, 9, device="cuda")
    out = m.updateOutput(x)
    go = torch.randn_like(out)
    h = m._handle
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    launches = capi.kernel_launches()
    host = torch.randn(2, 3, 9, 9)  # pageable host memory
    rc = lib.fbfftconv_update_output(h, p(host), p(m.weight), p(m.bias), p(out), _stream())
    assert rc == capi.ERR_INVALID_ARGUMENT and "input" in capi.last_error()
    pinned = torch.randn(2, 5, 7, 7).pin_memory()
    rc = lib.fbfftconv_update_grad_input(h, p(pinned), p(m.weight), p(x), _stream())
    assert rc == capi.ERR_INVALID_ARGUMENT and "gradOutput" in capi.last_error()
    rc = lib.fbfftconv_acc_grad_parameters(h, p(x), p(go), p(torch.empty(5, 3, 3, 3)), None, ctypes.c_float(1.0), _stream())
    assert rc == capi.ERR_INVALID_ARGUMENT and "gradWeight" in capi.last_error()
    assert capi.kernel_launches() == launches, "a refused call must launch nothing"
    if torch.cuda.device_count() >= 2:
        other = torch.randn(2, 3, 9, 9, device="cuda:1")
        rc = lib.fbfftconv_update_output(h, p(other), p(m.weight), p(m.bias), p(out), _stream())
        assert rc == capi.ERR_INVALID_ARGUMENT and "device" in capi.last_error()
    # the module still works afterwards
    m.updateOutput(x)
    torch.cuda.synchronize()
