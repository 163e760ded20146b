"""The allocation-free bias gradient (fbfftconv_acc_grad_parameters_bias_noalloc) for
callers that cannot get device memory when they need it (an allocator that owns the
whole GPU, a fixed memory budget): its partial sums live in a fixed array inside the
library instead of caller scratch.  Checked through the C ABI against the existing
entry point, twice in a row with different shapes so that whatever the first call left
in the shared array would show in the second.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest
import torch

from fbcunn_b200 import capi


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.gpu
def test_noalloc_bias_gradient_matches_scratch_variant():
    lib = capi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    gen = torch.Generator(device="cuda").manual_seed(31337)
    # first call larger than the second: stale partial sums would be picked up
    for call, (B, F, h, w, scale, accumulate) in enumerate([(32, 48, 13, 11, 0.75, 0), (5, 7, 6, 9, 1.5, 1)]):
        go = torch.empty((B, F, h, w), device="cuda").normal_(generator=gen)
        init = torch.empty(F, device="cuda").normal_(generator=gen)
        expect, got = init.clone(), init.clone()
        scratch = torch.empty(B * F, device="cuda")
        capi.check(lib.fbfftconv_acc_grad_parameters_bias(_ptr(go), _ptr(expect), _ptr(scratch), B, F, h, w,
                                                          ctypes.c_float(scale), accumulate, stream))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        capi.check(lib.fbfftconv_acc_grad_parameters_bias_noalloc(_ptr(go), _ptr(got), B, F, h, w,
                                                                  ctypes.c_float(scale), accumulate, stream))
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated"
        ref = scale * go.double().sum((0, 2, 3)) + (init.double() if accumulate else 0.0)
        # same kernels, same order of summation: identical to the scratch variant, and
        # within the 1e-4 * max|ref| bar of the pass tests against an fp64 sum
        assert torch.equal(got, expect), f"call {call}"
        assert float((got.double() - ref).abs().max()) <= 1e-4 * float(ref.abs().max())


@pytest.mark.gpu
def test_noalloc_bias_gradient_rejects_sizes_beyond_its_array():
    lib = capi.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    go = torch.zeros(8, device="cuda")
    gb = torch.zeros(8, device="cuda")
    rc = lib.fbfftconv_acc_grad_parameters_bias_noalloc(_ptr(go), _ptr(gb), 1024, 65, 1, 1,
                                                        ctypes.c_float(1.0), 0, stream)
    assert rc == capi.ERR_UNSUPPORTED_SIZE
    assert "65536" in capi.last_error()
    assert lib.fbfftconv_acc_grad_parameters_bias_noalloc(None, _ptr(gb), 1, 1, 1, 1, ctypes.c_float(1.0), 0,
                                                          stream) == capi.ERR_INVALID_ARGUMENT
