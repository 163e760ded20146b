"""ctypes binding of libfbfftconv.so (the C ABI in include/fbfftconv.h).

This is the same boundary a LuaJIT FFI caller binds (fbcunn_b200/lua/); Python is
only the harness used by the tests and the benchmark.  There is no fallback: if the
library cannot be loaded every call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_size_t, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# FBFFTCONV_LIB points at another build of the same library (tuning experiments)
LIB_PATH = os.environ.get("FBFFTCONV_LIB") or os.path.join(HERE, "libfbfftconv.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED_SIZE = 2
ERR_NOMEM = 3
ERR_CUDA = 4
ERR_COMM = 5

ACCUMULATE_GRADS = 1
CONTRACT_SIMT = 2
BIN_MAJOR_ONLY = 4
ALLREDUCE_SPATIAL = 8
REUSE_INPUT = 16
REUSE_OUTPUT = 32
REUSE_WEIGHT = 64
EXCHANGE_NCCL = 128


class Desc(ctypes.Structure):
    """struct fbfftconv_desc."""

    _fields_ = [
        ("batch", c_int32), ("n_input_plane", c_int32), ("n_output_plane", c_int32),
        ("input_h", c_int32), ("input_w", c_int32), ("kernel_h", c_int32), ("kernel_w", c_int32),
        ("stride_h", c_int32), ("stride_w", c_int32), ("pad_h", c_int32), ("pad_w", c_int32),
        ("device", c_int32), ("flags", c_uint32),
    ]


class FbfftconvError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"fbfftconv status {status}: {message}")
        self.status = status


_lib = None

_SIGNATURES = {
    "fbfftconv_create": (c_int, [POINTER(Desc), POINTER(c_void_p)]),
    "fbfftconv_destroy": (c_int, [c_void_p]),
    "fbfftconv_fft_size": (c_int, [c_void_p]),
    "fbfftconv_workspace_bytes": (c_size_t, [c_void_p]),
    "fbfftconv_set_workspace": (c_int, [c_void_p, c_void_p, c_size_t]),
    "fbfftconv_update_output": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_update_grad_input": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_acc_grad_parameters": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "fbfftconv_update_output_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_update_grad_input_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_acc_grad_parameters_host": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "fbfftconv_update_output_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_update_grad_input_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_acc_grad_parameters_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "fbfftconv_backward_host_async": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "fbfftconv_host_sync": (c_int, [c_void_p]),
    "fbfftconv_spectrum_bytes": (c_size_t, [c_int, c_int, c_int]),
    "fbfftconv_fft2d": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_ifft2d": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_fft1d": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_ifft1d": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_tiled_create": (c_int, [POINTER(Desc), c_int, c_int, POINTER(c_void_p)]),
    "fbfftconv_tiled_destroy": (c_int, [c_void_p]),
    "fbfftconv_tiled_inner": (c_void_p, [c_void_p]),
    "fbfftconv_tiled_workspace_bytes": (c_size_t, [c_void_p]),
    "fbfftconv_tiled_geometry": (c_int, [c_void_p, POINTER(c_int32)]),
    "fbfftconv_tiled_update_output": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_tiled_update_grad_input": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "fbfftconv_tiled_acc_grad_parameters": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "fbfftconv_fft2d_reference_layout": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_ifft2d_reference_layout": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_transpose_mm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_tensor_core_status": (c_int, [c_int]),
    "fbfftconv_tensor_core_wait_selftest": (c_int, [c_void_p]),
    "fbfftconv_peer_exchange_status": (c_int, [c_void_p, c_int]),
    "fbfftconv_peer_exchange_wait_selftest": (c_int, [c_void_p]),
    "fbfftconv_exchange_plan": (c_int, [c_void_p, c_int, c_int, c_void_p]),
    "fbfftconv_update_output_bias": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "fbfftconv_acc_grad_parameters_bias": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "fbfftconv_acc_grad_parameters_bias_noalloc": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]),
    "fbfftconv_profile_enable": (c_int, [c_void_p, c_int]),
    "fbfftconv_profile_reset": (c_int, [c_void_p]),
    "fbfftconv_profile_read": (c_int, [c_void_p, c_int, c_int, POINTER(ctypes.c_double), POINTER(c_int)]),
    "fbfftconv_profile_overlapped": (c_int, [c_void_p, c_int, c_int]),
    "fbfftconv_comm_unique_id": (c_int, [c_void_p]),
    "fbfftconv_comm_init": (c_int, [c_void_p, c_void_p, c_int, c_int]),
    "fbfftconv_comm_destroy": (c_int, [c_void_p]),
    "fbfftconv_comm_shutdown": (c_int, []),
    "fbfftconv_last_error": (c_char_p, []),
    "fbfftconv_status_string": (c_char_p, [c_int]),
    "fbfftconv_kernel_launches": (c_uint64, []),
}

EXPORTS = tuple(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python -m fbcunn_b200.build` "
                "(there is no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != OK:
        raise FbfftconvError(status, lib().fbfftconv_last_error().decode("utf-8", "replace"))


def last_error() -> str:
    return lib().fbfftconv_last_error().decode("utf-8", "replace")


def kernel_launches() -> int:
    return int(lib().fbfftconv_kernel_launches())
