"""ctypes front end of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

``liboracle.so`` is the fp64 restatement (refconv.c).  ``_ref/libfbcunn_ref.so`` is
the reference's own test/ReferenceConvolutions.cpp compiled unchanged against
stand-in headers (ref_bridge.cpp); it exists only where the reference checkout was
present at build time.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libfbcunn_ref.so")


class _CShape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("B", "P", "F", "iH", "iW", "kH", "kW", "padH", "padW")]


@dataclass(frozen=True)
class Shape:
    """Problem size of one convolution layer (stride 1, symmetric padding)."""

    B: int
    P: int
    F: int
    iH: int
    iW: int
    kH: int
    kW: int
    padH: int = 0
    padW: int = 0

    @property
    def oH(self) -> int:
        return self.iH + 2 * self.padH - self.kH + 1

    @property
    def oW(self) -> int:
        return self.iW + 2 * self.padW - self.kW + 1

    def c(self) -> _CShape:
        return _CShape(self.B, self.P, self.F, self.iH, self.iW, self.kH, self.kW, self.padH, self.padW)


def _reference_root() -> str:
    """Where the reference checkout lies: FBCUNN_REFERENCE_ROOT, else a directory `reference`
    beside this repository; '' when there is none (the prebuilt _ref/ library is then used)."""
    for cand in (os.environ.get("FBCUNN_REFERENCE_ROOT", ""),
                 os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "test", "ReferenceConvolutions.cpp")):
            return cand
    return ""


def _stale(lib: str, sources) -> str:
    """Content hash of the sources if it differs from the one `lib` was built from
    (file times do not survive a copy of the tree), else ''."""
    h = hashlib.sha256()
    for src in sources:
        with open(src, "rb") as f:
            h.update(f.read())
    digest = h.hexdigest()
    stamp = lib + ".stamp"
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return ""
    return digest


def build(force: bool = False) -> None:
    """Compile refconv.c and, where the reference checkout is present, the reference's own
    CPU convolution from where it lies (outputs stay under _ref/).  A machine without the
    checkout keeps using the prebuilt _ref/ library."""
    digest = _stale(_LIB, [os.path.join(_HERE, "refconv.c"), os.path.join(_HERE, "Makefile")])
    if force or digest:
        subprocess.check_call(["make", "-s", "-B", "-C", _HERE, os.path.join(_HERE, "liboracle.so")])
        with open(_LIB + ".stamp", "w") as f:
            f.write(digest or _stale(_LIB + ".none", [os.path.join(_HERE, "refconv.c"), os.path.join(_HERE, "Makefile")]))
    root = _reference_root()
    if root:
        reference_src = os.path.join(root, "test", "ReferenceConvolutions.cpp")
        shim = [os.path.join(_HERE, "shim", d, f) for d, f in
                (("thpp", "Tensor.h"), ("thpp", "Storage.h"), ("folly", "Optional.h"), ("glog", "logging.h"))]
        srcs = [os.path.join(_HERE, "ref_bridge.cpp"), reference_src] + shim
        digest = _stale(_REF, srcs)
        if force or digest:
            subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "REFERENCE_ROOT=" + root])
            with open(_REF + ".stamp", "w") as f:
                f.write(digest or _stale(_REF + ".none", srcs))


_lib = None
_ref = None


def _oracle():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB)
    return _lib


def reference_available() -> bool:
    if not os.path.exists(_REF):
        try:
            build()
        except Exception:
            return False
    return os.path.exists(_REF)


def _reference():
    global _ref
    if _ref is None:
        if not reference_available():
            raise RuntimeError("compiled reference (oracle/_ref) is not available")
        _ref = ctypes.CDLL(_REF)
    return _ref


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _pf(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _pd(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _pi(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))


def _check(s: Shape, input=None, weight=None, grad_output=None):
    if input is not None:
        assert input.shape == (s.B, s.P, s.iH, s.iW), (input.shape, s)
    if weight is not None:
        assert weight.shape == (s.F, s.P, s.kH, s.kW), (weight.shape, s)
    if grad_output is not None:
        assert grad_output.shape == (s.B, s.F, s.oH, s.oW), (grad_output.shape, s)


# ---- fp64 restatement ---------------------------------------------------------

def update_output(s: Shape, input, weight, bias=None) -> np.ndarray:
    input, weight = _f32(input), _f32(weight)
    _check(s, input=input, weight=weight)
    b = _f32(bias) if bias is not None else None
    out = np.empty((s.B, s.F, s.oH, s.oW), np.float64)
    rc = _oracle().oracle_update_output(ctypes.byref(s.c()), _pf(input), _pf(weight),
                                        _pf(b) if b is not None else None, _pd(out))
    assert rc == 0
    return out


def update_grad_input(s: Shape, grad_output, weight) -> np.ndarray:
    grad_output, weight = _f32(grad_output), _f32(weight)
    _check(s, weight=weight, grad_output=grad_output)
    out = np.empty((s.B, s.P, s.iH, s.iW), np.float64)
    rc = _oracle().oracle_update_grad_input(ctypes.byref(s.c()), _pf(grad_output), _pf(weight), _pd(out))
    assert rc == 0
    return out


def acc_grad_weight(s: Shape, input, grad_output, scale: float = 1.0) -> np.ndarray:
    input, grad_output = _f32(input), _f32(grad_output)
    _check(s, input=input, grad_output=grad_output)
    out = np.empty((s.F, s.P, s.kH, s.kW), np.float64)
    rc = _oracle().oracle_acc_grad_weight(ctypes.byref(s.c()), _pf(input), _pf(grad_output),
                                          ctypes.c_double(scale), _pd(out))
    assert rc == 0
    return out


def acc_grad_bias(s: Shape, grad_output, scale: float = 1.0) -> np.ndarray:
    grad_output = _f32(grad_output)
    _check(s, grad_output=grad_output)
    out = np.empty((s.F,), np.float64)
    rc = _oracle().oracle_acc_grad_bias(ctypes.byref(s.c()), _pf(grad_output), ctypes.c_double(scale), _pd(out))
    assert rc == 0
    return out


def _pairs(first, second):
    a = np.ascontiguousarray(first, dtype=np.int64)
    b = np.ascontiguousarray(second, dtype=np.int64)
    assert a.shape == b.shape and a.ndim == 1
    return a, b


def update_output_planes(s: Shape, input, weight, bias, b_idx, f_idx) -> np.ndarray:
    """output[b_idx[i], f_idx[i]] for each i, shape (n, oH, oW)."""
    input, weight = _f32(input), _f32(weight)
    _check(s, input=input, weight=weight)
    bb = _f32(bias) if bias is not None else None
    a, b = _pairs(b_idx, f_idx)
    out = np.empty((len(a), s.oH, s.oW), np.float64)
    rc = _oracle().oracle_update_output_planes(ctypes.byref(s.c()), _pf(input), _pf(weight),
                                               _pf(bb) if bb is not None else None,
                                               ctypes.c_int64(len(a)), _pi(a), _pi(b), _pd(out))
    assert rc == 0
    return out


def update_grad_input_planes(s: Shape, grad_output, weight, b_idx, p_idx) -> np.ndarray:
    grad_output, weight = _f32(grad_output), _f32(weight)
    _check(s, weight=weight, grad_output=grad_output)
    a, b = _pairs(b_idx, p_idx)
    out = np.empty((len(a), s.iH, s.iW), np.float64)
    rc = _oracle().oracle_update_grad_input_planes(ctypes.byref(s.c()), _pf(grad_output), _pf(weight),
                                                   ctypes.c_int64(len(a)), _pi(a), _pi(b), _pd(out))
    assert rc == 0
    return out


def acc_grad_weight_planes(s: Shape, input, grad_output, scale, f_idx, p_idx) -> np.ndarray:
    input, grad_output = _f32(input), _f32(grad_output)
    _check(s, input=input, grad_output=grad_output)
    a, b = _pairs(f_idx, p_idx)
    out = np.empty((len(a), s.kH, s.kW), np.float64)
    rc = _oracle().oracle_acc_grad_weight_planes(ctypes.byref(s.c()), _pf(input), _pf(grad_output),
                                                 ctypes.c_double(scale), ctypes.c_int64(len(a)),
                                                 _pi(a), _pi(b), _pd(out))
    assert rc == 0
    return out


# ---- the compiled reference (fp32 accumulation, as the reference has it) --------

def _dims(s: Shape):
    return [ctypes.c_long(v) for v in (s.B, s.P, s.F, s.iH, s.iW, s.kH, s.kW, s.padH, s.padW)]


def reference_update_output(s: Shape, input, weight, threads: int = 1) -> np.ndarray:
    input, weight = _f32(input), _f32(weight)
    _check(s, input=input, weight=weight)
    out = np.empty((s.B, s.F, s.oH, s.oW), np.float32)
    _reference().ref_update_output(_pf(input), _pf(weight), _pf(out), *_dims(s), ctypes.c_int(threads))
    return out


def reference_update_grad_input(s: Shape, grad_output, weight, threads: int = 1) -> np.ndarray:
    grad_output, weight = _f32(grad_output), _f32(weight)
    _check(s, weight=weight, grad_output=grad_output)
    out = np.empty((s.B, s.P, s.iH, s.iW), np.float32)
    _reference().ref_update_grad_input(_pf(grad_output), _pf(weight), _pf(out), *_dims(s), ctypes.c_int(threads))
    return out


def reference_acc_grad_weight(s: Shape, input, grad_output, scale: float = 1.0, threads: int = 1) -> np.ndarray:
    input, grad_output = _f32(input), _f32(grad_output)
    _check(s, input=input, grad_output=grad_output)
    out = np.empty((s.F, s.P, s.kH, s.kW), np.float32)
    _reference().ref_acc_grad_weight(_pf(input), _pf(grad_output), _pf(out), *_dims(s),
                                     ctypes.c_float(scale), ctypes.c_int(threads))
    return out
