"""Host-side mirror of the reference's Lua modules for the FFT convolution path.

``SpatialConvolutionFBFFT`` keeps the constructor, the method names, the argument
meaning, the fields and the error behaviour of ``nn.SpatialConvolutionFBFFT``
(fbcunn/SpatialConvolutionFBFFT.lua:26-354 on top of
fbcunn/SpatialConvolutionFFT.lua:150-315), so tests read like the reference's own
(test/test_FFT.lua:81-254).  Every pass is one call into the C ABI; PyTorch only
owns device memory and the current stream.  ``FFTWrapper`` mirrors
``nn.FFTWrapper`` (fbcunn/FFTWrapper.lua:30-132) over the stand-alone transforms.

Differences from the reference, on purpose:
  * no cudnn fallback (``wrapFallback``, fbcunn/SpatialConvolutionFFT.lua:323-393):
    a failed pass raises;
  * ``output`` / ``gradInput`` are re-allocated when the input shape changes (the
    reference allocates them once, fbcunn/SpatialConvolutionFFT.lua:434-441);
  * ``accGradParameters`` overwrites ``gradWeight`` / ``gradBias`` exactly as the
    reference does (fbcunn/SpatialConvolutionFBFFT.lua:337-349,
    src/ConvolutionBias.cu:95); ``accumulate=True`` selects the nn contract (+=).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import capi

memoryReuseNone = "none"
memoryReuseInput = "input"
memoryReuseOutput = "output"
memoryReuseWeight = "weight"
memoryReuseAll = "all"


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _is_number(x) -> bool:
    return isinstance(x, (int, float)) and not isinstance(x, bool)


class SpatialConvolutionFBFFT:
    """nn.SpatialConvolutionFBFFT(nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft,
    padUp, memoryReusePolicy, numCudaStreams)."""

    def __init__(self, nInputPlane, nOutputPlane, kW, kH, dW=1, dH=1, padLeft=0, padUp=0,
                 memoryReusePolicy=None, numCudaStreams=None, *, device="cuda", accumulate=False,
                 contraction: str = "auto", allreduce: str = "spectrum", exchange: str = "auto"):
        for v in (nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp):
            assert _is_number(v), "constructor arguments must be numbers"
        assert memoryReusePolicy is None or isinstance(memoryReusePolicy, (str, list, tuple))
        assert numCudaStreams is None or _is_number(numCudaStreams)
        self.nInputPlane, self.nOutputPlane = int(nInputPlane), int(nOutputPlane)
        self.kW, self.kH = int(kW), int(kH)
        self.dW, self.dH = int(dW or 1), int(dH or 1)
        self.padLeft, self.padUp = int(padLeft or 0), int(padUp or 0)
        self.padRight, self.padDown = self.padLeft, self.padUp
        assert self.dH == 1, "fft only supports stride-1 convolutions atm"
        assert self.dW == 1, "fft only supports stride-1 convolutions atm"
        assert (self.padUp < self.kH and self.padDown < self.kH and self.padLeft < self.kW
                and self.padRight < self.kW), "Padding must be smaller than kernel"
        self.fftImplementation = "fbfft"
        self.numCudaStreams = int(numCudaStreams or 16)
        if memoryReusePolicy is None or memoryReusePolicy == memoryReuseNone:
            self.memoryReusePolicy = [memoryReuseNone]
        elif memoryReusePolicy == memoryReuseAll or (
                not isinstance(memoryReusePolicy, str) and memoryReuseAll in memoryReusePolicy):
            self.memoryReusePolicy = [memoryReuseInput, memoryReuseOutput, memoryReuseWeight]
        elif isinstance(memoryReusePolicy, str):
            self.memoryReusePolicy = [memoryReusePolicy]
        else:
            self.memoryReusePolicy = list(memoryReusePolicy)
        for pol in self.memoryReusePolicy:
            assert pol in (memoryReuseNone, memoryReuseInput, memoryReuseOutput, memoryReuseWeight), \
                f"unknown memory reuse policy {pol}"

        self.device = torch.device(device)
        self._accumulate = bool(accumulate)
        assert contraction in ("auto", "simt", "bin_major")
        self._contraction = contraction
        # where accGradParameters sums across ranks once a communicator is attached: the
        # gradWeight spectrum before the inverse transform, or gradWeight itself after it
        assert allreduce in ("spectrum", "spatial")
        self._allreduce = allreduce
        # who carries that sum: the library's kernels over peer memory where they apply ("auto"), or NCCL only
        assert exchange in ("auto", "nccl")
        self._exchange = exchange
        shape_w = (self.nOutputPlane, self.nInputPlane, self.kH, self.kW)
        self.weight = torch.empty(shape_w, dtype=torch.float32, device=self.device)
        self.bias = torch.empty(self.nOutputPlane, dtype=torch.float32, device=self.device)
        self.gradWeight = torch.zeros(shape_w, dtype=torch.float32, device=self.device)
        self.gradBias = torch.zeros(self.nOutputPlane, dtype=torch.float32, device=self.device)
        self.output: Optional[torch.Tensor] = None
        self.gradInput: Optional[torch.Tensor] = None
        self.timeSteps = {"updateOutput": 0, "updateGradInput": 0, "accGradParameters": 0}
        # fields the reference's callers read or set on the module (fbcunn/SpatialConvolutionFFT.lua:162-163,
        # :259-268; fbnn.SpatialConvolution, fbcunn/SpatialConvolution.lua:188-422)
        self.printDebugLevel = -1
        self.cudnnDebug = False
        self.success = True
        self.autotuningPass = False
        self.reportErrors = True
        self._handle = None
        self._handle_key = None
        self._comm = None
        self.reset()

    # -- nn.Module surface -------------------------------------------------------
    def reset(self, stdv=None):
        """U(-stdv, stdv) for weight and bias (fbcunn/SpatialConvolutionFFT.lua:271-289)."""
        if stdv:
            stdv = stdv * math.sqrt(3)
        else:
            stdv = 1.0 / math.sqrt(self.kW * self.kH * self.nInputPlane)
        self.weight.uniform_(-stdv, stdv)
        self.bias.uniform_(-stdv, stdv)

    def updateOutput(self, input: torch.Tensor, skipBias: bool = False) -> torch.Tensor:
        self.timeSteps["updateOutput"] += 1
        self._check_input(input)
        h = self._prepare(input)
        B, _, iH, iW = input.shape
        oH, oW = iH + 2 * self.padUp - self.kH + 1, iW + 2 * self.padLeft - self.kW + 1
        shape = (B, self.nOutputPlane, oH, oW)
        if self.output is None or tuple(self.output.shape) != shape:
            self.output = torch.empty(shape, dtype=torch.float32, device=self.device)
        capi.check(capi.lib().fbfftconv_update_output(
            h, _ptr(input), _ptr(self.weight), None if skipBias else _ptr(self.bias),
            _ptr(self.output), _stream(self.device)))
        return self.output

    def updateGradInput(self, input: torch.Tensor, gradOutput: torch.Tensor) -> torch.Tensor:
        self.timeSteps["updateGradInput"] += 1
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        h = self._prepare(input)
        if self.gradInput is None or self.gradInput.shape != input.shape:
            self.gradInput = torch.empty_like(input)
        capi.check(capi.lib().fbfftconv_update_grad_input(
            h, _ptr(gradOutput), _ptr(self.weight), _ptr(self.gradInput), _stream(self.device)))
        return self.gradInput

    def accGradParameters(self, input: torch.Tensor, gradOutput: torch.Tensor, scale=None,
                          skipBias: bool = False) -> None:
        self.timeSteps["accGradParameters"] += 1
        scale = 1.0 if scale is None else float(scale)
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        h = self._prepare(input)
        capi.check(capi.lib().fbfftconv_acc_grad_parameters(
            h, _ptr(input), _ptr(gradOutput), _ptr(self.gradWeight),
            None if skipBias else _ptr(self.gradBias), ctypes.c_float(scale), _stream(self.device)))

    # The per-pass implementations the reference's subclasses and wrappers call directly
    # (fbcunn/SpatialConvolutionFBFFT.lua:102, :189, :269; callers
    # fbcunn/SpatialConvolutionFFTTiled.lua:262-263, :479, :593, :714).  `reuseList` is accepted for
    # signature compatibility (the reuse policy of the module decides); `metaData` may carry
    # skipBias, which the tiled callers set to add the bias once after the last tile.
    def updateOutputFFTImpl(self, input, reuseList=None, metaData=None):
        return self.updateOutput(input, skipBias=bool(metaData and metaData.get("skipBias")))

    def updateGradInputFFTImpl(self, input, gradOutput, reuseList=None, metaData=None):
        return self.updateGradInput(input, gradOutput)

    def accGradParametersFFTImpl(self, input, gradOutput, scale=None, reuseList=None, metaData=None):
        return self.accGradParameters(input, gradOutput, scale,
                                      skipBias=bool(metaData and metaData.get("skipBias")))

    def forward(self, input):
        return self.updateOutput(input)

    def backward(self, input, gradOutput, scale=None):
        """updateGradInput then accGradParameters (fbcunn/SpatialConvolutionFFT.lua:405-416)."""
        self.updateGradInput(input, gradOutput)
        self.accGradParameters(input, gradOutput, scale)
        return self.gradInput

    def zeroGradParameters(self):
        self.gradWeight.zero_()
        self.gradBias.zero_()

    def cleanupBuffers(self):
        """Frees the frequency buffers (fbcunn/SpatialConvolutionFFT.lua:852-870)."""
        if self._handle is not None:
            capi.lib().fbfftconv_destroy(self._handle)
            self._handle = None
            self._handle_key = None

    # the reference's reuse switches (fbcunn/SpatialConvolutionFFT.lua:405-416): a spectrum is
    # taken over from the earlier pass of the step where both passes read one layout (see
    # FBFFTCONV_REUSE_* in include/fbfftconv.h); the native handle is rebuilt on a change
    def setReuseInputs(self, val):
        self._toggle(memoryReuseInput, val)

    def setReuseOutputs(self, val):
        self._toggle(memoryReuseOutput, val)

    def setReuseWeights(self, val):
        self._toggle(memoryReuseWeight, val)

    # -- multi-GPU -----------------------------------------------------------------
    def attachCommunicator(self, unique_id: bytes, rank: int, nranks: int):
        """One rank per GPU: accGradParameters then sums the frequency-domain weight
        gradient (and gradBias) over all ranks with NCCL before the inverse transform
        (an all-reduce; for plane-major layers a reduce-scatter by filters, the inverse
        transform of the rank's own filters and an all-gather of the result).  With
        allreduce="spatial" the sum happens after the inverse transform instead.
        Replaces the gather/add/broadcast of nn.DataParallel
        (fbcunn/DataParallel.lua:105-131)."""
        assert len(unique_id) == 128
        self._comm = (bytes(unique_id), int(rank), int(nranks))
        if self._handle is not None:
            self._init_comm()

    def peerExchangeStatus(self, reset: bool = False) -> int:
        """1 = accGradParameters sums over peer memory, 0 = over NCCL (or not run yet), 100 + c = a
        bounded wait of the exchange gave up on rank c - 1 (fbfftconv_peer_exchange_status)."""
        return int(capi.lib().fbfftconv_peer_exchange_status(self._handle, int(reset))) if self._handle is not None else 0

    @staticmethod
    def makeUniqueId() -> bytes:
        buf = ctypes.create_string_buffer(128)
        capi.check(capi.lib().fbfftconv_comm_unique_id(buf))
        return buf.raw

    # -- internals -----------------------------------------------------------------
    def _toggle(self, what, val):
        if val and what not in self.memoryReusePolicy:
            self.memoryReusePolicy = [p for p in self.memoryReusePolicy if p != memoryReuseNone] + [what]
        elif not val and what in self.memoryReusePolicy:
            self.memoryReusePolicy = [p for p in self.memoryReusePolicy if p != what] or [memoryReuseNone]

    def _check_input(self, input):
        assert isinstance(input, torch.Tensor) and input.is_cuda, "CUDA support only!"
        assert input.dim() == 4, "2D convolutions on 4D tensors atm"
        assert input.dtype == torch.float32 and input.is_contiguous()
        assert input.shape[1] == self.nInputPlane, "num planes mismatch"

    def _check_grad_output(self, input, gradOutput):
        assert isinstance(gradOutput, torch.Tensor) and gradOutput.is_cuda, "CUDA support only!"
        assert gradOutput.dtype == torch.float32 and gradOutput.is_contiguous()
        B, _, iH, iW = input.shape
        oH, oW = iH + 2 * self.padUp - self.kH + 1, iW + 2 * self.padLeft - self.kW + 1
        assert tuple(gradOutput.shape) == (B, self.nOutputPlane, oH, oW), "gradOutput size mismatch"

    def _init_comm(self):
        uid, rank, nranks = self._comm
        capi.check(capi.lib().fbfftconv_comm_init(self._handle, ctypes.c_char_p(uid), rank, nranks))

    def _flags(self) -> int:
        return (capi.ACCUMULATE_GRADS if self._accumulate else 0) | \
                (capi.CONTRACT_SIMT if self._contraction == "simt" else 0) | \
                (capi.BIN_MAJOR_ONLY if self._contraction == "bin_major" else 0) | \
                (capi.ALLREDUCE_SPATIAL if self._allreduce == "spatial" else 0) | \
                (capi.EXCHANGE_NCCL if self._exchange == "nccl" else 0) | \
                (capi.REUSE_INPUT if memoryReuseInput in self.memoryReusePolicy else 0) | \
                (capi.REUSE_OUTPUT if memoryReuseOutput in self.memoryReusePolicy else 0) | \
                (capi.REUSE_WEIGHT if memoryReuseWeight in self.memoryReusePolicy else 0)

    def _prepare(self, input):
        """prepareSizeAndBuffers: a native handle per (batch, image size)."""
        B, _, iH, iW = input.shape
        flags = self._flags()
        key = (int(B), int(iH), int(iW), flags)
        if self._handle is not None and self._handle_key == key:
            return self._handle
        self.cleanupBuffers()
        desc = capi.Desc(B, self.nInputPlane, self.nOutputPlane, iH, iW, self.kH, self.kW,
                         self.dH, self.dW, self.padUp, self.padLeft,
                         self.device.index if self.device.index is not None else torch.cuda.current_device(),
                         flags)
        h = ctypes.c_void_p()
        capi.check(capi.lib().fbfftconv_create(ctypes.byref(desc), ctypes.byref(h)))
        self._handle, self._handle_key = h, key
        if self._comm is not None:
            self._init_comm()
        return self._handle

    @property
    def fftSize(self) -> int:
        return int(capi.lib().fbfftconv_fft_size(self._handle)) if self._handle is not None else 0

    def __del__(self):
        try:
            self.cleanupBuffers()
        except Exception:
            pass


class SpatialConvolutionFBFFTGemm(SpatialConvolutionFBFFT):
    """nn.SpatialConvolutionFBFFTGemm (fbcunn/SpatialConvolutionFBFFTGemm.lua:18-66): the variant of
    the reference that transposes its spectra with cublasCgeam and multiplies them with
    cublasCgemmBatched.  Here the spectra are written bin-major by the transform itself and the
    per-bin product is the same tensor-core contraction, so the variant is the same native path
    under the reference's second class name."""


class CuBLASWrapper:
    """nn.CuBLASWrapper (fbcunn/CuBLASWrapper.lua:1-49) for the one use the convolution makes of it:
    matmultComplex on bin-major operands, C[bin] = scale * op(A[bin]) * op(B[bin]) with op 'n' or 'c'
    (fbcunn/SpatialConvolutionFBFFTGemm.lua:179-186, :301-308, :424-431).  A is (bins, m, k),
    B is (bins, n, k), C is (bins, m, n), complex64, k and n padded to multiples of 4 (see
    fbfftconv_transpose_mm): the rows of B are what the reference reaches with transB."""

    def __init__(self, timed=False):
        self.timed = bool(timed)

    def matmultComplex(self, A, B, C, iterDims=(), batchDims=(), transA="n", transB="n", scale=1.0):
        assert transA in ("n", "c") and transB in ("n", "c")
        assert A.is_cuda and A.dtype == torch.complex64 and A.dim() == 3 and A.is_contiguous()
        assert B.dtype == torch.complex64 and B.dim() == 3 and B.is_contiguous()
        assert C.dtype == torch.complex64 and C.dim() == 3 and C.is_contiguous()
        bins, m, kpad = A.shape
        n = B.shape[1]
        assert B.shape[0] == bins and B.shape[2] == kpad and kpad % 4 == 0
        assert tuple(C.shape) == (bins, m, (n + 3) // 4 * 4)
        capi.check(capi.lib().fbfftconv_transpose_mm(
            _ptr(A), _ptr(B), _ptr(C), bins, m, n, kpad, ctypes.c_float(scale),
            int(transA == "c"), int(transB == "c"), 0, _stream(A.device)))
        return C


class FFTWrapper:
    """nn.FFTWrapper('fbfft', padLeft, padUp): fft(time, frequency) / ffti(time, frequency)
    for 4-D real tensors (two batch dimensions, 2-D transform), the case the
    convolution uses (fbcunn/FFTWrapper.lua:53-132).  ``frequency`` is a complex64
    tensor shaped (bins, d1, d2_padded) -- or (bins, d2, d1_padded) when
    ``transposed`` -- with bins = N*(N/2+1), bin = ky*(N/2+1) + kx; `to_plane_major` turns it
    into (d1, d2, N, N/2+1) [ky][kx]."""

    def __init__(self, implementation="fbfft", padLeft=0, padUp=0):
        assert implementation == "fbfft", "only the fbfft path exists here"
        self.padLeft, self.padUp = int(padLeft), int(padUp)

    @staticmethod
    def frequency_tensor(d1, d2, fft_size, device="cuda", transposed=False):
        rows, inner = (d2, d1) if transposed else (d1, d2)
        bins = (fft_size // 2 + 1) * fft_size
        return torch.empty((bins, rows, (inner + 3) // 4 * 4), dtype=torch.complex64, device=device)

    def fft(self, time: torch.Tensor, frequency: torch.Tensor, fft_size: int, transposed=False):
        assert time.is_cuda and time.dim() == 4 and time.is_contiguous() and time.dtype == torch.float32
        d1, d2, h, w = time.shape
        capi.check(capi.lib().fbfftconv_fft2d(_ptr(time), _ptr(frequency), d1, d2, h, w, fft_size,
                                              self.padUp, self.padLeft, int(transposed), _stream(time.device)))
        return frequency

    def ffti(self, time: torch.Tensor, frequency: torch.Tensor, fft_size: int, bias=None, accumulate=False):
        assert time.is_cuda and time.dim() == 4 and time.is_contiguous() and time.dtype == torch.float32
        d1, d2, h, w = time.shape
        capi.check(capi.lib().fbfftconv_ifft2d(_ptr(frequency), _ptr(time), _ptr(bias), d1, d2, h, w, fft_size,
                                               self.padUp, self.padLeft, int(accumulate), 0, _stream(time.device)))
        return time

    @staticmethod
    def to_plane_major(frequency: torch.Tensor, inner: int, fft_size: int, transposed=False):
        n = fft_size
        f = frequency[:, :, :inner].reshape(n, n // 2 + 1, frequency.shape[1], inner)  # ky, kx, row, inner
        f = f.permute(2, 3, 0, 1)  # row, inner, ky, kx
        return f.transpose(0, 1).contiguous() if transposed else f.contiguous()

    @staticmethod
    def from_plane_major(spec: torch.Tensor, fft_size: int):
        """(d1, d2, N, N/2+1) complex -> bin-major (bins, d1, d2_padded)."""
        d1, d2, n, half = spec.shape
        assert n == fft_size and half == n // 2 + 1
        out = torch.zeros((half * n, d1, (d2 + 3) // 4 * 4), dtype=torch.complex64, device=spec.device)
        out[:, :, :d2] = spec.permute(2, 3, 0, 1).reshape(half * n, d1, d2)
        return out

    # -- the reference's tensor contract (fbcunn/FFTWrapper.lua:53-132) ----------------------
    # time: (batch dims..., fft dims) real; frequency: the same with the first FFT dimension cut
    # to N/2+1, plus a trailing 2 for (re, im).  One FFT dimension: frequency[b][k].  Two:
    # sizes 8..32 keep the half spectrum along the first FFT dimension, frequency[b][i][j] =
    # X[ky=i][kx=j]; the other sizes keep it along the second and store it transposed,
    # frequency[b][i][j] = X[ky=j][kx=i] (test/test_FFTModule.lua:310-342).
    @staticmethod
    def _half_along_rows(n: int) -> bool:
        return 8 <= n <= 32

    def fft_reference_layout(self, time: torch.Tensor, frequency: torch.Tensor, batchDims: int):
        assert 1 <= batchDims <= 2 and time.is_cuda and time.dtype == torch.float32 and time.is_contiguous()
        fft_dims = time.dim() - batchDims
        assert fft_dims in (1, 2) and frequency.shape[-1] == 2 and frequency.is_contiguous()
        stream = _stream(time.device)
        if fft_dims == 1:
            n_fft = (frequency.shape[-2] - 1) * 2
            rows = time.numel() // time.shape[-1]
            capi.check(capi.lib().fbfftconv_fft1d(_ptr(time), _ptr(frequency), rows, time.shape[-1], n_fft,
                                                  self.padLeft, stream))
            return frequency
        n_fft = frequency.shape[-2]
        assert frequency.shape[-3] == n_fft // 2 + 1
        h, w = time.shape[-2:]
        planes = time.numel() // (h * w)
        scratch = self._scratch(planes, n_fft, time.device)
        capi.check(capi.lib().fbfftconv_fft2d_reference_layout(
            _ptr(time), _ptr(frequency), _ptr(scratch), planes, h, w, n_fft, self.padUp, self.padLeft, stream))
        return frequency

    def _scratch(self, planes, n_fft, device):
        """The library's own half spectrum of `planes` planes (a kernel converts it to / from the
        reference's tensor); kept between calls of the same size."""
        need = int(capi.lib().fbfftconv_spectrum_bytes(n_fft, 1, planes))
        buf = getattr(self, "_scratch_buf", None)
        if buf is None or buf.numel() < need or buf.device != torch.device(device):
            buf = torch.empty(need, dtype=torch.uint8, device=device)
            self._scratch_buf = buf
        return buf

    def ffti_reference_layout(self, time: torch.Tensor, frequency: torch.Tensor, batchDims: int):
        assert 1 <= batchDims <= 2 and time.is_cuda and time.dtype == torch.float32 and time.is_contiguous()
        fft_dims = time.dim() - batchDims
        assert fft_dims in (1, 2) and frequency.shape[-1] == 2 and frequency.is_contiguous()
        stream = _stream(time.device)
        if fft_dims == 1:
            n_fft = (frequency.shape[-2] - 1) * 2
            rows = time.numel() // time.shape[-1]
            capi.check(capi.lib().fbfftconv_ifft1d(_ptr(frequency), _ptr(time), rows, time.shape[-1], n_fft,
                                                   self.padLeft, stream))
            return time
        n_fft = frequency.shape[-2]
        h, w = time.shape[-2:]
        planes = time.numel() // (h * w)
        scratch = self._scratch(planes, n_fft, time.device)
        capi.check(capi.lib().fbfftconv_ifft2d_reference_layout(
            _ptr(frequency), _ptr(time), _ptr(scratch), planes, h, w, n_fft, self.padUp, self.padLeft, stream))
        return time
