"""nn.SpatialConvolutionFFTTiled: the FFT convolution on tiles of the image.

Mirrors the reference's tiled module (fbcunn/SpatialConvolutionFFTTiled.lua:265-365 for the
constructor, :489-563 / :601-683 / :724-802 for the three passes): the output is cut into
disjoint tiles of (tileSize - k + 1) pixels, each of which depends on an input tile of
tileSize pixels (overlap-save), so the transform size stays at tileSize whatever the image
size -- which also lifts the 128-pixel limit of the untiled module.

The work is the native library's (fbfftconv_tiled_* in include/fbfftconv.h): the tiles of one
image become extra batch entries of one untiled pass,

    updateOutput        input tiles (overlapping)  -> output tiles (disjoint)
    updateGradInput     gradOutput tiles (disjoint) -> gradInput tiles, overlap-added
    accGradParameters   the sum over the batch inside the contraction is also the sum
                        over tiles, so gradWeight / gradBias come out complete

and cutting, assembling and the overlap-add are kernels of the library.  This class only
owns the tensors and mirrors the reference's constructor and methods.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi
from .module import SpatialConvolutionFBFFT, _ptr, _stream


class SpatialConvolutionFFTTiled(SpatialConvolutionFBFFT):
    """nn.SpatialConvolutionFFTTiled(nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp,
    tileSizeW, tileSizeH, memoryReusePolicy, numCudaStreams); tile sizes default to 16
    (fbcunn/SpatialConvolutionFFTTiled.lua:357-358)."""

    def __init__(self, nInputPlane, nOutputPlane, kW, kH, dW=1, dH=1, padLeft=0, padUp=0,
                 tileSizeW=None, tileSizeH=None, memoryReusePolicy=None, numCudaStreams=None, **kw):
        super().__init__(nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp,
                         memoryReusePolicy, numCudaStreams, **kw)
        self.tileSizeH = int(tileSizeH or 16)
        self.tileSizeW = int(tileSizeW or 16)
        assert self.tileSizeH > self.kH - 1 and self.tileSizeW > self.kW - 1, \
            "tile size must exceed the kernel size minus one"
        self._tiled = None
        self._tiled_key = None

    # -- tiling geometry (what the native side computes; kept for callers that size buffers) --
    def _geometry(self, iH, iW):
        oH = iH + 2 * self.padUp - self.kH + 1
        oW = iW + 2 * self.padLeft - self.kW + 1
        assert oH > 0 and oW > 0, "kernel larger than the padded input"
        tH, tW = min(self.tileSizeH, iH + 2 * self.padUp), min(self.tileSizeW, iW + 2 * self.padLeft)
        sH, sW = tH - self.kH + 1, tW - self.kW + 1          # output tile = step of the input tiles
        nH, nW = -(-oH // sH), -(-oW // sW)                   # tiles per image
        pH, pW = (nH - 1) * sH + tH, (nW - 1) * sW + tW      # padded input extent the tiles cover
        return oH, oW, tH, tW, sH, sW, nH, nW, pH, pW

    def _prepare_tiled(self, input):
        B, _, iH, iW = input.shape
        flags = self._flags()
        key = (int(B), int(iH), int(iW), flags)
        if self._tiled is not None and self._tiled_key == key:
            return self._tiled
        self.cleanupBuffers()
        desc = capi.Desc(B, self.nInputPlane, self.nOutputPlane, iH, iW, self.kH, self.kW, self.dH, self.dW,
                         self.padUp, self.padLeft,
                         self.device.index if self.device.index is not None else torch.cuda.current_device(), flags)
        t = ctypes.c_void_p()
        capi.check(capi.lib().fbfftconv_tiled_create(ctypes.byref(desc), self.tileSizeH, self.tileSizeW,
                                                     ctypes.byref(t)))
        self._tiled, self._tiled_key = t, key
        # the untiled layer of the tiles: communicator, profiling and status queries go to it
        self._handle = ctypes.c_void_p(capi.lib().fbfftconv_tiled_inner(t))
        self._handle_key = None
        if self._comm is not None:
            self._init_comm()
        return t

    # -- passes ------------------------------------------------------------------------
    def updateOutput(self, input: torch.Tensor, skipBias: bool = False) -> torch.Tensor:
        self.timeSteps["updateOutput"] += 1
        self._check_input(input)
        t = self._prepare_tiled(input)
        B, _, iH, iW = input.shape
        oH, oW = self._geometry(iH, iW)[:2]
        shape = (B, self.nOutputPlane, oH, oW)
        if self.output is None or tuple(self.output.shape) != shape:
            self.output = torch.empty(shape, dtype=torch.float32, device=self.device)
        capi.check(capi.lib().fbfftconv_tiled_update_output(
            t, _ptr(input), _ptr(self.weight), None if skipBias else _ptr(self.bias), _ptr(self.output),
            _stream(self.device)))
        return self.output

    def updateGradInput(self, input: torch.Tensor, gradOutput: torch.Tensor) -> torch.Tensor:
        self.timeSteps["updateGradInput"] += 1
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        t = self._prepare_tiled(input)
        if self.gradInput is None or self.gradInput.shape != input.shape:
            self.gradInput = torch.empty_like(input)
        capi.check(capi.lib().fbfftconv_tiled_update_grad_input(
            t, _ptr(gradOutput), _ptr(self.weight), _ptr(self.gradInput), _stream(self.device)))
        return self.gradInput

    def accGradParameters(self, input: torch.Tensor, gradOutput: torch.Tensor, scale=None,
                          skipBias: bool = False) -> None:
        self.timeSteps["accGradParameters"] += 1
        scale = 1.0 if scale is None else float(scale)
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        t = self._prepare_tiled(input)
        capi.check(capi.lib().fbfftconv_tiled_acc_grad_parameters(
            t, _ptr(input), _ptr(gradOutput), _ptr(self.gradWeight), None if skipBias else _ptr(self.gradBias),
            ctypes.c_float(scale), _stream(self.device)))

    def cleanupBuffers(self):
        if getattr(self, "_tiled", None) is not None:
            capi.lib().fbfftconv_tiled_destroy(self._tiled)  # destroys the untiled layer of the tiles with it
            self._tiled = None
            self._tiled_key = None
            self._handle = None
            self._handle_key = None

    def attachCommunicator(self, unique_id: bytes, rank: int, nranks: int):
        assert len(unique_id) == 128
        self._comm = (bytes(unique_id), int(rank), int(nranks))
        if self._tiled is not None:
            self._init_comm()
