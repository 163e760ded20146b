"""nn.SpatialConvolutionFFTTiled: the FFT convolution on tiles of the image.

Mirrors the reference's tiled module (fbcunn/SpatialConvolutionFFTTiled.lua:265-365 for the
constructor, :489-563 / :601-683 / :724-802 for the three passes): the output is cut into
disjoint tiles of (tileSize - k + 1) pixels, each of which depends on an input tile of
tileSize pixels (overlap-save), so the transform size stays at tileSize whatever the image
size -- which also lifts the 128-pixel limit of the untiled module.

Here the tiles of one image are laid out as extra batch entries and go through the
untiled native path in one call per pass:

    updateOutput        input tiles (overlapping)  -> output tiles (disjoint)
    updateGradInput     gradOutput tiles (disjoint) -> gradInput tiles, overlap-added
    accGradParameters   the sum over the batch inside the contraction is also the sum
                        over tiles, so gradWeight / gradBias come out complete

Cutting and reassembling the tiles is data movement only and is done with torch copy
kernels (unfold / fold); all arithmetic is the native library's.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .module import SpatialConvolutionFBFFT


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
        # the tiles run through an unpadded module that shares this module's parameters
        self._inner = SpatialConvolutionFBFFT(nInputPlane, nOutputPlane, kW, kH, 1, 1, 0, 0,
                                              memoryReusePolicy, numCudaStreams, **kw)
        self._share()

    def _share(self):
        inner = self._inner
        inner.weight, inner.bias = self.weight, self.bias
        inner.gradWeight, inner.gradBias = self.gradWeight, self.gradBias

    # -- tiling geometry ---------------------------------------------------------------
    def _geometry(self, iH, iW):
        oH = iH + 2 * self.padUp - self.kH + 1
        oW = iW + 2 * self.padLeft - self.kW + 1
        assert oH > 0 and oW > 0, "kernel larger than the padded input"
        tH, tW = min(self.tileSizeH, iH + 2 * self.padUp), min(self.tileSizeW, iW + 2 * self.padLeft)
        sH, sW = tH - self.kH + 1, tW - self.kW + 1          # output tile = step of the input tiles
        nH, nW = -(-oH // sH), -(-oW // sW)                   # tiles per image
        pH, pW = (nH - 1) * sH + tH, (nW - 1) * sW + tW      # padded input extent the tiles cover
        return oH, oW, tH, tW, sH, sW, nH, nW, pH, pW

    def _input_tiles(self, input, geo):
        """(B, P, iH, iW) -> (B * nH * nW, P, tH, tW), zero outside the image."""
        oH, oW, tH, tW, sH, sW, nH, nW, pH, pW = geo
        B, P, iH, iW = input.shape
        padded = F.pad(input, (self.padLeft, pW - iW - self.padLeft, self.padUp, pH - iH - self.padUp))
        t = padded.unfold(2, tH, sH).unfold(3, tW, sW)       # B, P, nH, nW, tH, tW
        return t.permute(0, 2, 3, 1, 4, 5).reshape(B * nH * nW, P, tH, tW).contiguous()

    def _output_tiles(self, grad_output, geo):
        """(B, F, oH, oW) -> (B * nH * nW, F, sH, sW), zero outside the image."""
        oH, oW, tH, tW, sH, sW, nH, nW, pH, pW = geo
        B, Fo = grad_output.shape[:2]
        padded = F.pad(grad_output, (0, nW * sW - oW, 0, nH * sH - oH))
        t = padded.reshape(B, Fo, nH, sH, nW, sW).permute(0, 2, 4, 1, 3, 5)
        return t.reshape(B * nH * nW, Fo, sH, sW).contiguous()

    # -- passes ------------------------------------------------------------------------
    def updateOutput(self, input: torch.Tensor, skipBias: bool = False) -> torch.Tensor:
        self.timeSteps["updateOutput"] += 1
        self._check_input(input)
        self._share()
        geo = self._geometry(input.shape[2], input.shape[3])
        oH, oW, tH, tW, sH, sW, nH, nW, pH, pW = geo
        B = input.shape[0]
        tiles = self._inner.updateOutput(self._input_tiles(input, geo), skipBias=True)
        out = tiles.reshape(B, nH, nW, self.nOutputPlane, sH, sW).permute(0, 3, 1, 4, 2, 5)
        out = out.reshape(B, self.nOutputPlane, nH * sH, nW * sW)[:, :, :oH, :oW]
        # the bias goes on once, at the very end (fbcunn/SpatialConvolutionFFTTiled.lua:541-544)
        self.output = out.contiguous() if skipBias else out + self.bias.view(1, -1, 1, 1)
        return self.output

    def updateGradInput(self, input: torch.Tensor, gradOutput: torch.Tensor) -> torch.Tensor:
        self.timeSteps["updateGradInput"] += 1
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        self._share()
        B, P, iH, iW = input.shape
        geo = self._geometry(iH, iW)
        oH, oW, tH, tW, sH, sW, nH, nW, pH, pW = geo
        like = torch.empty((B * nH * nW, P, tH, tW), dtype=torch.float32, device=input.device)
        gi = self._inner.updateGradInput(like, self._output_tiles(gradOutput, geo))   # B*nT, P, tH, tW
        full = self._overlap_add(gi, B, P, geo)
        self.gradInput = full[:, :, self.padUp:self.padUp + iH, self.padLeft:self.padLeft + iW].contiguous()
        return self.gradInput

    @staticmethod
    def _overlap_add(gi, B, P, geo):
        """Sum of the gradInput tiles (B * nH * nW, P, tH, tW) at their places, steps (sH, sW)."""
        oH, oW, tH, tW, sH, sW, nH, nW, pH, pW = geo
        eh, ew = tH - sH, tW - sW                                 # rows / columns shared with the next tile
        if eh > sH or ew > sW:                                    # a tile reaches beyond its neighbour
            cols = gi.reshape(B, nH * nW, P * tH * tW).transpose(1, 2)
            return F.fold(cols, (pH, pW), (tH, tW), stride=(sH, sW))
        # a tile = its own block plus the strips it shares with the right / lower / diagonal
        # neighbour: four strided adds instead of a scatter
        full = gi.new_zeros((B, P, (nH + 1) * sH, (nW + 1) * sW))
        blocks = full.unflatten(2, (nH + 1, sH)).unflatten(4, (nW + 1, sW))  # B, P, nH+1, sH, nW+1, sW (a view)
        t = gi.reshape(B, nH, nW, P, tH, tW).permute(0, 3, 1, 4, 2, 5)       # B, P, nH, tH, nW, tW
        blocks[:, :, :nH, :, :nW, :] = t[:, :, :, :sH, :, :sW]
        if eh:
            blocks[:, :, 1:, :eh, :nW, :] += t[:, :, :, sH:, :, :sW]
        if ew:
            blocks[:, :, :nH, :, 1:, :ew] += t[:, :, :, :sH, :, sW:]
        if eh and ew:
            blocks[:, :, 1:, :eh, 1:, :ew] += t[:, :, :, sH:, :, sW:]
        return full

    def accGradParameters(self, input: torch.Tensor, gradOutput: torch.Tensor, scale=None,
                          skipBias: bool = False) -> None:
        self.timeSteps["accGradParameters"] += 1
        self._check_input(input)
        self._check_grad_output(input, gradOutput)
        self._share()
        geo = self._geometry(input.shape[2], input.shape[3])
        self._inner.accGradParameters(self._input_tiles(input, geo), self._output_tiles(gradOutput, geo),
                                      scale, skipBias=skipBias)

    def cleanupBuffers(self):
        super().cleanupBuffers()
        inner = getattr(self, "_inner", None)
        if inner is not None:
            inner.cleanupBuffers()

    def attachCommunicator(self, unique_id: bytes, rank: int, nranks: int):
        self._inner.attachCommunicator(unique_id, rank, nranks)
