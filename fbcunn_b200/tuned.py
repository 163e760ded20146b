"""fbnn.SpatialConvolution: the autotuning wrapper real models construct.

Mirrors fbcunn/SpatialConvolution.lua: on the first updateOutput it times the candidate
implementations on tensors of the caller's shape (:188-422), keeps the fastest one within the
allowed memory overhead and forwards every later call to it.  The candidates here are the
flavours of the native FFT path:

    SpatialConvolutionFBFFT       untiled (padded image up to 128 pixels), reuse none / all
    SpatialConvolutionFFTTiled    tiles of 16 or 32 pixels, reuse none / all

with the reference's pruning by kernel size (:281-312: 16- and 32-pixel tiles up to 9x9
kernels, 32-pixel tiles above).  The reference also times cudnn and can fall back to it; no
library convolution exists on this path, so a strided convolution, which no FFT candidate
serves, is an error here.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch

from . import capi
from .module import SpatialConvolutionFBFFT, memoryReuseAll, memoryReuseNone
from .tiled import SpatialConvolutionFFTTiled

Candidate = Tuple[str, Callable[[], SpatialConvolutionFBFFT]]


def candidate_list(nInputPlane, nOutputPlane, kW, kH, padLeft, padUp, iH, iW, **kw) -> List[Candidate]:
    """(label, constructor) of every implementation worth timing for this layer and image."""
    out: List[Candidate] = []
    args = (nInputPlane, nOutputPlane, kW, kH, 1, 1, padLeft, padUp)
    if max(iH + 2 * padUp, iW + 2 * padLeft, kH, kW) <= 128:
        for reuse in (memoryReuseNone, memoryReuseAll):
            out.append((f"FBFFT reuse={reuse}",
                        lambda reuse=reuse: SpatialConvolutionFBFFT(*args, reuse, **kw)))
    tiles = (16, 32) if (kH <= 9 and kW <= 9) else (32,)
    oH, oW = iH + 2 * padUp - kH + 1, iW + 2 * padLeft - kW + 1
    for t in tiles:
        if t < max(kH, kW) or (t - kH + 1 >= oH and t - kW + 1 >= oW):
            continue  # tile smaller than the kernel, or one tile would cover the image anyway
        for reuse in (memoryReuseNone, memoryReuseAll):
            out.append((f"FFTTiled {t}x{t} reuse={reuse}",
                        lambda t=t, reuse=reuse: SpatialConvolutionFFTTiled(*args, t, t, reuse, **kw)))
    return out


def time_module(m, input, gradOutput, scale, inference_only, iters=3):
    """Milliseconds per (updateOutput, updateGradInput, accGradParameters), CUDA events on the
    current stream, after one untimed round; and the bytes of device memory the module took."""
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()

    def run(which):
        if which == 0:
            m.updateOutput(input)
        elif which == 1:
            m.updateGradInput(input, gradOutput)
        else:
            m.accGradParameters(input, gradOutput, scale)

    passes = (0,) if inference_only else (0, 1, 2)
    times = [0.0, 0.0, 0.0]
    for which in passes:
        run(which)
    for which in passes:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            run(which)
        stop.record()
        stop.synchronize()
        times[which] = start.elapsed_time(stop) / iters
    # device memory the library allocated itself (torch does not see it)
    native = 0
    if getattr(m, "_tiled", None) is not None:
        native = int(capi.lib().fbfftconv_tiled_workspace_bytes(m._tiled))
    elif getattr(m, "_handle", None) is not None:
        native = int(capi.lib().fbfftconv_workspace_bytes(m._handle))
    return times, native + max(0, torch.cuda.memory_allocated() - before)


class SpatialConvolution:
    """fbnn.SpatialConvolution(nInputPlane, nOutputPlane, kW, kH, dW, dH, padLeft, padUp,
    maximalMemoryOverhead, inferenceOnly)."""

    reportLevel = 0

    def __init__(self, nInputPlane, nOutputPlane, kW, kH, dW=1, dH=1, padLeft=0, padUp=0,
                 maximalMemoryOverhead=None, inferenceOnly=False, *, device="cuda",
                 timer: Optional[Callable] = None, **kw):
        self.inputPlanes, self.outputPlanes = int(nInputPlane), int(nOutputPlane)
        self.kW, self.kH = int(kW), int(kH)
        self.dW, self.dH = int(dW or 1), int(dH or 1)
        self.padLeft, self.padUp = int(padLeft or 0), int(padUp or 0)
        if self.dW != 1 or self.dH != 1:
            raise ValueError("only stride-1 convolutions have an FFT implementation; no other path exists here")
        self.maximalMemoryOverhead = maximalMemoryOverhead
        self.inferenceOnly = bool(inferenceOnly)
        self.device = device
        self._kw = dict(kw, device=device)
        self._timer = timer or time_module
        self.bestModuleInst = None
        self.timings = {}
        # parameters live here until a winner adopts them (fbcunn/SpatialConvolution.lua:405-410)
        probe = SpatialConvolutionFBFFT(nInputPlane, nOutputPlane, kW, kH, 1, 1, padLeft, padUp, **self._kw)
        self.weight, self.bias = probe.weight, probe.bias
        self.gradWeight, self.gradBias = probe.gradWeight, probe.gradBias
        self.output = None
        self.gradInput = None

    # -- tuning ---------------------------------------------------------------------------
    def _tune(self, input):
        B, P, iH, iW = input.shape
        oH, oW = iH + 2 * self.padUp - self.kH + 1, iW + 2 * self.padLeft - self.kW + 1
        probe_in = torch.randn_like(input)
        probe_go = torch.randn((B, self.outputPlanes, oH, oW), dtype=torch.float32, device=input.device)
        best, best_time, best_label = None, float("inf"), None
        for label, make in candidate_list(self.inputPlanes, self.outputPlanes, self.kW, self.kH, self.padLeft,
                                          self.padUp, iH, iW, **self._kw):
            inst = make()
            times, mem = self._timer(inst, probe_in, probe_go, 0.5, self.inferenceOnly)
            self.timings[label] = {"ms": times, "memory": mem}
            total = sum(times)
            too_big = self.maximalMemoryOverhead is not None and mem > self.maximalMemoryOverhead
            if total < best_time and not too_big:
                if best is not None:
                    best.cleanupBuffers()
                best, best_time, best_label = inst, total, label
            else:
                inst.cleanupBuffers()
        if best is None:
            raise RuntimeError("no FFT implementation fits this layer within the allowed memory overhead")
        if self.reportLevel >= 1:
            print(f"Best FFT: {best_time:.3f} ms  {best_label}")
        if self.reportLevel >= 3:
            print("Timings:", self.timings)
        self.bestLabel = best_label
        self.bestModuleInst = best
        self._adopt()

    def _adopt(self):
        inst = self.bestModuleInst
        inst.weight, inst.bias = self.weight, self.bias
        inst.gradWeight, inst.gradBias = self.gradWeight, self.gradBias

    # -- nn.Module surface ----------------------------------------------------------------
    def updateOutput(self, input):
        assert input.dim() == 4, "Only supports 4-D tensors atm"
        if self.bestModuleInst is None:
            self._tune(input)
        self._adopt()
        self.output = self.bestModuleInst.updateOutput(input)
        return self.output

    def updateGradInput(self, input, gradOutput):
        assert self.bestModuleInst is not None, "updateOutput runs first (it tunes)"
        assert not self.inferenceOnly, "module was built for inference only"
        self.gradInput = self.bestModuleInst.updateGradInput(input, gradOutput)
        return self.gradInput

    def accGradParameters(self, input, gradOutput, scale=None):
        assert self.bestModuleInst is not None, "updateOutput runs first (it tunes)"
        assert not self.inferenceOnly, "module was built for inference only"
        self.bestModuleInst.accGradParameters(input, gradOutput, scale)

    def forward(self, input):
        return self.updateOutput(input)

    def backward(self, input, gradOutput, scale=None):
        self.updateGradInput(input, gradOutput)
        self.accGradParameters(input, gradOutput, scale)
        return self.gradInput

    def zeroGradParameters(self):
        self.gradWeight.zero_()
        self.gradBias.zero_()

    def cleanupBuffers(self):
        if self.bestModuleInst is not None:
            self.bestModuleInst.cleanupBuffers()

