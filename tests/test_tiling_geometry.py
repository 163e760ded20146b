"""Tile cutting and reassembly of SpatialConvolutionFFTTiled on the CPU: the native per-tile
convolution is replaced by a float64 torch stand-in (test infrastructure only), so what is
checked is the overlap-save / overlap-add index arithmetic around it."""
import pytest
import torch
import torch.nn.functional as F

from fbcunn_b200 import tiled


class _StandIn:
    """Unpadded per-tile convolution and its adjoint."""

    def __init__(self, weight):
        self.weight = weight
        self.calls = []

    def updateOutput(self, x, skipBias=False):
        self.calls.append(tuple(x.shape))
        return F.conv2d(x.double(), self.weight.double()).float()

    def updateGradInput(self, like, go):
        return F.conv_transpose2d(go.double(), self.weight.double()).float()


def _module(P, Fo, kH, kW, padU, padL, tH, tW):
    m = tiled.SpatialConvolutionFFTTiled.__new__(tiled.SpatialConvolutionFFTTiled)
    m.nInputPlane, m.nOutputPlane, m.kH, m.kW, m.padUp, m.padLeft = P, Fo, kH, kW, padU, padL
    m.tileSizeH, m.tileSizeW = tH, tW
    m.timeSteps = {"updateOutput": 0, "updateGradInput": 0, "accGradParameters": 0}
    g = torch.Generator().manual_seed(P * 100 + Fo)
    m.weight = torch.randn(Fo, P, kH, kW, generator=g)
    m.bias = torch.randn(Fo, generator=g)
    m._inner = _StandIn(m.weight)
    m._share = lambda: None
    m._check_input = lambda x: None
    m._check_grad_output = lambda a, b: None
    return m


@pytest.mark.parametrize("case", [
    (2, 3, 4, 70, 61, 5, 4, 2, 1, 16, 16),
    (1, 2, 2, 33, 40, 3, 3, 0, 0, 8, 8),
    (1, 1, 2, 150, 140, 3, 3, 1, 1, 32, 32),
    (2, 2, 2, 12, 12, 3, 3, 0, 0, 16, 16),
    (1, 2, 1, 20, 31, 7, 2, 3, 1, 16, 32),
    (1, 1, 1, 20, 20, 7, 7, 0, 0, 8, 8),      # tiles reach beyond their neighbours: the fold path
])
def test_tiles_reassemble_to_the_whole_convolution(case):
    B, P, Fo, iH, iW, kH, kW, padU, padL, tH, tW = case
    m = _module(P, Fo, kH, kW, padU, padL, tH, tW)
    x = torch.randn(B, P, iH, iW, generator=torch.Generator().manual_seed(1))
    out = m.updateOutput(x)
    ref = F.conv2d(x.double(), m.weight.double(), padding=(padU, padL)) + m.bias.view(1, -1, 1, 1).double()
    assert out.shape == ref.shape
    assert float((out - ref).abs().max()) <= 1e-4
    # every tile that went through the per-tile convolution has the tile's size
    (nb, p, th, tw), = set(m._inner.calls)
    assert p == P and th <= tH and tw <= tW and nb % B == 0
    go = torch.randn(ref.shape, generator=torch.Generator().manual_seed(2))
    gi = m.updateGradInput(x, go)
    ref_gi = F.conv_transpose2d(go.double(), m.weight.double(), padding=(padU, padL))
    assert gi.shape == x.shape
    assert float((gi - ref_gi).abs().max()) <= 1e-4
    # the disjoint gradOutput tiles carry every element exactly once
    geo = m._geometry(iH, iW)
    assert float(m._output_tiles(go, geo).double().sum() - go.double().sum()) == pytest.approx(0.0, abs=1e-6)
