"""nn.SpatialConvolutionFFTTiled on the GPU against the CPU oracle: the three passes on images
cut into tiles (overlap-save), including images beyond the 128-pixel limit of the untiled
module.  Tolerance: max|x - ref| <= 1e-4 * max|ref| against the fp64 oracle, as for the untiled
passes (the reference's tiled tests use the same bound as its untiled ones,
test/test_SpatialConvolutionFFTTiled.lua).
"""
import numpy as np
import pytest
import torch

import oracle
from fbcunn_b200 import SpatialConvolutionFBFFT, SpatialConvolutionFFTTiled

pytestmark = pytest.mark.gpu
PASS_TOL = 1e-4

CASES = [
    # shape (B, P, F, iH, iW, kH, kW, padH, padW), tileH, tileW
    (oracle.Shape(2, 3, 4, 70, 61, 5, 4, 2, 1), 16, 16),
    (oracle.Shape(2, 3, 4, 70, 61, 5, 4, 2, 1), 32, 16),
    (oracle.Shape(3, 5, 2, 33, 40, 3, 3, 0, 0), 8, 8),
    (oracle.Shape(1, 2, 3, 150, 140, 3, 3, 1, 1), 32, 32),     # beyond the untiled limit
    (oracle.Shape(2, 8, 16, 40, 40, 7, 7, 3, 3), 32, 32),       # tensor-core contraction inside
    (oracle.Shape(2, 2, 2, 12, 12, 3, 3, 0, 0), 16, 16),        # tile larger than the image: one tile
]


def _rel(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def _data(s, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
    bound = 1.0 / np.sqrt(s.kH * s.kW * s.P)
    w = rng.uniform(-bound, bound, (s.F, s.P, s.kH, s.kW)).astype(np.float32)
    go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, s.F).astype(np.float32)
    return x, w, go, b


@pytest.mark.parametrize("idx", range(len(CASES)))
def test_tiled_passes_match_the_oracle(idx):
    s, th, tw = CASES[idx]
    x, w, go, b = _data(s, 300 + idx)
    m = SpatialConvolutionFFTTiled(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, tw, th)
    m.weight.copy_(torch.from_numpy(w))
    m.bias.copy_(torch.from_numpy(b))
    dx, dgo = torch.from_numpy(x).cuda(), torch.from_numpy(go).cuda()
    out = m.updateOutput(dx).cpu().numpy()
    gi = m.updateGradInput(dx, dgo).cpu().numpy()
    m.accGradParameters(dx, dgo, 0.6)
    assert out.shape == (s.B, s.F, s.oH, s.oW) and gi.shape == x.shape
    assert _rel(out, oracle.update_output(s, x, w, b)) <= PASS_TOL
    assert _rel(gi, oracle.update_grad_input(s, go, w)) <= PASS_TOL
    assert _rel(m.gradWeight.cpu().numpy(), oracle.acc_grad_weight(s, x, go, 0.6)) <= PASS_TOL
    assert _rel(m.gradBias.cpu().numpy(), oracle.acc_grad_bias(s, go, 0.6)) <= PASS_TOL


def test_tiled_agrees_with_untiled():
    s = oracle.Shape(4, 6, 5, 48, 52, 5, 5, 2, 2)
    x, w, go, b = _data(s, 77)
    dx, dgo = torch.from_numpy(x).cuda(), torch.from_numpy(go).cuda()
    outs = []
    for m in (SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH),
              SpatialConvolutionFFTTiled(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, 16, 16)):
        m.weight.copy_(torch.from_numpy(w))
        m.bias.copy_(torch.from_numpy(b))
        o = m.updateOutput(dx).clone()
        g = m.updateGradInput(dx, dgo).clone()
        m.accGradParameters(dx, dgo)
        outs.append((o, g, m.gradWeight.clone(), m.gradBias.clone()))
    for a, c in zip(*outs):
        assert float((a - c).abs().max()) <= 2e-5 * float(c.abs().max())


def test_untiled_module_refuses_what_the_tiled_one_takes():
    m = SpatialConvolutionFBFFT(1, 1, 3, 3)
    with pytest.raises(Exception):
        m.updateOutput(torch.zeros(1, 1, 150, 150, device="cuda"))
