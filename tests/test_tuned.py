"""fbnn.SpatialConvolution, the autotuning wrapper: candidate pruning and the choice among
timed candidates on the CPU (with an injected timer), and an end-to-end run on the GPU."""
import numpy as np
import pytest
import torch

import oracle
from fbcunn_b200 import SpatialConvolution
from fbcunn_b200.tuned import candidate_list


def _labels(*a):
    return [label for label, _ in candidate_list(*a, device="cpu")]


def test_candidates_follow_the_pruning_of_the_reference():
    # small image: untiled and both tile sizes (fbcunn/SpatialConvolution.lua:262-276, :281-305)
    assert _labels(4, 4, 3, 3, 1, 1, 40, 40) == [
        "FBFFT reuse=none", "FBFFT reuse=all", "FFTTiled 16x16 reuse=none", "FFTTiled 16x16 reuse=all",
        "FFTTiled 32x32 reuse=none", "FFTTiled 32x32 reuse=all"]
    # kernels above 9x9: 32-pixel tiles only (:306-311)
    assert _labels(4, 4, 11, 11, 0, 0, 100, 100) == [
        "FBFFT reuse=none", "FBFFT reuse=all", "FFTTiled 32x32 reuse=none", "FFTTiled 32x32 reuse=all"]
    # images beyond 128 pixels: tiled only
    assert all(l.startswith("FFTTiled") for l in _labels(4, 4, 3, 3, 0, 0, 200, 200))
    # an image that one tile covers is not tiled
    assert _labels(4, 4, 3, 3, 0, 0, 12, 12) == ["FBFFT reuse=none", "FBFFT reuse=all"]


def test_fastest_candidate_within_the_memory_limit_wins():
    cost = {"FBFFT reuse=none": ([3.0, 3.0, 3.0], 100), "FBFFT reuse=all": ([1.0, 1.0, 1.0], 900),
            "FFTTiled 16x16 reuse=none": ([2.0, 2.0, 2.0], 50), "FFTTiled 16x16 reuse=all": ([2.0, 2.5, 2.0], 60),
            "FFTTiled 32x32 reuse=none": ([4.0, 1.0, 1.5], 70), "FFTTiled 32x32 reuse=all": ([5.0, 5.0, 5.0], 80)}
    seen = []

    def timer(inst, x, go, scale, inference_only):
        label = [l for l, _ in candidate_list(4, 4, 3, 3, 1, 1, 40, 40, device="cpu")][len(seen)]
        seen.append(label)
        t, mem = cost[label]
        return (t[:1] + [0.0, 0.0] if inference_only else t), mem

    x = torch.zeros(2, 4, 40, 40)
    m = SpatialConvolution(4, 4, 3, 3, 1, 1, 1, 1, None, False, device="cpu", timer=timer)
    m._tune(x)
    assert m.bestLabel == "FBFFT reuse=all" and len(seen) == 6
    seen.clear()
    m = SpatialConvolution(4, 4, 3, 3, 1, 1, 1, 1, 500, False, device="cpu", timer=timer)
    m._tune(x)
    assert m.bestLabel == "FFTTiled 16x16 reuse=none"          # the 900-byte candidate is over the limit
    seen.clear()
    m = SpatialConvolution(4, 4, 3, 3, 1, 1, 1, 1, 500, True, device="cpu", timer=timer)
    m._tune(x)
    assert m.bestLabel == "FFTTiled 16x16 reuse=none"          # forward time only: 2.0 is the best within the limit
    assert m.bestModuleInst.weight is m.weight and m.bestModuleInst.gradWeight is m.gradWeight
    with pytest.raises(ValueError):
        SpatialConvolution(4, 4, 3, 3, 2, 2, device="cpu")


@pytest.mark.gpu
def test_tuned_module_runs_and_matches_the_oracle():
    s = oracle.Shape(4, 6, 8, 40, 36, 3, 3, 1, 1)
    rng = np.random.default_rng(5)
    x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
    go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
    m = SpatialConvolution(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH)
    w, b = m.weight.cpu().numpy(), m.bias.cpu().numpy()
    dx, dgo = torch.from_numpy(x).cuda(), torch.from_numpy(go).cuda()
    out = m.updateOutput(dx).cpu().numpy()
    assert len(m.timings) == 6 and m.bestLabel in m.timings
    gi = m.updateGradInput(dx, dgo).cpu().numpy()
    m.accGradParameters(dx, dgo, 1.0)

    def rel(a, ref):
        return float(np.abs(a - ref).max() / np.abs(ref).max())

    assert rel(out, oracle.update_output(s, x, w, b)) <= 1e-4
    assert rel(gi, oracle.update_grad_input(s, go, w)) <= 1e-4
    assert rel(m.gradWeight.cpu().numpy(), oracle.acc_grad_weight(s, x, go, 1.0)) <= 1e-4
    assert rel(m.gradBias.cpu().numpy(), oracle.acc_grad_bias(s, go, 1.0)) <= 1e-4
