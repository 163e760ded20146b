"""The communicator path of accGradParameters on the GPU, against the CPU oracle.

With a communicator attached the weight and bias gradients are summed over ranks
inside accGradParameters (what nn.DataParallel's gradient combine does for the
reference module, fbcunn/DataParallel.lua:105-131): either the gradWeight spectrum
before the inverse transform or gradWeight after it.  A one-rank communicator runs
the whole path on a single GPU; the 2-, 3-, 4- and 8-rank cases need that many GPUs and
are skipped otherwise.  Tolerance: max|x - ref| <= 1e-4 * max|ref| against the fp64 oracle.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import oracle
from fbcunn_b200 import SpatialConvolutionFBFFT

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PASS_TOL = 1e-4

SHAPES = [
    oracle.Shape(B=6, P=5, F=7, iH=12, iW=11, kH=3, kW=4, padH=1, padW=0),      # CUDA-core contraction, N=16
    oracle.Shape(B=8, P=16, F=24, iH=20, iW=20, kH=5, kW=5, padH=0, padW=0),    # tensor-core contraction, N=32
    oracle.Shape(B=4, P=3, F=8, iH=40, iW=36, kH=7, kW=7, padH=0, padW=0),      # plane-major streaming, N=64
]


def _rel(a, ref):
    return float(np.abs(np.asarray(a, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def _data(s, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
    go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
    return x, go


def _grads(s, x, go, scale, allreduce, comm, accumulate=False, device="cuda", exchange="auto", status=None):
    m = SpatialConvolutionFBFFT(s.P, s.F, s.kW, s.kH, 1, 1, s.padW, s.padH, device=device,
                                allreduce=allreduce, accumulate=accumulate, exchange=exchange)
    if comm is not None:
        m.attachCommunicator(*comm)
    dx = torch.from_numpy(x).to(device)
    dgo = torch.from_numpy(go).to(device)
    if accumulate:
        m.gradWeight.fill_(1.0)
        m.gradBias.fill_(2.0)
    m.accGradParameters(dx, dgo, scale)
    m.accGradParameters(dx, dgo, scale)  # a second call: the exchange's buffers and epochs must be reusable
    if accumulate:  # two calls added twice
        m.gradWeight.sub_(1.0).div_(2.0).add_(1.0)
        m.gradBias.sub_(2.0).div_(2.0).add_(2.0)
    torch.cuda.synchronize()
    if status is not None:
        status.append(m.peerExchangeStatus())
    return m.gradWeight.cpu().numpy(), m.gradBias.cpu().numpy()


@pytest.mark.parametrize("allreduce", ["spectrum", "spatial"])
@pytest.mark.parametrize("idx", range(len(SHAPES)))
def test_one_rank_communicator(idx, allreduce):
    s = SHAPES[idx]
    x, go = _data(s, 40 + idx)
    uid = SpatialConvolutionFBFFT.makeUniqueId()
    gw, gb = _grads(s, x, go, 0.5, allreduce, (uid, 0, 1))
    assert _rel(gw, oracle.acc_grad_weight(s, x, go, 0.5)) <= PASS_TOL
    assert _rel(gb, oracle.acc_grad_bias(s, go, 0.5)) <= PASS_TOL
    # the accumulating form adds the summed gradient to what is already there
    gw2, gb2 = _grads(s, x, go, 0.5, allreduce, (uid, 0, 1), accumulate=True)
    assert _rel(gw2, oracle.acc_grad_weight(s, x, go, 0.5) + 1.0) <= PASS_TOL
    assert _rel(gb2, oracle.acc_grad_bias(s, go, 0.5) + 2.0) <= PASS_TOL


def _free_port():
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    return port


# Shapes for the ranks: every exchange of accGradParameters is reached --
#   plane-major, filters divisible by the ranks   -> reduce-scatter by filters + all-gather
#   plane-major, filters not divisible             -> all-reduce of the whole spectrum
#   bin-major, bins divisible by the ranks         -> reduce-scatter by bin range + all-reduce of partial transforms
#   bin-major, bins not divisible (3 ranks: N = 16 has 144 bins, N = 32 has 544)  -> all-reduce of the whole spectrum
RANK_SHAPES = [
    oracle.Shape(B=8, P=5, F=7, iH=12, iW=11, kH=3, kW=4, padH=1, padW=0),      # bin-major, CUDA-core contraction, N=16
    oracle.Shape(B=16, P=16, F=24, iH=20, iW=20, kH=5, kW=5, padH=0, padW=0),   # bin-major, tensor cores, N=32
    oracle.Shape(B=8, P=3, F=8, iH=40, iW=36, kH=7, kW=7, padH=0, padW=0),      # plane-major, F = 8
    oracle.Shape(B=9, P=2, F=7, iH=33, iW=40, kH=5, kW=3, padH=1, padW=1),      # plane-major, F = 7, ragged batch split
]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from fbcunn_b200 import capi
    from fbcunn_b200.sharding import batch_slice, share_unique_id

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        uid = share_unique_id(dist, SpatialConvolutionFBFFT.makeUniqueId, device="cpu")
        worst, cases, status = 0.0, 0, []
        for idx, s in enumerate(RANK_SHAPES):
            x, go = _data(s, 70 + idx)  # same on every rank
            b0, b1 = batch_slice(s.B, rank, world)
            local = oracle.Shape(b1 - b0, s.P, s.F, s.iH, s.iW, s.kH, s.kW, s.padH, s.padW)
            ref_w = oracle.acc_grad_weight(s, x, go, 2.0)
            ref_b = oracle.acc_grad_bias(s, go, 2.0)
            for exchange in ("auto", "nccl"):
                for allreduce in ("spectrum", "spatial"):
                    for accumulate in (False, True):
                        gw, gb = _grads(local, np.ascontiguousarray(x[b0:b1]), np.ascontiguousarray(go[b0:b1]), 2.0,
                                        allreduce, (uid, rank, world), accumulate=accumulate, device=f"cuda:{rank}",
                                        exchange=exchange, status=status)
                        worst = max(worst, _rel(gw, ref_w + (1.0 if accumulate else 0.0)),
                                    _rel(gb, ref_b + (2.0 if accumulate else 0.0)))
                        cases += 1
        import gc
        gc.collect()  # the modules detach from the communicator before it is shut down
        rc = capi.lib().fbfftconv_comm_shutdown()
        with open(os.path.join(out_dir, f"rank{rank}"), "w") as f:
            f.write(repr((worst, cases, rc, status)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_ranks_sum_the_gradient(tmp_path, world):
    """Every rank ends with the gradient of the whole batch, as the reference's data-parallel
    test asserts of its replicas (test/test_DataParallel.lua:73-159)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    results = [eval(open(tmp_path / f"rank{rank}").read()) for rank in range(world)]
    for rank, (worst, cases, rc, status) in enumerate(results):
        assert cases == 8 * len(RANK_SHAPES)
        assert rc == 0, f"rank {rank}: communicator still attached at shutdown"
        assert worst <= PASS_TOL, f"rank {rank}: {worst}"
        assert all(st in (0, 1) for st in status), f"rank {rank}: a wait of the peer exchange gave up: {status}"
        assert status == results[0][3], "every rank must make the same choice of exchange"
        # "nccl" handles never use peer memory; "auto" handles do on a box whose GPUs can map one another
        per_shape = 8
        for i, st in enumerate(status):
            if (i % per_shape) >= per_shape // 2:
                assert st == 0
    over_peers = sum(results[0][3])
    print(f"world {world}: {8 * len(RANK_SHAPES)} cases per rank, {over_peers} of them summed over peer memory, "
          f"worst relative error {max(r[0] for r in results):.2e}")
