"""World-size-2 checks of the multi-rank layout on CPU (gloo): the batch split, the
exchange of the communicator id, and the identity the GPU path relies on -- per-rank
outputs concatenate to the full output, per-rank weight/bias gradients sum to the full
gradient (what the all-reduce inside accGradParameters computes)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import oracle
    from fbcunn_b200.sharding import batch_slice, share_unique_id

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        uid = share_unique_id(dist, lambda: bytes(range(128)))
        assert uid == bytes(range(128))
        s = oracle.Shape(B=5, P=3, F=4, iH=9, iW=8, kH=3, kW=2, padH=1, padW=0)
        rng = np.random.default_rng(99)  # same data on every rank
        x = rng.standard_normal((s.B, s.P, s.iH, s.iW)).astype(np.float32)
        w = rng.standard_normal((s.F, s.P, s.kH, s.kW)).astype(np.float32)
        go = rng.standard_normal((s.B, s.F, s.oH, s.oW)).astype(np.float32)
        b0, b1 = batch_slice(s.B, rank, world)
        local = oracle.Shape(b1 - b0, s.P, s.F, s.iH, s.iW, s.kH, s.kW, s.padH, s.padW)
        out = oracle.update_output(local, x[b0:b1], w)
        gw = torch.from_numpy(oracle.acc_grad_weight(local, x[b0:b1], go[b0:b1], 0.5))
        gb = torch.from_numpy(oracle.acc_grad_bias(local, go[b0:b1], 0.5))
        dist.all_reduce(gw)
        dist.all_reduce(gb)
        gathered = [None] * world
        dist.all_gather_object(gathered, (b0, b1, out))
        if rank == 0:
            full = np.concatenate([g[2] for g in sorted(gathered, key=lambda g: g[0])], axis=0)
            np.testing.assert_allclose(full, oracle.update_output(s, x, w), rtol=0, atol=1e-12)
            np.testing.assert_allclose(gw.numpy(), oracle.acc_grad_weight(s, x, go, 0.5), rtol=1e-12, atol=1e-12)
            np.testing.assert_allclose(gb.numpy(), oracle.acc_grad_bias(s, go, 0.5), rtol=1e-12, atol=1e-12)
            assert [g[:2] for g in sorted(gathered, key=lambda g: g[0])] == [(0, 3), (3, 5)]
            with open(os.path.join(out_dir, "ok"), "w") as f:
                f.write("ok")
    finally:
        dist.destroy_process_group()


def test_batch_slice_covers_the_batch():
    from fbcunn_b200.sharding import batch_slice
    for B in (1, 2, 7, 16, 128):
        for world in (1, 2, 3, 4, 8):
            parts = [batch_slice(B, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            sizes = [b - a for a, b in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_slice(8, 2, 2)


def test_two_ranks_on_gloo(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(os.path.join(str(tmp_path), "ok"))
