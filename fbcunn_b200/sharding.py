"""Host-side helpers for the one-process-per-GPU layout of the convolution.

updateOutput and updateGradInput split the minibatch across ranks and exchange
nothing; accGradParameters sums its weight (and bias) gradient over ranks.  This is
what nn.DataParallel does in one process (fbcunn/DataParallel.lua:51-80 for the
split, :105-131 for the gradient combine), restated for torch.distributed ranks.
"""
from __future__ import annotations

from typing import Tuple


def batch_slice(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of rank's share of the batch: contiguous, sizes differ by at most one,
    earlier ranks take the larger shares (the split of nn.DataParallel's
    _distributeInput, fbcunn/DataParallel.lua:51-80, without its remainder restriction)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def share_unique_id(dist, make_id, device=None) -> bytes:
    """Rank 0 makes the 128-byte communicator id, every rank returns the same bytes.
    `dist` is torch.distributed (any backend), `make_id` a zero-argument callable."""
    import torch

    dev = device if device is not None else ("cuda" if dist.get_backend() == "nccl" else "cpu")
    buf = torch.zeros(128, dtype=torch.uint8, device=dev)
    if dist.get_rank() == 0:
        raw = make_id()
        assert len(raw) == 128
        buf.copy_(torch.frombuffer(bytearray(raw), dtype=torch.uint8))
    dist.broadcast(buf, 0)
    return bytes(buf.cpu().numpy().tobytes())
