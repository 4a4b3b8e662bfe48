"""Data-parallel sharding of decode streams over GPUs: replicated weights, independent streams, no
collective on the data path. The only communication is the control-plane reduction that turns
per-rank timings into one whole-job number (max time over ranks, sum of work)."""
from __future__ import annotations


def shard_streams(total_streams: int, world_size: int, rank: int) -> tuple[int, int]:
    """(first stream, stream count) owned by `rank`: contiguous, disjoint, covering; the first
    `total % world` ranks take one extra stream when the split is ragged."""
    if world_size < 1 or not 0 <= rank < world_size or total_streams < 0:
        raise ValueError("invalid shard request")
    base, extra = divmod(total_streams, world_size)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def whole_job_rate(units_local: float, seconds_local: float, dist=None, device=None) -> tuple[float, float, float]:
    """(rate, total units, slowest seconds) over all ranks: units are summed, time is the maximum.
    With `dist` None (single process) the local numbers are returned."""
    import torch
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return units_local / seconds_local, units_local, seconds_local
    units = torch.tensor([units_local], dtype=torch.float64, device=device)
    seconds = torch.tensor([seconds_local], dtype=torch.float64, device=device)
    dist.all_reduce(units, op=dist.ReduceOp.SUM)
    dist.all_reduce(seconds, op=dist.ReduceOp.MAX)
    return float(units.item() / seconds.item()), float(units.item()), float(seconds.item())
