"""Multi-GPU execution: independent event streams are the shard.

Nothing is shared between streams -- every reservoir, mask and tile list belongs to one stream and the weights are
read-only -- so stream s runs on rank s mod world with replicated weights and the data path has no collective.
``torch.distributed`` is used only to agree on the timing: a barrier around the timed region and a MAX over ranks
of the measured time (the job is as slow as its slowest rank)."""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def streams_of_rank(n_streams: int, world: int, rank: int) -> List[int]:
    """Global stream ids owned by ``rank`` (round-robin, as even as possible)."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    return list(range(rank, n_streams, world))


def job_throughput(local_steps: int, local_seconds: float, device=None) -> Tuple[float, int, float]:
    """(timesteps per second of the whole job, total stream-timesteps, seconds of the slowest rank).

    Every rank passes the stream-timesteps it processed and its own device-measured time."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([local_seconds], dtype=torch.float64, device=device)
        n = torch.tensor([local_steps], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
        secs, total = float(t.item()), int(n.item())
    else:
        secs, total = float(local_seconds), int(local_steps)
    return total / secs, total, secs
