"""Host-side helpers for running one engine per GPU: how queries are split over ranks and
how the per-rank counters are combined.  The walk itself never communicates."""
import numpy as np


def shard_range(n, rank, world):
    """Contiguous id range [lo, hi) of rank `rank` out of `world` for n queries."""
    if world < 1 or not 0 <= rank < world or n < 0:
        raise ValueError("bad shard arguments n=%r rank=%r world=%r" % (n, rank, world))
    return (rank * n) // world, ((rank + 1) * n) // world


def reduce_counters(dist, counters, times_ms, device=None):
    """Sum of integer counters and max of times over all ranks (identity when `dist` is None
    or not initialised).  `dist` is torch.distributed; works with nccl (device tensors) and
    gloo (host tensors)."""
    import torch
    c = torch.tensor([int(x) for x in counters], dtype=torch.int64, device=device)
    t = torch.tensor([float(x) for x in times_ms], dtype=torch.float64, device=device)
    if dist is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [int(x) for x in c.tolist()], [float(x) for x in t.tolist()]


def gather_rows(dist, rows, n_total, rank, world):
    """All ranks' result rows stacked in id order (gloo/nccl all_gather of padded shards)."""
    import torch
    D = rows.shape[1]
    per = max(shard_range(n_total, r, world)[1] - shard_range(n_total, r, world)[0] for r in range(world))
    pad = torch.full((per, D), -2, dtype=torch.int32)
    pad[: rows.shape[0]] = torch.as_tensor(np.ascontiguousarray(rows))
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad)
    parts = []
    for r in range(world):
        lo, hi = shard_range(n_total, r, world)
        parts.append(bufs[r][: hi - lo].numpy())
    return np.vstack(parts)
