"""Data-parallel decoding across the GPUs of one box: one process per GPU, a full model replica in
each, every rank decoding its own slice of the requests with no collective on the decode path.
The reference has no multi-GPU inference code of its own (its benchmark scripts start one
independent process per GPU, recurrent_drafting/benchmark/perf_wrt_candidates/run.bash:28-50); the
helpers here are the only places where ranks talk: splitting the batch, and one final gather of
the generated tokens and per-rank statistics (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_requests: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous slice [lo, hi) of the request batch decoded by `rank`; the first
    n_requests % world_size ranks take one more request."""
    base, extra = divmod(n_requests, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_tokens(tokens: torch.Tensor, pad_id: int, dst: int = 0, group=None) -> Optional[List[torch.Tensor]]:
    """Gathers every rank's (rows, length) int64 token matrix on rank `dst`.  Ranks may hold different
    numbers of rows and different lengths (acceptance differs per request): shapes are exchanged
    first, matrices are left-padded with pad_id to the longest length, and rank `dst` gets back the
    list of unpadded-in-rows matrices in rank order.  Other ranks get None."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shape = torch.tensor(list(tokens.shape), dtype=torch.int64, device=tokens.device)
    shapes = [torch.empty_like(shape) for _ in range(world)]
    dist.all_gather(shapes, shape, group=group)
    max_rows = int(max(s[0] for s in shapes))
    max_len = int(max(s[1] for s in shapes))
    padded = torch.full((max_rows, max_len), pad_id, dtype=torch.int64, device=tokens.device)
    if tokens.numel():
        padded[: tokens.shape[0], max_len - tokens.shape[1] :] = tokens
    bucket = [torch.empty_like(padded) for _ in range(world)] if rank == dst else None
    dist.gather(padded, bucket, dst=dst, group=group)
    if rank != dst:
        return None
    return [b[: int(s[0])] for b, s in zip(bucket, shapes)]


def reduce_stats(elapsed_ms: float, generated_tokens: float, accepted_tokens: float, device, group=None) -> Tuple[float, float, float]:
    """Whole-job figures from per-rank ones: the slowest rank's time (MAX) and the summed token
    counts (SUM).  Returned on every rank."""
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
    n = torch.tensor([generated_tokens, accepted_tokens], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
    return float(t[0]), float(n[0]), float(n[1])
