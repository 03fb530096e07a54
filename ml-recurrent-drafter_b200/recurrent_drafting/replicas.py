"""Data-parallel decoding across the GPUs of one box: one process per GPU, a full model replica in
each, every rank decoding its own slice of the requests with no collective on the decode path.
The reference has no multi-GPU inference code of its own (its benchmark scripts start one
independent process per GPU, recurrent_drafting/benchmark/perf_wrt_candidates/run.bash:28-50); the
helpers here are the only places where ranks talk: splitting the batch, and one final gather of
the generated tokens and per-rank statistics (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from dataclasses import dataclass
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
    # an all-gather (a collective on the channels the process group already uses) rather than a gather, whose
    # point-to-point connections NCCL sets up lazily at first use: the matrices are a few hundred KB
    bucket = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bucket, padded, group=group)
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



@dataclass
class ShardedResult:
    """What generate_sharded() returns on every rank."""

    tokens: Optional[torch.Tensor]  # rank `dst` only: (n_requests, length) int64, rows in request order, left-padded
    generated_local: int  # tokens this rank generated for its rows (the first token, from the prefill, included)
    steps_local: int  # decode steps this rank ran
    d2h_bytes: int  # bytes copied to host_sink


def _left_pads(tokens: torch.Tensor, pad_id: int) -> torch.Tensor:
    return torch.sum(torch.cumprod(torch.eq(tokens, pad_id).to(torch.int64), dim=-1), dim=-1)


def generate_sharded(model, input_ids_all: torch.Tensor, max_length: int, beam_shape, sampling_args, special_tokens,
                     device=None, max_steps: Optional[int] = None, host_sink: Optional[torch.Tensor] = None, dst: int = 0,
                     group=None, ledger=None) -> ShardedResult:
    """One batch of requests in, one token matrix out, on however many ranks the process group has.

    Every rank is given the same (n_requests, prompt_len) int64 matrix (host or device memory), decodes
    the rows shard_bounds() assigns to it with `model.generate` until max_length (or for max_steps
    decode steps), and rank `dst` receives all rows back in request order.  The only communication is
    the final gather.  Without an initialised process group the call runs as a single rank.  The
    reference spreads requests over GPUs by starting one process per GPU from a shell script
    (recurrent_drafting/benchmark/perf_wrt_candidates/run.bash:28-50); this is that, as one call.

    host_sink, if given, is a pinned (rows, >= max_length + 1) int64 host tensor that receives every
    yielded matrix (the per-step read-back a serving loop does)."""
    from . import stats

    if dist.is_available() and dist.is_initialized():
        rank, world = dist.get_rank(group), dist.get_world_size(group)
    else:
        rank, world = 0, 1
    lo, hi = shard_bounds(input_ids_all.shape[0], rank, world)
    local = input_ids_all[lo:hi]
    if device is not None:
        local = local.to(device, non_blocking=True)
    pad = int(special_tokens.pad)
    out, steps, d2h = None, 0, 0
    if hi > lo:
        gen = model.generate(ledger if ledger is not None else stats.Ledger(), local, max_length, beam_shape, sampling_args,
                             special_tokens)
        try:
            for out in gen:
                steps += 1
                if host_sink is not None:
                    host_sink[: out.shape[0], : out.shape[1]].copy_(out, non_blocking=True)
                    d2h += out.numel() * out.element_size()
                    if out.is_cuda:
                        torch.cuda.current_stream(out.device).synchronize()
                if max_steps is not None and steps >= max_steps:
                    break
        finally:
            gen.close()
    if out is None:  # a rank without rows, or max_length already reached by the prompt
        out = local
    generated = int(((out.shape[1] - _left_pads(out, pad)) - (local.shape[1] - _left_pads(local, pad))).sum()) if hi > lo else 0
    if world == 1:
        return ShardedResult(out, generated, steps, d2h)
    parts = gather_tokens(out, pad, dst=dst, group=group)
    tokens = torch.cat(parts, dim=0) if parts is not None else None
    return ShardedResult(tokens, generated, steps, d2h)
