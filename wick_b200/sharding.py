"""Host-side logic for running the path on several GPUs of one node.

wick serves independent sequences (one Session per conversation, wick/src/session.rs:303-420): a
sequence's KV cache and conv state never leave the device that decodes it, so the path shards by
sequence with one process per GPU and NO data-path collective.  The only exchanges are host-side
bookkeeping: a barrier around the timed region, the maximum of the per-rank device times and the
sum of the per-rank token counts.  These helpers work on any torch.distributed backend (nccl on
GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch
import torch.distributed as dist


def shard_sequences(n_sequences: int, world: int, rank: int) -> List[int]:
    """Indices of the sequences rank `rank` decodes: round-robin, so any prefix of the request
    queue is spread evenly and every index lands on exactly one rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return list(range(rank, n_sequences, world))


def prompt_seed(base_seed: int, sequence_index: int) -> int:
    """Seed of a sequence's synthetic prompt: distinct per sequence, independent of the world size,
    so the same sequence gets the same prompt whichever rank it lands on."""
    return base_seed + sequence_index


@dataclass
class JobTotals:
    tokens: int          # tokens all ranks produced
    seconds: float       # slowest rank's device time
    per_rank_tokens: List[int]

    @property
    def tokens_per_second(self) -> float:
        return self.tokens / self.seconds if self.seconds > 0 else float("nan")


def _device_for_backend() -> torch.device:
    if dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def job_totals(local_tokens: int, local_seconds: float) -> JobTotals:
    """Whole-job throughput figures: tokens summed over ranks, time = max over ranks."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return JobTotals(local_tokens, local_seconds, [local_tokens])
    dev = _device_for_backend()
    world = dist.get_world_size()
    tok = torch.zeros(world, dtype=torch.int64, device=dev)
    tok[dist.get_rank()] = local_tokens
    dist.all_reduce(tok, op=dist.ReduceOp.SUM)
    sec = torch.tensor([local_seconds], dtype=torch.float64, device=dev)
    dist.all_reduce(sec, op=dist.ReduceOp.MAX)
    per_rank = [int(v) for v in tok.tolist()]
    return JobTotals(sum(per_rank), float(sec.item()), per_rank)


def gather_token_streams(local: Sequence[Sequence[int]], local_indices: Sequence[int], n_sequences: int):
    """Collect every rank's generated sequences on all ranks, ordered by sequence index (used to
    check that sharding does not change any sequence's tokens)."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        out = [None] * n_sequences
        for i, s in zip(local_indices, local):
            out[i] = list(s)
        return out
    payload = [(int(i), [int(t) for t in s]) for i, s in zip(local_indices, local)]
    gathered = [None] * dist.get_world_size()
    dist.all_gather_object(gathered, payload)
    out = [None] * n_sequences
    for part in gathered:
        for i, s in part:
            if out[i] is not None:
                raise RuntimeError(f"sequence {i} was decoded by two ranks")
            out[i] = s
    return out
