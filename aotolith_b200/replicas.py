"""Serving the path on several GPUs: independent replicas, one process per GPU.

A batch-1 decode step of the static-cache path has no exchange step: every
request owns its cache and reads the whole weight set, so the path shards by
REQUEST, not by tensor. Each rank loads the same packed weights, takes a strided
share of the request stream and never talks to its peers on the data path. The
only collectives are the ones a measurement needs: a barrier on both sides of the
timed region, the maximum of the ranks' device times and the sum of their token
counts. They run on whichever backend the process group was created with (NCCL on
GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence, TypeVar

import torch

Item = TypeVar("Item")


def shard_indices(count: int, world: int, rank: int) -> range:
    """Indices of the requests rank ``rank`` of ``world`` serves: ``rank, rank + world, ...``.

    Strided rather than blocked so that a stream ordered by arrival time keeps
    every replica busy from the first request on.
    """

    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is not in a world of {world}")
    if count < 0:
        raise ValueError("count must be non-negative")
    return range(rank, count, world)


def shard(items: Sequence[Item], world: int, rank: int) -> list[Item]:
    """This rank's share of ``items`` (see :func:`shard_indices`)."""

    return [items[i] for i in shard_indices(len(items), world, rank)]


@dataclass(frozen=True)
class JobThroughput:
    """Whole-job figures: units of all ranks over the slowest rank's time."""

    units: float
    milliseconds: float
    world: int

    @property
    def per_second(self) -> float:
        return self.units / (self.milliseconds / 1e3) if self.milliseconds > 0 else 0.0


def job_throughput(local_units: float, local_ms: float, device: torch.device | None = None) -> JobThroughput:
    """Sum of the ranks' units and maximum of their times.

    Without an initialised process group this is the local pair. With one, every
    rank gets the same answer (two all-reduces on ``device``; pass the CUDA
    device under NCCL, nothing under gloo).
    """

    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return JobThroughput(float(local_units), float(local_ms), 1)
    units = torch.tensor([float(local_units)], dtype=torch.float64, device=device)
    slowest = torch.tensor([float(local_ms)], dtype=torch.float64, device=device)
    dist.all_reduce(units, op=dist.ReduceOp.SUM)
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    return JobThroughput(float(units.item()), float(slowest.item()), dist.get_world_size())


def gather_results(local: Sequence[tuple[int, list[int]]]) -> dict[int, list[int]]:
    """Collect ``(request index, generated tokens)`` pairs of all ranks on every rank."""

    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return dict(local)
    everyone: list = [None] * dist.get_world_size()
    dist.all_gather_object(everyone, list(local))
    merged: dict[int, list[int]] = {}
    for part in everyone:
        for index, tokens in part:
            if index in merged:
                raise RuntimeError(f"request {index} was served by two ranks")
            merged[index] = tokens
    return merged
