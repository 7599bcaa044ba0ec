"""Replica data parallelism over independent observations (one process per GPU).

PI0.5 observations share nothing — the KV cache is per observation — so a global batch is
cut into contiguous shards, one per rank, each rank replays its own captured graph on its
own weight replica, and no collective runs on the data path. The only communication is an
optional gather of the finished action chunks (and of timings) after the timed region,
over whatever torch.distributed backend the launcher initialised (NCCL on GPUs, gloo in
the CPU tests). The reference has no multi-device code at all (every entry point opens
device 0: crates/apxinf-cuda/src/context.rs:39-57); this module is the added scale-out.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Sequence, Tuple

import numpy as np


@dataclass(frozen=True)
class Shard:
    rank: int
    start: int
    stop: int

    @property
    def size(self) -> int:
        return self.stop - self.start


def shard_bounds(global_batch: int, world: int) -> List[Shard]:
    """Contiguous shards, sizes differing by at most one (the first `global % world` ranks
    take the extra observation). An empty global batch gives empty shards."""
    if global_batch < 0 or world <= 0:
        raise ValueError(f"bad sharding request: batch {global_batch}, world {world}")
    base, extra = divmod(global_batch, world)
    shards, cursor = [], 0
    for rank in range(world):
        size = base + (1 if rank < extra else 0)
        shards.append(Shard(rank, cursor, cursor + size))
        cursor += size
    return shards


def run_sharded(infer: Callable[[np.ndarray, np.ndarray, np.ndarray], np.ndarray],
                images: np.ndarray, tokens: np.ndarray, noise: np.ndarray, rank: int, world: int,
                gather: bool = True, dist=None) -> Tuple[np.ndarray, Shard]:
    """Runs `infer` on this rank's shard; with `gather`, every rank returns the whole
    [global_batch, H, D] result in observation order. `infer` maps a shard's host arrays to
    its action chunks (e.g. CapturedGraph.infer_host of a graph captured for that shard size)."""
    shard = shard_bounds(images.shape[0], world)[rank]
    sl = slice(shard.start, shard.stop)
    local = infer(images[sl], tokens[sl], noise[sl]) if shard.size > 0 else None
    if not gather or world == 1:
        return local, shard
    import torch
    dist = dist or __import__("torch.distributed", fromlist=["distributed"])
    pieces: List = [None] * world
    dist.all_gather_object(pieces, None if local is None else np.ascontiguousarray(local))
    present = [p for p in pieces if p is not None]
    return (np.concatenate(present, axis=0) if present else None), shard
