"""Feature sharding across the GPUs of one node (one process per GPU).

Rank ``r`` of ``world`` owns the contiguous block of features
``[r * block, min(F, (r + 1) * block))`` with ``block = ceil(F / world)``; feature ``f`` sits
at local row ``f - r * block``.  (Contiguous blocks, not a modulo deal, so that a rank's columns
are one strip of every row of the caller's row-major matrix and can be brought to the device
with a single strided copy.)  Every rank keeps the row state (targets, predictions, gradients,
row -> node map) replicated and runs the same host control flow with the same seed, so the
per-depth feature subsets agree without communication.
"""

from __future__ import annotations

import numpy as np


def block_size(n_features: int, world: int) -> int:
    return (int(n_features) + max(world, 1) - 1) // max(world, 1)


def owned_range(n_features: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of the global feature ids rank ``rank`` holds."""
    if world <= 1:
        return 0, int(n_features)
    blk = block_size(n_features, world)
    return min(n_features, rank * blk), min(n_features, (rank + 1) * blk)


def feature_map(n_features: int, rank: int, world: int) -> np.ndarray:
    """``int32 [F]``: local feature row of each global feature, -1 when another rank holds it."""
    f = np.arange(n_features, dtype=np.int64)
    if world <= 1:
        return f.astype(np.int32)
    c0, c1 = owned_range(n_features, rank, world)
    return np.where((f >= c0) & (f < c1), f - c0, -1).astype(np.int32)


def local_part(subset: np.ndarray, rank: int, world: int, n_features: int | None = None) -> tuple[np.ndarray, np.ndarray]:
    """For a sampled feature list: ``(local feature rows, positions in the sampled order)`` of the
    features this rank holds, both int32, positions ascending.  ``n_features`` (the width of the
    data set) is needed when ``world > 1``."""
    subset = np.asarray(subset)
    if world <= 1:
        return subset.astype(np.int32), np.arange(subset.shape[0], dtype=np.int32)
    if n_features is None:
        raise ValueError("n_features is required to locate a rank's block of features")
    c0, c1 = owned_range(n_features, rank, world)
    pos = np.nonzero((subset >= c0) & (subset < c1))[0].astype(np.int32)
    return (subset[pos] - c0).astype(np.int32), pos


def dealt_part(subset: np.ndarray, rank: int, world: int) -> tuple[np.ndarray, np.ndarray]:
    """Share of a sampled feature list when every rank holds every feature row: the list is dealt
    round-robin by position, ``(feature rows == feature ids, positions)``, both int32.  Every
    rank gets the same number of features (to within one) at every depth and the same number in
    every round, which is what lets a round be replayed as a fixed CUDA graph."""
    subset = np.asarray(subset)
    pos = np.arange(rank, subset.shape[0], max(world, 1), dtype=np.int32)
    return subset[pos].astype(np.int32), pos


def agree_all(flag: bool, device=None) -> bool:
    """True only when ``flag`` is true on every rank of the default process group (a MIN
    all-reduce).  Decisions that change the sequence of collectives a rank issues — such as the
    choice between the replicated and the memory-sharded layout of the packed matrix, which
    depends on the free memory of each rank's own GPU — must be taken this way: ranks that chose
    differently would wait for each other's collectives forever."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return bool(flag)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


def choose_replicated(packed_bytes: int, free_bytes: int, world: int, force_sharded: bool, device=None) -> bool:
    """Layout of the packed matrix on ``world`` GPUs: replicated on every rank when it takes less
    than a quarter of the free memory of EVERY rank's GPU (and sharding is not forced), else
    feature-sharded.  Collective: every rank must call it, and every rank gets the same answer."""
    if world <= 1:
        return False
    local = (not force_sharded) and packed_bytes < 0.25 * free_bytes
    return agree_all(local, device)
