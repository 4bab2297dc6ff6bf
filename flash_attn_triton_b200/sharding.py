"""Partitioning of independent attention work units across the GPUs of one box.

Every (batch, head) pair -- and every sequence of a packed batch -- is independent in the
forward and the backward pass, so multi-GPU execution needs no exchange step: each rank
takes a slice of the units, generates (or receives) only its own inputs and keeps its own
outputs.  GQA groups are kept whole (units are KV heads), because dK/dV of a KV head sums
over its query heads.  A collective is only used by callers that want all outputs in one
place (the benchmark's optional all_gather).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple


def shard_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, balanced slice [lo, hi) of n_units for `rank` (sizes differ by <= 1)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def causal_pairs(length: int, window_left: int = -1) -> int:
    """Number of visible (query, key) pairs of one causal sequence, with an optional left
    window: the cost model used to balance packed batches."""
    if window_left < 0 or length <= window_left + 1:
        return length * (length + 1) // 2
    w = window_left + 1
    return w * (w + 1) // 2 + (length - w) * w


def balance_sequences(lengths: Sequence[int], world: int, window_left: int = -1) -> List[List[int]]:
    """Longest-processing-time-first assignment of sequences to ranks by causal_pairs().
    Returns, per rank, the sorted list of sequence indices it owns."""
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(len(lengths)), key=lambda i: (-causal_pairs(lengths[i], window_left), i))
    load = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owned[r].append(i)
        load[r] += causal_pairs(lengths[i], window_left)
    return [sorted(o) for o in owned]


def unit_seed(base_seed: int, unit: int) -> int:
    """Seed of one work unit: a rank that owns unit u generates exactly the tensor the
    single-GPU run generates for u."""
    return (base_seed * 1000003 + unit * 7919 + 12345) % (2 ** 31 - 1)
