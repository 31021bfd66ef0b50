"""Batch sharding for the multi-GPU EM step.

The reference has no multi-GPU data path.  Here the rows of a global mini-batch are split into
contiguous, equally sized shards (one per rank); every rank accumulates the statistics vector
[edge flows by parameter id | leaf flow slots | batch log-likelihood sum] of its shard, the
vectors are summed over ranks (one all-reduce), and every rank applies the identical update to
its replica of the parameters.  Samples of `sample()` shard the same way and need no exchange.
"""
from __future__ import annotations

import numpy as np


def shard_bounds(n: int, rank: int, world: int):
    """Contiguous shard [lo, hi) of n items; sizes differ by at most one."""
    base, rem = divmod(n, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_rows(row_ids: np.ndarray, rank: int, world: int) -> np.ndarray:
    lo, hi = shard_bounds(len(row_ids), rank, world)
    return row_ids[lo:hi]


def statistics_length(num_inner_params: int, leaf_cats) -> int:
    """Length of the all-reduced vector: one slot per sum edge, C + 1 per learnable leaf, one
    for the log-likelihood sum."""
    return int(num_inner_params + sum(int(c) + 1 for c in leaf_cats) + 1)


def carried_rate(rate: float, world: int) -> float:
    """Decay each rank applies to the statistics it carries from the last step when `flow_memory`
    is on (regularization/reg_em.jl:276-284: edge_aggr .*= rate).  After an all-reduced step every
    rank holds the same global sums, and the next all-reduce adds the ranks' vectors again, so each
    rank keeps rate / world of them: the sum is rate * previous + this step's flows, as on one
    device.  pcb_em_step applies the same rule when a communicator is attached."""
    return rate / world if world > 1 else rate
