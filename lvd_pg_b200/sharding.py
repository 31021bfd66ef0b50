"""Batch sharding for the multi-GPU EM step.

The reference has no multi-GPU data path.  Here the rows of a global mini-batch are split into
contiguous, equally sized shards (one per rank); every rank accumulates the statistics vector
[edge flows by parameter id | leaf flow slots | batch log-likelihood sum] of its shard, the
vectors are summed over ranks (one all-reduce), and every rank applies the identical update to
its replica of the parameters.  Samples of `sample()` shard the same way and need no exchange.
"""
from __future__ import annotations

import time

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


class RankFailure(RuntimeError):
    """A peer did not check in for a step (or announced that it leaves): do not launch the step."""

    def __init__(self, step: int, missing, left):
        self.step, self.missing, self.left = step, sorted(missing), sorted(left)
        what = f"ranks {self.left} left" if self.left else f"ranks {self.missing} did not check in"
        super().__init__(f"step {step}: {what}; the collective of this step was not launched")


class RankWatch:
    """Host-side heartbeat over a key-value store (any `torch.distributed.Store`: the TCPStore of
    the process group, a FileStore, a HashStore between threads).

    A collective that a dead peer never joins does not end, and a kernel that waits for it blocks
    the GPU for whoever comes next.  So the ranks agree on the host BEFORE they launch: every rank
    calls `check_in(step)` ahead of the step's kernels; it returns when all ranks have checked in
    for that step and raises `RankFailure` when one has announced that it leaves (`leave()`, called
    between steps with nothing of its own in flight) or stays silent for `timeout_s`.  After a
    failure the survivors drop the communicator (`detach_comm`) and continue alone or re-form a
    smaller group; nothing was launched, so there is nothing to abort.  The reference has no
    counterpart: its workers are independent jobs whose death goes unobserved
    (exps/progressive_growing/pg.sh:2-7)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, poll_s: float = 0.002,
                 prefix: str = "pcb200/watch"):
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.poll_s, self.prefix = float(timeout_s), float(poll_s), prefix

    def _key(self, step, rank):
        return f"{self.prefix}/step{step}/{rank}"

    def _left_key(self, rank):
        return f"{self.prefix}/left/{rank}"

    def leave(self):
        """Announce an orderly exit; the peers' next `check_in` raises at once instead of waiting."""
        self.store.set(self._left_key(self.rank), b"1")

    def check_in(self, step: int):
        self.store.set(self._key(step, self.rank), b"1")
        others = [r for r in range(self.world) if r != self.rank]
        deadline = time.monotonic() + self.timeout_s
        while True:
            missing = [r for r in others if not self.store.check([self._key(step, r)])]
            if not missing:
                break
            left = [r for r in missing if self.store.check([self._left_key(r)])]
            if left or time.monotonic() > deadline:
                raise RankFailure(step, missing, left)
            time.sleep(self.poll_s)
        if step >= 2:   # every rank has passed step - 1, nobody reads the keys of step - 2 any more
            try:
                self.store.delete_key(self._key(step - 2, self.rank))
            except (RuntimeError, NotImplementedError):
                pass    # a store without deletion only grows by one short key per step
