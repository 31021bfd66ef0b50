"""Failure detection of the multi-GPU step, made on the host: ranks are CPU processes (gloo) that
share the process group's store; a rank leaves between steps or goes silent, and the survivor has to
learn of it BEFORE it would launch the next step's collective.  No GPU is involved."""
import os
import socket
import sys
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from lvd_pg_b200.sharding import RankFailure, RankWatch  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir, mode):
    sys.path.insert(0, ROOT)
    from lvd_pg_b200.sharding import RankFailure, RankWatch
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world)
    watch = RankWatch(store, rank, world, timeout_s=1.5)
    launched, failure = [], None
    t = torch.ones(4)
    for step in range(6):
        if rank == 1 and step == 3:
            if mode == "leaves":
                watch.leave()      # orderly: between steps, nothing in flight
            break                  # "silent": just stops checking in (as a crashed host loop would)
        try:
            t0 = time.monotonic()
            watch.check_in(step)
        except RankFailure as e:
            failure = (e.step, e.missing, e.left, time.monotonic() - t0)
            break
        dist.all_reduce(t)         # stands for the step with its collective
        launched.append(step)
    torch.save({"launched": launched, "failure": failure, "sum": float(t[0])}, os.path.join(out_dir, f"r{rank}.pt"))
    if rank == 1:
        time.sleep(2.5)            # keep the process (and rank 0's store clients) alive past the peer's timeout
    os._exit(0)                    # no destroy_process_group: the peer is gone or about to go


@pytest.mark.parametrize("mode", ["leaves", "silent"])
def test_survivor_learns_of_a_lost_rank_before_it_launches(tmp_path, mode):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path), mode), nprocs=2, join=True)
    r0 = torch.load(tmp_path / "r0.pt")
    r1 = torch.load(tmp_path / "r1.pt")
    assert r0["launched"] == [0, 1, 2] and r1["launched"] == [0, 1, 2]   # step 3 was never launched by anyone
    assert r0["sum"] == 8.0                                               # three all-reduces of two ranks
    step, missing, left, waited = r0["failure"]
    assert step == 3 and missing == [1]
    if mode == "leaves":
        assert left == [1] and waited < 1.0      # announced: no need to sit out the timeout
    else:
        assert left == [] and 1.4 < waited < 3.0


def test_watch_between_threads_of_one_process():
    """The same protocol over an in-process store: all ranks present -> every check-in returns; old keys go."""
    import threading
    store = dist.HashStore()
    errs = []

    def run(rank):
        w = RankWatch(store, rank, 3, timeout_s=5.0)
        try:
            for step in range(5):
                w.check_in(step)
        except Exception as e:  # noqa: BLE001
            errs.append(e)

    th = [threading.Thread(target=run, args=(r,)) for r in range(3)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs
    assert not store.check(["pcb200/watch/step0/0"]) and store.check(["pcb200/watch/step4/0"])
    w = RankWatch(store, 0, 3, timeout_s=0.2)
    with pytest.raises(RankFailure) as e:
        w.check_in(7)
    assert e.value.missing == [1, 2] and e.value.left == []
