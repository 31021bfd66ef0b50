"""The N > 1 path on CPU ranks (gloo, world size 2): shard the batch, accumulate per-rank
statistics, all-reduce, apply the replicated update.  The per-rank compute is done by the CPU
oracle here; on GPUs the same vector is all-reduced by NCCL inside pcb_em_step."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from lvd_pg_b200.sharding import shard_rows, statistics_length
    from oracle import oracle as orc
    from tests.helpers import flat_stats, random_data, random_hclt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc.set_num_threads(1)
    fc = random_hclt(8, 4, 3, seed=1)
    data, _ = random_data(101, 8, 3, 2)
    ids = (np.random.default_rng(0).permutation(101)[:64] + 1).astype(np.int32)   # the global batch
    mine = shard_rows(ids, rank, world)
    mars = orc.forward(fc, data, row_ids=mine)
    flows, aggr = orc.backward(fc, mars)
    orc.input_flows(fc, flows, data, row_ids=mine)
    e2p = orc.meta(fc)["edge2param"]
    stats = np.concatenate([flat_stats(fc, aggr, fc.heap, e2p), [mars[:, -1].astype(np.float64).sum()]])
    cats = fc.node_num_cats[fc.input_node_ids.astype(np.int64) - 1]
    assert statistics_length(fc.num_inner_params, cats) == len(stats) + len(cats)  # + the missing slots
    t = torch.from_numpy(stats)
    dist.all_reduce(t)
    np.save(os.path.join(out_dir, f"stats_{rank}.npy"), t.numpy())
    dist.barrier()
    dist.destroy_process_group()


def _flow_slots(fc):
    """Heap indices of the leaf flow accumulators (C + 1 per learnable leaf)."""
    idx = []
    for nid in fc.input_node_ids.astype(np.int64):
        if not fc.node_fixed[nid - 1]:
            c, hs = int(fc.node_num_cats[nid - 1]), int(fc.node_heap_start[nid - 1]) - 1
            idx.extend(range(hs + c, hs + 2 * c + 1))
    return np.asarray(idx, np.int64)


def _flow_memory_worker(rank, world, port, out_dir):
    """Three mini-batch steps with flow_memory > 0 on `world` ranks: every rank decays the summed
    statistics it carries by rate / world, adds its shard's flows, all-reduces, updates."""
    sys.path.insert(0, ROOT)
    from lvd_pg_b200.sharding import carried_rate, shard_rows
    from oracle import oracle as orc
    from tests.helpers import random_data, random_hclt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc.set_num_threads(1)
    fc = random_hclt(8, 4, 3, seed=1)
    data, _ = random_data(101, 8, 3, 2)
    slots = _flow_slots(fc)
    aggr = np.zeros(fc.num_edges, np.float32)
    rng = np.random.default_rng(0)
    for step in range(3):
        ids = (rng.permutation(101)[:64] + 1).astype(np.int32)
        orc.clear_flows(fc, aggr, carried_rate(0.7, world))
        mine = shard_rows(ids, rank, world)
        mars = orc.forward(fc, data, row_ids=mine)
        flows, aggr = orc.backward(fc, mars, aggr)
        orc.input_flows(fc, flows, data, row_ids=mine)
        t = torch.from_numpy(np.concatenate([aggr.astype(np.float64), fc.heap[slots].astype(np.float64)]))
        dist.all_reduce(t)
        aggr[:] = t.numpy()[:fc.num_edges]
        fc.heap[slots] = t.numpy()[fc.num_edges:]
        orc.em_update(fc, aggr, 0.1, 0.8)
    np.save(os.path.join(out_dir, f"params_{rank}.npy"), orc.vectorize(fc))
    np.save(os.path.join(out_dir, f"aggr_{rank}.npy"), aggr)
    dist.barrier()
    dist.destroy_process_group()


def test_flow_memory_on_two_ranks_equals_one_rank(oracle, tmp_path):
    """With clear_rate != 0 the carried statistics must sum to rate * previous over the ranks: if
    every rank kept rate * (global sum) the history would be counted `world` times per step."""
    from tests.helpers import random_data, random_hclt
    world = 2
    mp.spawn(_flow_memory_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = [np.load(tmp_path / f"params_{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1])
    fc = random_hclt(8, 4, 3, seed=1)
    data, _ = random_data(101, 8, 3, 2)
    aggr = np.zeros(fc.num_edges, np.float32)
    rng = np.random.default_rng(0)
    for step in range(3):
        ids = (rng.permutation(101)[:64] + 1).astype(np.int32)
        oracle.em_step(fc, data, row_ids=ids, pseudocount=0.1, inertia=0.8, edge_aggr=aggr, clear_rate=0.7)
    assert np.abs(np.exp(got[0]) - np.exp(oracle.vectorize(fc))).max() <= 1e-5
    assert np.allclose(np.load(tmp_path / "aggr_0.npy"), aggr, rtol=1e-5, atol=1e-6)


def test_sharded_statistics_equal_the_full_batch(oracle, tmp_path):
    from tests.helpers import flat_stats, random_data, random_hclt
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = [np.load(tmp_path / f"stats_{r}.npy") for r in range(world)]
    assert np.array_equal(got[0], got[1])                       # every rank holds the same sum
    fc = random_hclt(8, 4, 3, seed=1)
    data, _ = random_data(101, 8, 3, 2)
    ids = (np.random.default_rng(0).permutation(101)[:64] + 1).astype(np.int32)
    mars = oracle.forward(fc, data, row_ids=ids)
    flows, aggr = oracle.backward(fc, mars)
    oracle.input_flows(fc, flows, data, row_ids=ids)
    full = np.concatenate([flat_stats(fc, aggr, fc.heap, oracle.meta(fc)["edge2param"]),
                           [mars[:, -1].astype(np.float64).sum()]])
    assert np.allclose(got[0], full, rtol=1e-5, atol=1e-6)


def test_shard_bounds_cover_everything():
    from lvd_pg_b200.sharding import shard_bounds
    for n in (0, 1, 7, 64, 2048):
        for world in (1, 2, 3, 8):
            cuts = [shard_bounds(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1
