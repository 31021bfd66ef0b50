"""Shared builders and comparison rules for the test-suite."""
import numpy as np

from lvd_pg_b200 import structures as st
from lvd_pg_b200.circuit import compile_circuit


def rel_err(a, ref, floor_frac=1e-6):
    """|a - ref| / max(|ref|, floor_frac * max|ref|): the parity metric for flows and parameters
    (values can be exactly 0)."""
    a = np.asarray(a, np.float64)
    ref = np.asarray(ref, np.float64)
    scale = np.maximum(np.abs(ref), floor_frac * max(np.abs(ref).max(), 1e-30))
    return float((np.abs(a - ref) / scale).max()) if ref.size else 0.0


def random_hclt(v, k, c, seed, tree_seed=None):
    rng = np.random.default_rng(seed if tree_seed is None else tree_seed)
    parent = st.root_tree_at_center(v, st.random_spanning_tree(v, rng))
    return st.hclt_flat(parent, c, k, seed=seed)


def random_data(rows, v, c, seed, missing_frac=0.0):
    rng = np.random.default_rng(seed)
    data = rng.integers(0, c, (rows, v)).astype(np.uint8)
    miss = None
    if missing_frac > 0:
        miss = (rng.random((rows, v)) < missing_frac).astype(np.uint8)
    return data, miss


def simple3(fixed=False, num_cats=5, seed=0):
    rng = np.random.default_rng(seed)
    return compile_circuit(st.simple_3vars_circuit(num_cats=num_cats, fixed=fixed, rng=rng))


# ---- golden fixtures (tests/golden/make_golden.py) -------------------------------------------
import os

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ["simple3", "hclt_v6_k3_c4", "hclt_chain5_k2_c2"]


def load_golden(name):
    """Returns (golden arrays, FlatCircuit with the golden's parameters)."""
    from oracle import oracle as orc
    g = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    if name == "simple3":
        fc = compile_circuit(st.simple_3vars_circuit(num_cats=5, fixed=False, rng=None))
    else:
        fc = compile_circuit(st.hclt_graph(g["parent"], int(g["num_cats"]), int(g["k"]), None))
    orc.update_parameters(fc, g["theta"].astype(np.float32))
    return g, fc


def flat_stats(fc, edge_aggr_down, heap, edge2param):
    """Sufficient statistics in flat parameter order: edge flows of sum edges, then the C flow
    slots of every learnable leaf."""
    out = np.zeros(fc.num_parameters, np.float64)
    up = fc.down2up.astype(np.int64) - 1
    pid = edge2param[up].astype(np.int64)
    ok = pid > 0
    out[pid[ok] - 1] = edge_aggr_down[ok]
    pos = fc.num_inner_params
    for nid in fc.input_node_ids.astype(np.int64):
        if fc.node_fixed[nid - 1]:
            continue
        c = int(fc.node_num_cats[nid - 1])
        hs = int(fc.node_heap_start[nid - 1]) - 1
        out[pos:pos + c] = heap[hs + c:hs + 2 * c]
        pos += c
    return out
