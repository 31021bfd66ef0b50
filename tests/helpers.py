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
