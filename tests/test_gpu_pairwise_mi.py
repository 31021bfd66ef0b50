"""pcb_pairwise_mi (pairwise_MI_chunked, utils/information.jl:3-157) against the float64 restatement in
lvd_pg_b200.structures.pairwise_mi: category counts from 2 to 256, row counts that end inside a chunk of
64 and inside a group of 8, variable counts whose (variable, category) rows end inside a 128-row tile."""
import numpy as np
import pytest

from lvd_pg_b200 import structures as st

pytestmark = pytest.mark.gpu

CASES = [(2, 37, 1000), (2, 200, 64), (4, 33, 517), (8, 19, 4099), (16, 9, 130), (32, 11, 777), (64, 5, 1500),
         (128, 3, 900), (256, 3, 2051)]


def _data(c, v, rows, seed):
    rng = np.random.default_rng(seed)
    # correlated columns: a latent class shifts every column's distribution
    z = rng.integers(0, 4, rows)
    x = (rng.integers(0, c, (rows, v)) + z[:, None] * rng.integers(0, 2, v)[None, :]) % c
    return x.astype(np.uint8)


@pytest.mark.parametrize("c,v,rows", CASES, ids=[f"c{c}_v{v}_n{n}" for c, v, n in CASES])
@pytest.mark.parametrize("pseudocount", [0.1, 0.0])
def test_pairwise_mi(c, v, rows, pseudocount):
    import torch
    from lvd_pg_b200 import api
    data = _data(c, v, rows, c + v)
    want = st.pairwise_mi(data, c, pseudocount) if pseudocount > 0 else _mi_numpy(data, c)
    got = api.pairwise_mi(data, c, pseudocount).cpu().numpy().astype(np.float64)
    assert got.shape == (v, v)
    np.testing.assert_allclose(got, got.T, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)


def _mi_numpy(data, c):
    """MI from plain counts (no smoothing): empty cells contribute nothing."""
    rows, v = data.shape
    oh = np.zeros((rows, v * c))
    oh[np.arange(rows)[:, None], np.arange(v)[None, :] * c + data] = 1.0
    joint = (oh.T @ oh).reshape(v, c, v, c).transpose(0, 2, 1, 3) / rows
    single = oh.sum(0).reshape(v, c) / rows
    with np.errstate(divide="ignore", invalid="ignore"):
        t = joint * (np.log(joint) - np.log(single[:, None, :, None]) - np.log(single[None, :, None, :]))
    return np.where(joint > 0, t, 0.0).sum((2, 3))


def test_chow_liu_tree_from_the_kernel_equals_the_reference_path():
    """The maximum spanning tree over the kernel's MI equals the one over the float64 MI."""
    import torch
    from lvd_pg_b200 import api
    rng = np.random.default_rng(5)
    parent = st.root_tree_at_center(24, st.random_spanning_tree(24, rng))
    data = np.zeros((3000, 24), np.uint8)
    order = [int(np.nonzero(parent < 0)[0][0])] if (parent < 0).any() else [0]
    data[:, order[0]] = rng.integers(0, 2, 3000)
    done = {order[0]}
    while len(done) < 24:
        for y in range(24):
            if y not in done and int(parent[y]) in done:
                flip = rng.random(3000) < 0.2
                data[:, y] = np.where(flip, 1 - data[:, int(parent[y])], data[:, int(parent[y])])
                done.add(y)
    mi_ref = st.pairwise_mi(data, 2, 0.1)
    mi = api.pairwise_mi(data, 2, 0.1).cpu().numpy().astype(np.float64)
    a = sorted(tuple(sorted(e)) for e in st.max_spanning_tree(mi_ref))
    b = sorted(tuple(sorted(e)) for e in st.max_spanning_tree(mi))
    assert a == b
    want = st.root_tree_at_center(24, st.max_spanning_tree(mi_ref))
    assert np.array_equal(api.learn_chow_liu_tree(data, 2, 0.1), want)
