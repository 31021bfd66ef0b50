"""Host-side structure code and size-independent properties of the oracle."""
import itertools
import math

import numpy as np
import pytest

from lvd_pg_b200 import structures as st, synth
from lvd_pg_b200.circuit import compile_circuit
from tests.helpers import random_data, random_hclt, rel_err


def test_hclt_flat_matches_the_literal_construction(oracle):
    """The shared-product compiled HCLT and hclts.jl:100-145 taken literally (k*k products per CLT
    node) define the same distribution."""
    rng = np.random.default_rng(5)
    parent = st.root_tree_at_center(7, st.random_spanning_tree(7, rng))
    flat = st.hclt_flat(parent, 3, 4, seed=None)
    lit = compile_circuit(st.hclt_graph(parent, 3, 4, None))
    assert lit.num_inner_params == flat.num_inner_params and lit.num_input_params == flat.num_input_params
    data, _ = random_data(50, 7, 3, 1)
    assert np.allclose(oracle.forward(flat, data)[:, -1], oracle.forward(lit, data)[:, -1], atol=1e-5)
    # counts of hclts.jl:116-138: E_s = (I - 1) k^2 + k, leaf params V k C
    inner = sum(1 for v in range(7) if (parent == v).any())
    assert flat.num_inner_params == (inner - 1) * 16 + 4
    assert flat.num_input_params == 7 * 4 * 3


@pytest.mark.parametrize("v,k,c", [(5, 2, 2), (6, 3, 3), (4, 5, 2)])
def test_hclt_is_normalised(oracle, v, k, c):
    fc = random_hclt(v, k, c, seed=v * 10 + k)
    allx = np.array(list(itertools.product(range(c), repeat=v)), np.uint8)
    ll = oracle.forward(fc, allx)[:, -1].astype(np.float64)
    assert abs(np.exp(ll).sum() - 1.0) < 1e-5


def test_missing_values_marginalise(oracle):
    fc = random_hclt(5, 3, 3, seed=2)
    allx = np.array(list(itertools.product(range(3), repeat=5)), np.uint8)
    ll = oracle.forward(fc, allx)[:, -1].astype(np.float64)
    x = np.array([[1, 0, 2, 0, 1]], np.uint8)
    miss = np.array([[0, 1, 0, 1, 0]], np.uint8)
    marg = np.exp(ll[(allx[:, 0] == 1) & (allx[:, 2] == 2) & (allx[:, 4] == 1)]).sum()
    assert np.isclose(np.exp(oracle.forward(fc, x, miss=miss)[0, -1]), marg, rtol=1e-5)


def test_flow_conservation_and_em_monotonicity(oracle):
    fc = random_hclt(8, 4, 3, seed=3)
    data, _ = random_data(200, 8, 3, 4)
    mars = oracle.forward(fc, data)
    flows, aggr = oracle.backward(fc, mars)
    # the flow entering the leaves of one variable sums to one per example
    for v in range(1, 9):
        leaves = np.nonzero(fc.node_var == v)[0]
        assert np.allclose(flows[:, leaves].sum(1), 1.0, atol=1e-5)
    # full-batch EM (inertia 0) never decreases the training likelihood
    lls = []
    for _ in range(4):
        ll, _ = oracle.em_step(fc, data, pseudocount=1e-6, inertia=0.0)
        lls.append(ll)
    assert all(b >= a - 1e-3 for a, b in zip(lls, lls[1:]))
    # parameters stay normalised (the validity check of utils/utils.jl:88-105)
    m = oracle.meta(fc)
    p = np.exp(oracle.vectorize(fc).astype(np.float64))
    for gid in range(1, m["num_param_groups"] + 1):
        assert abs(p[:m["num_inner_params"]][m["param2group"] == gid].sum() - 1) < 1e-4
    assert np.allclose(p[m["num_inner_params"]:].reshape(-1, 3).sum(1), 1.0, atol=1e-4)


def test_gumbel_key_is_an_accurate_log(oracle):
    rng = np.random.default_rng(0)
    for x in np.concatenate([rng.random(200), rng.random(50) * 20, [1e-6, 1.0, 2.0, 0.70710678, 1.41421357]]):
        if x > 0:
            assert abs(oracle.det_log(float(x)) - math.log(x)) <= 4e-16 * max(1.0, abs(math.log(x)))
    for lp, u in [(-1.25, 0.5), (-0.1, 0.0), (-7.0, 0.99999994)]:
        want = float(np.float32(lp)) + -math.log(-math.log(np.float32(u).astype(np.float64) * (1.0 - 1e-6) + 1e-6))
        assert abs(oracle.gumbel_key(lp, u) - want) < 1e-12


def test_hard_sampling_follows_the_distribution(oracle):
    fc = random_hclt(4, 3, 2, seed=9)
    allx = np.array(list(itertools.product(range(2), repeat=4)), np.uint8)
    probs = np.exp(oracle.forward(fc, allx)[:, -1].astype(np.float64))
    S = 20000
    _, R = oracle.sum_regions(fc)
    rng = np.random.default_rng(1)
    x = oracle.sample_hard(fc, oracle.vectorize(fc), rng.random((S, R, 3), dtype=np.float32),
                           rng.random((S, 4, 2), dtype=np.float32), S)
    counts = np.bincount((x * (2 ** np.arange(3, -1, -1))).sum(1), minlength=16) / S
    assert np.abs(counts - probs).max() < 0.015


def test_chow_liu_recovers_a_tree_and_synthetic_shapes():
    data = synth.tree_bernoulli_data(4000, 12, 3)
    assert data.shape == (4000, 12) and data.max() == 1
    parent = st.learn_clt(data, 2, 0.1)
    assert (parent < 0).sum() == 1 and len(parent) == 12
    img = synth.blurred_noise_images(64, 8, 2.0, 0)
    assert img.shape == (64, 192) and img.dtype.is_floating_point is False
    m = img.float().mean().item()
    assert 100 < m < 156
    # neighbouring pixels of the same channel are strongly correlated, as in natural images
    a, b = img[:, 0].float(), img[:, 3].float()
    assert np.corrcoef(a.numpy(), b.numpy())[0, 1] > 0.5


def test_compile_rejects_nothing_valid_and_counts(oracle):
    fc = compile_circuit(st.fully_factorized_categorical_fixed(3, 8))
    assert fc.num_nodes == 29 and fc.node_kind[[8, 17, 26]].tolist() == [2, 2, 2]
    assert fc.num_input_params == 0 and fc.heap.shape[0] == 3 * 8 * 8
