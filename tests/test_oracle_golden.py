"""The CPU oracle against the committed golden vectors (float64 torch/autograd evaluation of the
node graph, tests/golden/make_golden.py)."""
import numpy as np
import pytest

from tests.helpers import GOLDEN_CASES, flat_stats, load_golden, rel_err


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_forward_backward_update(oracle, name):
    g, fc = load_golden(name)
    data = g["data"]
    mars = oracle.forward(fc, data)
    assert rel_err(mars[:, -1], g["ll"]) <= 2e-6
    flows, aggr = oracle.backward(fc, mars)
    oracle.input_flows(fc, flows, data)
    stats = flat_stats(fc, aggr, fc.heap, oracle.meta(fc)["edge2param"])
    assert rel_err(stats, g["stats"]) <= 2e-5
    oracle.em_update(fc, aggr, float(g["pseudocount"]), float(g["inertia"]))
    assert np.abs(oracle.vectorize(fc) - g["new_theta"]).max() <= 1e-5


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_kld_and_gradients(oracle, name):
    g, fc = load_golden(name)
    p1, p2 = g["theta"].astype(np.float32), g["theta2"].astype(np.float32)
    klds, ek = oracle.kld(fc, p1, p2)
    assert abs(klds[0, -1] - g["kld"]) <= 1e-5 * max(1.0, abs(g["kld"]))
    out = oracle.kld_backward(fc, p1, p2, klds, ek)
    ni = int(g["num_inner"])
    # sum-edge gradients are the autograd gradients of the recursion
    assert rel_err(out["param_grads1"][0, :ni], g["kld_grad1"][:ni], 1e-3) <= 1e-4
    assert rel_err(out["param_grads2"][0, :ni], g["kld_grad2"][:ni], 1e-3) <= 1e-4
    # leaf gradients follow the reference's own formula (fixable_categorical_dist.jl:219):
    # (g (p1 - p2 + 1), +g exp(p1 - p2)) with g the leaf's node gradient
    grads = out["grads"][0]
    pos = ni
    for nid in fc.input_node_ids.astype(np.int64):
        c = int(fc.node_num_cats[nid - 1])
        a, b = p1[pos:pos + c], p2[pos:pos + c]
        assert np.allclose(out["param_grads1"][0, pos:pos + c], grads[nid - 1] * (a - b + 1), rtol=1e-5, atol=1e-7)
        assert np.allclose(out["param_grads2"][0, pos:pos + c], grads[nid - 1] * np.exp(a - b), rtol=1e-5, atol=1e-7)
        pos += c
