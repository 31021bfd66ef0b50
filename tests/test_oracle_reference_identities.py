"""The identities and closed forms asserted by the reference's own unit tests, restated on the
CPU oracle.  Each test names the file of VariationalJuice.jl/test it follows.  Indices below
are the reference's 1-based ones minus one."""
import numpy as np

from lvd_pg_b200 import structures as st
from lvd_pg_b200.circuit import compile_circuit
from tests.helpers import simple3

DATA = np.array([[1, 2, 3], [2, 3, 1]], np.uint8)


def lse(a, b):
    return np.logaddexp(a, b)


def test_bits_circuit_maps(oracle):
    """bits_circuit_tests.jl:13-24"""
    m = oracle.meta(simple3(True))
    assert m["edge2param"].tolist() == [0, 0, 0, 0, 1, 2]
    assert m["param2edge"].tolist() == [5, 6]
    assert m["param2group"].tolist() == [1, 1]
    assert m["innode2ncumparam"].tolist() == [0] * 6 and m["num_input_params"] == 0
    m = oracle.meta(simple3(False))
    assert m["innode2ncumparam"].tolist() == [5, 10, 15, 20, 25, 30] and m["num_input_params"] == 30


def test_parameter_transfer_and_vectorization(oracle):
    """misc_tests.jl:9-61"""
    fc = compile_circuit(st.simple_3vars_circuit(fixed=True))
    assert fc.num_parameters == 2
    assert np.allclose(oracle.vectorize(fc), np.log(0.5))
    oracle.update_parameters(fc, np.log(np.array([0.4, 0.6], np.float32)))
    assert np.isclose(fc.up_logp[4], np.log(0.4)) and np.isclose(fc.up_logp[5], np.log(0.6))
    # up-edges 5, 6 are down-edges 1, 2 (the root's edges lead the downward order)
    assert fc.down2up[:2].tolist() == [5, 6]
    fc = simple3(False, 5, 3)
    assert fc.num_parameters == 32
    p = oracle.vectorize(fc)
    assert np.isclose(p[0], fc.up_logp[4])
    n1, n4 = fc.input_node_ids[0] - 1, fc.input_node_ids[3] - 1
    assert np.isclose(p[2], fc.heap[fc.node_heap_start[n1] - 1])
    assert np.isclose(p[17], fc.heap[fc.node_heap_start[n4] - 1])
    p[0], p[2], p[17] = 0.0, 0.1, 0.2
    oracle.update_parameters(fc, p)
    assert np.isclose(fc.up_logp[4], 0.0)
    assert np.isclose(fc.heap[fc.node_heap_start[n1] - 1], 0.1)
    assert np.isclose(fc.heap[fc.node_heap_start[n4] - 1], 0.2)


def test_likelihoods(oracle):
    """queries/likelihood_tests.jl:9-40"""
    fc = simple3(True, 5, 1)
    fc.up_logp[4:6] = np.log(np.array([0.3, 0.7], np.float32))
    mars, em = oracle.forward(fc, DATA, want_edge_mars=True)
    for b in range(2):
        assert np.isclose(lse(em[b, -2], em[b, -1]), mars[b, -1])
        assert np.isclose(mars[b, 0] + mars[b, 1], em[b, 0])
        assert np.isclose(mars[b, 2], em[b, 1])
        assert np.isclose(mars[b, 4] + mars[b, 5], em[b, 2])
        assert np.isclose(mars[b, 6], em[b, 3])


def test_flows(oracle):
    """queries/flow_tests.jl:8-64"""
    fc = simple3(False, 5, 2)
    mars, em = oracle.forward(fc, DATA, want_edge_mars=True)
    flows, ef, _ = oracle.backward(fc, mars, want_edge_flows=True)
    for b in range(2):
        assert np.isclose(ef[b, 4] + ef[b, 5], flows[b, 8])
        assert np.isclose(ef[b, 2], flows[b, 7]) and np.isclose(ef[b, 3], flows[b, 7])
        assert np.isclose(ef[b, 0], flows[b, 3]) and np.isclose(ef[b, 1], flows[b, 3])
        assert np.isclose(np.exp(em[b, 4] - lse(em[b, 4], em[b, 5])), ef[b, 4])   # flow_tests.jl:109-110
    # input edge flows: the flow of leaf 1 goes to the observed category only (:58-63)
    before = fc.heap.copy()
    oracle.input_flows(fc, flows[:1], DATA[:1])
    hs, c = fc.node_heap_start[0] - 1, 5
    got = fc.heap[hs + c:hs + 2 * c] - before[hs + c:hs + 2 * c]
    want = np.zeros(5)
    want[DATA[0, 0]] = flows[0, 0]
    assert np.allclose(got, want)


def _two_sets(oracle, fc):
    pars = oracle.vectorize(fc)
    return np.tile(pars, (2, 1)).astype(np.float32), np.tile(pars, (2, 1)).astype(np.float32)


def test_klds(oracle):
    """queries/kld_tests.jl:8-69"""
    fc = simple3(False, 5, 4)
    p1, p2 = _two_sets(oracle, fc)
    klds, ek = oracle.kld(fc, p1, p2)
    assert np.allclose(klds, 0) and np.allclose(ek, 0)
    p1[:, :2] = np.log(np.array([[0.2, 0.8], [0.5, 0.5]], np.float32))
    p2[:, :2] = np.log(np.array([[0.4, 0.6], [0.9, 0.1]], np.float32))
    klds, _ = oracle.kld(fc, p1, p2)
    assert np.isclose(klds[0, -1], 0.2 * np.log(0.2 / 0.4) + 0.8 * np.log(0.8 / 0.6), rtol=1e-5)
    assert np.isclose(klds[1, -1], 0.5 * np.log(0.5 / 0.9) + 0.5 * np.log(0.5 / 0.1), rtol=1e-5)
    p2[:, :2] = p1[:, :2]
    p1[0, 2:7] = np.log(np.array([0.1, 0.2, 0.3, 0.2, 0.2], np.float32))
    p2[0, 2:7] = np.log(np.array([0.2, 0.1, 0.1, 0.3, 0.3], np.float32))
    p1[1, 2:7] = np.log(np.array([0.1, 0.2, 0.3, 0.2, 0.2], np.float32))
    p2[1, 2:7] = np.log(np.array([0.2, 0.1, 0.2, 0.3, 0.2], np.float32))
    klds, _ = oracle.kld(fc, p1, p2)
    for s, w in ((0, 0.2), (1, 0.5)):
        assert np.isclose(klds[s, -1], (np.exp(p1[s, 2:7]) * (p1[s, 2:7] - p2[s, 2:7])).sum() * w, rtol=1e-5)


def test_klds_backward(oracle):
    """queries/kld_tests.jl:71-129"""
    fc = simple3(False, 5, 5)
    p1, p2 = _two_sets(oracle, fc)
    klds, ek = oracle.kld(fc, p1, p2)
    out = oracle.kld_backward(fc, p1, p2, klds, ek)
    eg1, eg2 = out["edge_grads1"], out["edge_grads2"]
    assert np.isclose(eg1[0, 4], np.exp(p1[0, 0])) and np.isclose(eg1[0, 5], np.exp(p1[0, 1]))
    assert np.allclose(eg1[:, 4:6], -eg2[:, 4:6])
    assert np.allclose(eg1[:, :4], 0) and np.allclose(eg2[:, :4], 0)
    p1[:, :2] = np.log(np.array([[0.2, 0.8], [0.5, 0.5]], np.float32))
    p2[:, :2] = np.log(np.array([[0.4, 0.6], [0.9, 0.1]], np.float32))
    klds, ek = oracle.kld(fc, p1, p2)
    out = oracle.kld_backward(fc, p1, p2, klds, ek)
    eg1, eg2 = out["edge_grads1"], out["edge_grads2"]
    assert np.isclose(eg1[0, 4], 0.2 * (np.log(0.2) - np.log(0.4) + 1), rtol=1e-5)
    assert np.isclose(eg2[0, 4], -0.2, rtol=1e-5)
    assert np.isclose(eg1[0, 5], 0.8 * (np.log(0.8) - np.log(0.6) + 1), rtol=1e-5)
    assert np.isclose(eg2[0, 5], -0.8, rtol=1e-5)


def test_kld_inner_nodes(oracle):
    """queries/kld_tests.jl:168-208 (two variables, fixed near-one-hot leaves)"""
    fc = compile_circuit(st.fully_factorized_categorical_fixed(num_vars=2, num_cats=8))
    pars = oracle.vectorize(fc)
    rng = np.random.default_rng(0)
    p1 = pars.copy()
    for sl in (slice(0, 8), slice(8, 16)):
        w = rng.random(8)
        p1[sl] = np.log(w / w.sum())
    klds, ek = oracle.kld(fc, p1, pars)
    assert np.isclose(klds[0, 8], (np.exp(p1[:8]) * (p1[:8] - pars[:8])).sum(), rtol=1e-5)
    assert np.isclose(klds[0, 17], (np.exp(p1[8:16]) * (p1[8:16] - pars[8:16])).sum(), rtol=1e-5)
    out = oracle.kld_backward(fc, p1, pars, klds, ek)
    for i in range(8):
        assert np.isclose(np.exp(p1[i]), out["grads"][0, i], rtol=1e-5)
        assert np.isclose(out["param_grads1"][0, i], np.exp(p1[i]) * (p1[i] - pars[i] + 1), rtol=1e-4)
    for i in range(8, 16):
        assert np.isclose(np.exp(p1[i]), out["grads"][0, i + 1], rtol=1e-5)


def test_gumbel_softmax_samples(oracle):
    """queries/sample_tests.jl:9-54 and :120-148"""
    fc = simple3(False, 2, 6)
    pars = np.tile(oracle.vectorize(fc), (2, 1))
    u = np.random.default_rng(1).random((2, 2), dtype=np.float32)
    out, aux = oracle.sample_soft(fc, pars, u, 1.0, 2, 2)
    ep, cp, td = aux["edge_probs"], aux["cum_probs"], aux["td_probs"]
    for s in range(2):
        assert np.isclose(ep[s].sum(), cp[s, 0])
        assert np.isclose(ep[s, 0] / cp[s, 0], td[s, 3]) and np.isclose(ep[s, 1] / cp[s, 0], td[s, 7])
        assert np.allclose(td[s, 0:3], td[s, 3]) and np.allclose(td[s, 4:7], td[s, 7])
        assert np.allclose(out[s].sum(1), 1.0)
    fc = compile_circuit(st.fully_factorized_categorical_fixed(num_vars=3, num_cats=8))
    pars = oracle.vectorize(fc)[None, :]
    out, aux = oracle.sample_soft(fc, pars, None, 1.0, 1, 8)
    ep, cp, td = aux["edge_probs"], aux["cum_probs"], aux["td_probs"]
    assert np.isclose(td[0, 8], 1) and np.isclose(td[0, 17], 1) and np.isclose(td[0, 26], 1)
    assert np.isclose(cp[0, 0], ep[0, :8].sum()) and np.isclose(cp[0, 2], ep[0, 16:24].sum())
    assert np.isclose(td[0, 0], ep[0, 0] / cp[0, 0])
    assert np.isclose(out[0, 0, 0], td[0, 0], atol=1e-5) and np.isclose(out[0, 0, 1], td[0, 1], atol=1e-5)


def test_em_update_relations(oracle):
    """conditional_pc/custom_em_tests.jl:88-91,131,195-207: edge_aggr is in down-edge order and the
    update is log((1 - lr) e^theta + lr * normalised flow) with inertia = 1 - lr."""
    fc = simple3(False, 5, 7)
    before = oracle.vectorize(fc)
    data = np.random.default_rng(3).integers(0, 5, (40, 3)).astype(np.uint8)
    mars = oracle.forward(fc, data)
    flows, aggr = oracle.backward(fc, mars)
    oracle.input_flows(fc, flows, data)
    assert np.isclose(aggr[0] + aggr[1], 40.0, rtol=1e-5)      # the root's two edges come first
    lr, pc = 0.25, 0.1
    a = aggr[:2] + pc / 2
    heap = fc.heap.copy()
    oracle.em_update(fc, aggr, pc, 1 - lr)
    after = oracle.vectorize(fc)
    assert np.allclose(after[:2], np.log((1 - lr) * np.exp(before[:2]) + lr * a / a.sum()), atol=1e-6)
    hs = fc.node_heap_start[0] - 1
    f = heap[hs + 5:hs + 10]
    new = (f + pc / 5) / (f.sum() + pc)
    assert np.allclose(after[2:7], np.log((1 - lr) * np.exp(before[2:7]) + lr * new), atol=1e-6)
