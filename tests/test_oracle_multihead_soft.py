"""The oracle's multi-head and soft-evidence paths against the reference's own known answers
(test/multi_head_pc/multi_head_pc_learning_tests.jl) and against identities that follow from the
reference's definitions (regularization/reg_likelihood.jl, reg_flow.jl)."""
import numpy as np

from lvd_pg_b200 import structures as st
from lvd_pg_b200.circuit import TAG_USER, compile_circuit, compile_multihead
from oracle import oracle as orc


def _reference_multihead():
    """The circuit and inputs of the reference's "Multi-head PC likelihood & flow" test set."""
    pcs = st.simple_multihead_circuit(num_cats=5)
    pcs[0].children[0].children[0].logps[:] = np.log(np.array([0.1, 0.2, 0.3, 0.3, 0.1], np.float32))
    pcs[0].logps[:] = np.log(np.array([0.2, 0.8], np.float32))
    pcs[1].logps[:] = np.log(np.array([0.6, 0.4], np.float32))
    fc, roots = compile_multihead(pcs)
    data = np.array([[0, 0, 0], [2, 0, 0]], np.uint8)
    mask = np.array([[1.0, 0.0], [0.0, 1.0]], np.float32)
    return fc, roots, data, mask


def test_multihead_numbering_follows_the_reference():
    fc, roots, _, _ = _reference_multihead()
    assert fc.num_nodes == 11
    assert roots.tolist() == [9, 10]          # flows[:, 9], flows[:, 10] in the reference's test; 11 = fake root
    tagged = (fc.up_tag & TAG_USER) != 0
    assert tagged.sum() == 2 and (fc.up_parent[tagged] == 11).all()


def test_multihead_likelihoods_known_answers():
    fc, roots, data, mask = _reference_multihead()
    mars = orc.forward_ex(fc, data)
    lls = orc.multihead_lls(fc, mars, roots, mask)
    # multi_head_pc_learning_tests.jl:23-26
    np.testing.assert_allclose(lls[0], np.log(0.1 * 0.2 * 0.2 * 0.2 + 0.2 ** 3 * 0.8), rtol=1e-5)
    np.testing.assert_allclose(lls[1], np.log(0.3 * 0.2 * 0.2 * 0.6 + 0.2 ** 3 * 0.4), rtol=1e-5)
    per_head = orc.multihead_lls(fc, mars, roots, None)
    assert per_head.shape == (2, 2)
    np.testing.assert_allclose(per_head[:, 0], mars[:, 8])
    np.testing.assert_allclose(per_head[:, 1], mars[:, 9])


def test_multihead_flows_known_answers():
    fc, roots, data, mask = _reference_multihead()
    # multi_head_pc_learning_tests.jl:33-49 (soft_reg = 0.01, soft_reg_width = 3)
    mars = orc.forward_ex(fc, data, soft_reg=0.01, soft_reg_width=3)
    flows, aggr = orc.backward_ex(fc, mars, roots, mask)
    f = lambda b, n: flows[b - 1, n - 1]
    m = lambda b, n: mars[b - 1, n - 1]
    np.testing.assert_allclose(f(1, 9), 1.0)
    np.testing.assert_allclose(f(1, 10), 0.0)
    np.testing.assert_allclose(flows[:, 10], 0.0)
    np.testing.assert_allclose(f(2, 9), 0.0)
    np.testing.assert_allclose(f(2, 10), 1.0)
    l = lambda x: np.log(np.float32(x))
    np.testing.assert_allclose(f(1, 4), np.exp(m(1, 1) + m(1, 2) + m(1, 3) + l(0.2) - m(1, 9)), rtol=1e-5)
    np.testing.assert_allclose(f(1, 8), np.exp(m(1, 5) + m(1, 6) + m(1, 7) + l(0.8) - m(1, 9)), rtol=1e-5)
    np.testing.assert_allclose(f(2, 4), np.exp(m(2, 1) + m(2, 2) + m(2, 3) + l(0.6) - m(2, 10)), rtol=1e-5)
    np.testing.assert_allclose(f(2, 8), np.exp(m(2, 5) + m(2, 6) + m(2, 7) + l(0.4) - m(2, 10)), rtol=1e-5)
    # the fake root's edges gather nothing
    tagged = (fc.up_tag & TAG_USER) != 0
    assert (aggr[np.argsort(fc.down2up)][tagged] == 0).all() or (aggr[tagged[fc.down2up - 1]] == 0).all()


def test_soft_regularised_leaf_values():
    # soft_loglikelihood, reg_likelihood.jl:4-14, restated with numpy on one leaf
    fc = compile_circuit(st.simple_3vars_circuit(num_cats=5, fixed=False, rng=np.random.default_rng(1)))
    data = np.array([[0, 2, 4], [3, 1, 0]], np.uint8)
    reg, width = np.float32(0.1), 3
    mars = orc.forward_ex(fc, data, soft_reg=float(reg), soft_reg_width=width)
    for i, n in enumerate(fc.input_node_ids):
        n0 = int(n) - 1
        C = int(fc.node_num_cats[n0]); hs = int(fc.node_heap_start[n0]) - 1
        tab = fc.heap[hs:hs + C]
        for b in range(2):
            x = int(data[b, int(fc.node_var[n0]) - 1])
            c0 = max(0, x - width // 2); c1 = min(c0 + width - 1, C - 1)
            sp = np.exp(tab[c0:c1 + 1]).sum() / (c1 - c0 + 1)
            want = np.logaddexp(tab[x] + np.log(1 - reg), np.log(sp) + np.log(reg))
            np.testing.assert_allclose(mars[b, n0], want, rtol=1e-5, atol=1e-6)


def test_one_hot_soft_evidence_equals_hard_evidence():
    # log-weights 0 on the observed category and -inf elsewhere select that category's parameter
    # (init_mar!_with_reg_cat_kernel, reg_likelihood.jl:51-72) and send the whole flow to its slot
    rng = np.random.default_rng(3)
    fc = compile_circuit(st.simple_3vars_circuit(num_cats=5, fixed=False, rng=rng))
    data = rng.integers(0, 5, size=(7, 3)).astype(np.uint8)
    soft = np.full((7, 3, 5), -np.inf, np.float32)
    for r in range(7):
        for v in range(3):
            soft[r, v, data[r, v]] = 0.0
    hard = orc.forward(fc, data)
    np.testing.assert_allclose(orc.forward_ex(fc, soft=soft), hard, rtol=1e-6, atol=1e-6)
    a, b = fc.copy(), fc.copy()
    ll_a, ea = orc.em_step(a, data, pseudocount=0.1)
    ll_b, eb = orc.em_step_ex(b, soft=soft, pseudocount=0.1)
    np.testing.assert_allclose(ll_a, ll_b, rtol=1e-6)
    np.testing.assert_allclose(ea, eb, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(a.heap, b.heap, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(a.up_logp, b.up_logp, rtol=1e-5, atol=1e-6)


def test_soft_evidence_flows_sum_to_the_node_flow():
    # input_flows_circuit_with_reg_cat_kernel (reg_flow.jl:50-82): the posterior over the categories
    # of a leaf sums to one, so the slots of a leaf gather exactly its flow
    rng = np.random.default_rng(5)
    fc = compile_circuit(st.simple_3vars_circuit(num_cats=4, fixed=False, rng=rng))
    soft = np.log(rng.dirichlet(np.ones(4), size=(6, 3))).astype(np.float32)
    mars = orc.forward_ex(fc, soft=soft)
    flows, _ = orc.backward(fc, mars)
    orc.input_flows_ex(fc, flows, soft=soft)
    for n in fc.input_node_ids:
        n0 = int(n) - 1
        C = int(fc.node_num_cats[n0]); hs = int(fc.node_heap_start[n0]) - 1
        np.testing.assert_allclose(fc.heap[hs + C:hs + 2 * C].sum(), flows[:, n0].sum(), rtol=1e-5)


def test_per_sample_normalized_flows_definitions():
    # map_flows_kernel / map_input_flows_kernel (queries/flow.jl:496-612): the shares of a sum node's
    # edges add up to one, a leaf gives everything to the observed category, and per-row parameter
    # vectors that all equal the circuit's give the circuit's answer
    rng = np.random.default_rng(2)
    fc = compile_circuit(st.simple_3vars_circuit(num_cats=5, fixed=False, rng=rng))
    data = rng.integers(0, 5, size=(6, 3)).astype(np.uint8)
    out = orc.per_sample_normalized_flows(fc, data)
    ni = orc.counts(fc)[0]
    np.testing.assert_allclose(np.exp(out[:, :ni]).sum(1), 1.0, rtol=1e-5)     # one sum node: the root
    leaf = out[:, ni:].reshape(6, -1, 5)
    for r in range(6):
        for i, nid in enumerate(fc.input_node_ids.astype(np.int64)):
            x = data[r, int(fc.node_var[nid - 1]) - 1]
            assert leaf[r, i, x] == 0.0 and np.isneginf(np.delete(leaf[r, i], x)).all()
    same = np.tile(orc.vectorize(fc), (6, 1))
    got = orc.per_sample_normalized_flows(fc, data, same)
    np.testing.assert_array_equal(np.isneginf(got), np.isneginf(out))
    np.testing.assert_allclose(np.exp(got), np.exp(out), atol=1e-6)
    # the root's edge flows are the posterior of the mixture component (flow_tests.jl:112-113)
    mars, em = orc.forward(fc, data, want_edge_mars=True)
    root_edges = np.nonzero(fc.up_parent == fc.num_nodes)[0]
    post = np.exp(em[:, root_edges] - mars[:, [-1]])
    e2p = orc.meta(fc)["edge2param"].astype(np.int64)
    np.testing.assert_allclose(np.exp(out[:, e2p[root_edges] - 1]), post, atol=1e-6)


def test_normalize_params_definitions():
    # normalize_params (misc.jl:363-392, 405-480): leaves become probabilities, sum groups are
    # log-normalised; undo takes log(p + 1e-6) of the leaves and normalises the sum groups again
    rng = np.random.default_rng(4)
    fc = compile_circuit(st.simple_3vars_circuit(num_cats=4, fixed=False, rng=rng))
    ni, nl, _ = orc.counts(fc)
    params = rng.normal(-1.0, 1.0, (3, ni + nl)).astype(np.float32)
    n = orc.normalize_params(fc, params)
    np.testing.assert_allclose(np.exp(n[:, :ni]).sum(1), 1.0, rtol=1e-5)         # the root's two edges
    np.testing.assert_allclose(n[:, ni:].reshape(3, -1, 4).sum(2), 1.0, rtol=1e-5)
    np.testing.assert_allclose(n[:, ni:ni + 4], np.exp(params[:, ni:ni + 4]) / np.exp(params[:, ni:ni + 4]).sum(1, keepdims=True),
                               rtol=1e-5)
    u = orc.normalize_params(fc, n, undo=True)
    np.testing.assert_allclose(u[:, ni:], np.log(n[:, ni:] + 1e-6), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(u[:, :ni], n[:, :ni], atol=1e-6)


def test_conditioned_td_prob_definitions():
    # conditioned_td_prob (queries/td_prob.jl:161-291): with the root marked and given probability one
    # the leaves' spread is the marginal of every variable; nothing flows without a marked node
    from tests.helpers import random_hclt
    fc = random_hclt(5, 3, 4, 1)
    N = fc.num_nodes
    mv, mc = np.zeros(N, np.int32), np.zeros(N, np.int32)
    out, td = orc.conditioned_td_prob(fc, mv, mc, np.ones((2, 1, 1), np.float32))
    assert not out.any() and not td.any()
    mv[N - 1] = mc[N - 1] = 1
    out, td = orc.conditioned_td_prob(fc, mv, mc, np.ones((2, 1, 1), np.float32))
    np.testing.assert_allclose(out.sum(2), 1.0, rtol=1e-5)
    # the marginal of variable v by brute force over all assignments
    import itertools
    grid = np.array(list(itertools.product(range(4), repeat=5)), np.uint8)
    p = np.exp(orc.forward(fc, grid)[:, -1].astype(np.float64))
    for v in range(5):
        want = np.array([p[grid[:, v] == c].sum() for c in range(4)])
        np.testing.assert_allclose(out[0, v], want, rtol=1e-4)
