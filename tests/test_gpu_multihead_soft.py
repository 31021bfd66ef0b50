"""CUDA path vs the CPU oracle on multi-head circuits, soft evidence and soft-regularised leaves
(through pcb_forward_ex / pcb_em_step_ex), and the reference's own known answers for the multi-head case."""
import numpy as np
import pytest

from lvd_pg_b200 import structures as st
from lvd_pg_b200.circuit import Sum, compile_circuit, compile_multihead
from tests.helpers import random_data, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4  # relative, fp32


def _cuda():
    import torch
    from lvd_pg_b200 import api
    assert torch.cuda.is_available()
    return torch, api


def _multihead_hclt(v, k, c, heads, seed):
    """`heads` root mixtures over the sub-circuits of one HCLT root."""
    rng = np.random.default_rng(seed)
    parent = st.root_tree_at_center(v, st.random_spanning_tree(v, rng))
    root = st.hclt_graph(parent, c, k, rng)
    pcs = []
    for _ in range(heads):
        w = rng.dirichlet(np.ones(len(root.children)))
        pcs.append(Sum(list(root.children), np.log(w).astype(np.float32)))
    return compile_multihead(pcs)


def _mask(rows, heads, seed):
    rng = np.random.default_rng(seed)
    mask = rng.random((rows, heads)).astype(np.float32)
    mask[rng.random((rows, heads)) < 0.4] = 0.0
    mask[np.arange(rows), rng.integers(0, heads, rows)] += 0.5   # no all-zero row
    return mask


def test_reference_known_answers():
    # test/multi_head_pc/multi_head_pc_learning_tests.jl:11-50
    torch, api = _cuda()
    pcs = st.simple_multihead_circuit(num_cats=5)
    pcs[0].children[0].children[0].logps[:] = np.log(np.array([0.1, 0.2, 0.3, 0.3, 0.1], np.float32))
    pcs[0].logps[:] = np.log(np.array([0.2, 0.8], np.float32))
    pcs[1].logps[:] = np.log(np.array([0.6, 0.4], np.float32))
    m = api.CuMultiHeadBitsProbCircuit(pcs)
    assert m.root_ids.tolist() == [9, 10]
    data = api.DeviceData(np.array([[0, 0, 0], [2, 0, 0]], np.uint8), m.device)
    mask = api.colmajor(np.array([[1.0, 0.0], [0.0, 1.0]], np.float32), m.device)
    lls = api.multihead_loglikelihoods(m, data, mask, batch_size=2).cpu().numpy()
    np.testing.assert_allclose(lls[0], np.log(0.1 * 0.2 * 0.2 * 0.2 + 0.2 ** 3 * 0.8), rtol=1e-5)
    np.testing.assert_allclose(lls[1], np.log(0.3 * 0.2 * 0.2 * 0.6 + 0.2 ** 3 * 0.4), rtol=1e-5)

    ws, B = api.forward_ex(m, data, head_mask=mask, soft_reg=0.01, soft_reg_width=3)
    m.lib.pcb_clear_flows(m.handle, 0.0, None)
    api.backward(m, ws)
    mars, flows = m.mars(ws, B), m.flows(ws, B)
    f = lambda b, n: flows[b - 1, n - 1]
    mm = lambda b, n: mars[b - 1, n - 1]
    l = lambda x: np.log(np.float32(x))
    np.testing.assert_allclose([f(1, 9), f(1, 10), f(2, 9), f(2, 10)], [1.0, 0.0, 0.0, 1.0])
    np.testing.assert_allclose(flows[:, 10], 0.0)
    np.testing.assert_allclose(f(1, 4), np.exp(mm(1, 1) + mm(1, 2) + mm(1, 3) + l(0.2) - mm(1, 9)), rtol=1e-5)
    np.testing.assert_allclose(f(1, 8), np.exp(mm(1, 5) + mm(1, 6) + mm(1, 7) + l(0.8) - mm(1, 9)), rtol=1e-5)
    np.testing.assert_allclose(f(2, 4), np.exp(mm(2, 1) + mm(2, 2) + mm(2, 3) + l(0.6) - mm(2, 10)), rtol=1e-5)
    np.testing.assert_allclose(f(2, 8), np.exp(mm(2, 5) + mm(2, 6) + mm(2, 7) + l(0.4) - mm(2, 10)), rtol=1e-5)


def test_flows_of_a_multihead_circuit_need_a_mask():
    torch, api = _cuda()
    from lvd_pg_b200 import _lib
    m = api.CuMultiHeadBitsProbCircuit(st.simple_multihead_circuit(num_cats=5))
    data = api.DeviceData(np.zeros((4, 3), np.uint8), m.device)
    ws, B = api.forward_ex(m, data)
    with pytest.raises(_lib.PcbError):
        api.backward(m, ws)
    with pytest.raises(_lib.PcbError):
        api.em_step_ex(m, data)


MH_CASES = [("k4_sparse", 7, 4, 3, 3, 45), ("k16_dense", 9, 16, 4, 2, 100), ("k32_dense", 6, 32, 5, 5, 70),
            ("k16_heads_in_a_dense_block", 6, 16, 3, 16, 60)]


@pytest.mark.parametrize("name,v,k,c,heads,rows", MH_CASES, ids=[x[0] for x in MH_CASES])
def test_multihead_forward_backward_and_steps(oracle, name, v, k, c, heads, rows):
    torch, api = _cuda()
    fc, roots = _multihead_hclt(v, k, c, heads, seed=21)
    ref = fc.copy()
    m = api.CuMultiHeadBitsProbCircuit(fc)
    assert m.root_ids.tolist() == roots.tolist()
    data, miss = random_data(rows, v, c, 5, 0.1)
    mask = _mask(rows, heads, 9)
    dd = api.DeviceData(data, m.device, miss)
    dmask = api.colmajor(mask, m.device)

    # likelihoods, with and without a mask
    mars_ref = oracle.forward_ex(ref, data, miss=miss)
    got = api.multihead_loglikelihoods(m, dd, dmask, batch_size=32).cpu().numpy()
    assert rel_err(got, oracle.multihead_lls(ref, mars_ref, roots, mask)) <= TOL
    got = api.multihead_loglikelihoods(m, dd, None, batch_size=32).cpu().numpy()
    assert got.shape == (rows, heads)
    assert rel_err(got, oracle.multihead_lls(ref, mars_ref, roots, None)) <= TOL

    # flows from the head mask, on a permuted batch
    ids = (np.random.default_rng(2).permutation(rows)[:rows - 3] + 1).astype(np.int32)
    dids = torch.from_numpy(ids).to(m.device)
    mars_ref = oracle.forward_ex(ref, data, row_ids=ids, miss=miss)
    flows_ref, aggr_ref = oracle.backward_ex(ref, mars_ref, roots, mask, row_ids=ids)
    oracle.input_flows_ex(ref, flows_ref, data, row_ids=ids, miss=miss)
    ws, B = api.forward_ex(m, dd, head_mask=dmask, row_ids=dids)
    m.lib.pcb_clear_flows(m.handle, 0.0, None)
    api.backward(m, ws)
    assert rel_err(m.flows(ws, B), flows_ref) <= TOL
    sum_edges = ref.edge_is_sum[ref.down2up.astype(np.int64) - 1]
    assert rel_err(m.edge_aggr()[sum_edges], aggr_ref[sum_edges]) <= TOL
    assert rel_err(m.heap(), ref.heap) <= TOL

    # EM steps (the third replays the captured graph), with flow memory
    ref = fc.copy()
    api.update_parameters(m, oracle.vectorize(ref))
    ll = torch.zeros(1, device=m.device)
    aggr = np.zeros(ref.num_edges, np.float32)
    for step in range(4):
        rate = 0.0 if step == 0 else 0.7
        ll_ref, _ = oracle.em_step_ex(ref, data, head_roots=roots, head_mask=mask, row_ids=ids, pseudocount=0.1,
                                      inertia=0.2, miss=miss, edge_aggr=aggr, clear_rate=rate)
        api.em_step_ex(m, dd, head_mask=dmask, row_ids=dids, pseudocount=0.1, inertia=0.2, clear_rate=rate, ll_sum=ll)
        assert abs(float(ll.item()) - ll_ref) <= TOL * abs(ll_ref)
        p = api.vectorize_parameters(m)
        assert np.abs(np.exp(p) - np.exp(oracle.vectorize(ref))).max() <= TOL


def test_mini_batch_em_for_multihead_pc_improves_the_likelihood():
    torch, api = _cuda()
    fc, roots = _multihead_hclt(8, 8, 4, 3, seed=4)
    m = api.CuMultiHeadBitsProbCircuit(fc)
    data, _ = random_data(256, 8, 4, 6)
    mask = api.colmajor(_mask(256, 3, 1), m.device)
    lls = api.mini_batch_em_for_multihead_pc(m, data, mask, 6, batch_size=64, pseudocount=0.1, param_inertia=0.3,
                                             seed=0)
    assert len(lls) == 6 and all(np.isfinite(lls)) and lls[-1] > lls[0]


SOFT_CASES = [("simple3", None, 5, 9), ("hclt_k4", (9, 4, 3), 3, 37), ("hclt_k16_dense", (12, 16, 4), 4, 100),
              ("hclt_k32_c40", (6, 32, 40), 40, 66)]


def _soft_case(case, c):
    if case is None:
        return compile_circuit(st.simple_3vars_circuit(num_cats=c, fixed=False, rng=np.random.default_rng(0)))
    v, k, cc = case
    rng = np.random.default_rng(31)
    parent = st.root_tree_at_center(v, st.random_spanning_tree(v, rng))
    return st.hclt_flat(parent, cc, k, seed=7)


@pytest.mark.parametrize("name,case,c,rows", SOFT_CASES, ids=[x[0] for x in SOFT_CASES])
def test_soft_evidence(oracle, name, case, c, rows):
    torch, api = _cuda()
    fc = _soft_case(case, c)
    ref = fc.copy()
    m = api.CuMetaBitsProbCircuit(fc)
    rng = np.random.default_rng(17)
    soft = np.log(rng.dirichlet(np.full(c, 0.3), size=(rows, fc.num_vars)) + 1e-30).astype(np.float32)
    soft[rng.random(soft.shape) < 0.1] = -np.inf          # impossible categories
    soft[:, :, 0] = np.maximum(soft[:, :, 0], -20.0)      # never a whole row of them
    dsoft = api.colmajor(soft, m.device)
    w = rng.random(rows).astype(np.float32) + 0.5
    dw = torch.from_numpy(w).to(m.device)

    mars_ref = oracle.forward_ex(ref, soft=soft)
    ll = torch.empty(rows, device=m.device)
    ws, B = api.forward_ex(m, soft=dsoft, ll_out=ll)
    mars = m.mars(ws, B)
    assert np.abs(mars - mars_ref).max() <= TOL * max(1.0, np.abs(mars_ref).max())
    assert rel_err(ll.cpu().numpy(), mars_ref[:, -1]) <= TOL

    flows_ref, aggr_ref = oracle.backward(ref, mars_ref)
    oracle.input_flows_ex(ref, flows_ref, soft=soft, weights=w)
    m.lib.pcb_clear_flows(m.handle, 0.0, None)
    api.backward(m, ws, dw)
    assert rel_err(m.flows(ws, B), flows_ref) <= TOL
    assert rel_err(m.heap(), ref.heap) <= TOL

    ref = fc.copy()
    api.update_parameters(m, oracle.vectorize(ref))
    ids = (rng.permutation(rows)[:rows - 2] + 1).astype(np.int32)
    dids = torch.from_numpy(ids).to(m.device)
    lls = torch.zeros(1, device=m.device)
    for step in range(3):
        ll_ref, _ = oracle.em_step_ex(ref, soft=soft, row_ids=ids, pseudocount=0.1, inertia=0.1, weights=w)
        api.em_step_ex(m, soft=dsoft, row_ids=dids, pseudocount=0.1, inertia=0.1, weights=dw, ll_sum=lls)
        assert abs(float(lls.item()) - ll_ref) <= TOL * abs(ll_ref)
        p = api.vectorize_parameters(m)
        assert np.abs(np.exp(p) - np.exp(oracle.vectorize(ref))).max() <= TOL


def test_one_hot_soft_evidence_equals_hard_evidence_on_the_gpu():
    torch, api = _cuda()
    fc = _soft_case((9, 16, 5), 5)
    m = api.CuMetaBitsProbCircuit(fc)
    data, _ = random_data(50, 9, 5, 3)
    soft = np.full((50, 9, 5), -np.inf, np.float32)
    np.put_along_axis(soft, data[:, :, None].astype(np.int64), 0.0, axis=2)
    a = torch.empty(50, device=m.device)
    b = torch.empty(50, device=m.device)
    api.forward(m, api.DeviceData(data, m.device), ll_out=a)
    api.forward_ex(m, soft=api.colmajor(soft, m.device), ll_out=b)
    assert rel_err(b.cpu().numpy(), a.cpu().numpy()) <= 1e-6


@pytest.mark.parametrize("width", [1, 3, 6])
def test_soft_regularised_leaves(oracle, width):
    # mini_batch_em_with_reg with soft_reg > 0 on hard evidence (reg_likelihood.jl:4-49, reg_flow.jl:3-48)
    torch, api = _cuda()
    fc = _soft_case((8, 16, 12), 12)
    ref = fc.copy()
    m = api.CuMetaBitsProbCircuit(fc)
    rows = 77
    data, miss = random_data(rows, 8, 12, 8, 0.15)
    dd = api.DeviceData(data, m.device, miss)
    mars_ref = oracle.forward_ex(ref, data, miss=miss, soft_reg=0.05, soft_reg_width=width)
    ws, B = api.forward_ex(m, dd, soft_reg=0.05, soft_reg_width=width)
    mars = m.mars(ws, B)
    assert np.abs(mars - mars_ref).max() <= TOL * max(1.0, np.abs(mars_ref).max())
    flows_ref, aggr_ref = oracle.backward(ref, mars_ref)
    oracle.input_flows_ex(ref, flows_ref, data, miss=miss, soft_reg=0.05, soft_reg_width=width)
    m.lib.pcb_clear_flows(m.handle, 0.0, None)
    api.backward(m, ws)
    assert rel_err(m.heap(), ref.heap) <= TOL
    lls = torch.zeros(1, device=m.device)
    ref = fc.copy()
    api.update_parameters(m, oracle.vectorize(ref))
    for step in range(3):
        ll_ref, _ = oracle.em_step_ex(ref, data, miss=miss, pseudocount=0.2, inertia=0.0, soft_reg=0.05,
                                      soft_reg_width=width)
        api.em_step_ex(m, dd, pseudocount=0.2, inertia=0.0, soft_reg=0.05, soft_reg_width=width, ll_sum=lls)
        assert abs(float(lls.item()) - ll_ref) <= TOL * abs(ll_ref)
        p = api.vectorize_parameters(m)
        assert np.abs(np.exp(p) - np.exp(oracle.vectorize(ref))).max() <= TOL
