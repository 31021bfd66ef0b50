"""CUDA path vs the CPU oracle: forward, backward, leaf statistics, EM update (through the C ABI)."""
import numpy as np
import pytest

from tests.helpers import random_data, random_hclt, rel_err, simple3

pytestmark = pytest.mark.gpu
TOL = 1e-4  # relative, fp32 (the tolerance the north star states)


def _cuda():
    import torch
    from lvd_pg_b200 import api
    assert torch.cuda.is_available()
    return torch, api


CASES = [
    ("simple3", lambda: simple3(False, 5, 0), 5, 2),
    ("hclt_k4", lambda: random_hclt(9, 4, 3, 1), 3, 37),
    ("hclt_k16_dense", lambda: random_hclt(12, 16, 2, 2), 2, 100),
    ("hclt_k32_dense", lambda: random_hclt(20, 32, 7, 3), 7, 130),
    ("hclt_k48_ragged", lambda: random_hclt(7, 48, 5, 4), 5, 33),
    ("hclt_k128_dense", lambda: random_hclt(5, 128, 3, 5), 3, 260),
    ("hclt_k256_dense", lambda: random_hclt(4, 256, 2, 6), 2, 131),
    ("hclt_k272_two_column_tiles", lambda: random_hclt(3, 272, 2, 8), 2, 70),
]


@pytest.mark.parametrize("name,make,c,rows", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("missing", [0.0, 0.2])
def test_forward_backward_update(oracle, name, make, c, rows, missing):
    torch, api = _cuda()
    fc = make()
    data, miss = random_data(rows, fc.num_vars, c, 11, missing)
    ref = fc.copy()
    m = api.CuMetaBitsProbCircuit(fc)
    dd = api.DeviceData(data, m.device, miss)

    # forward
    mars_ref = oracle.forward(ref, data, miss=miss)
    ll = torch.empty(rows, device=m.device)
    ws, B = api.forward(m, dd, ll_out=ll)
    mars = m.mars(ws, B)
    assert np.abs(mars - mars_ref).max() <= TOL * max(1.0, np.abs(mars_ref).max())
    assert rel_err(ll.cpu().numpy(), mars_ref[:, -1]) <= TOL

    # backward + leaf statistics
    flows_ref, aggr_ref = oracle.backward(ref, mars_ref)
    oracle.input_flows(ref, flows_ref, data, miss=miss)
    m.lib.pcb_clear_flows(m.handle, 0.0, None)
    api.backward(m, ws)
    flows = m.flows(ws, B)
    assert rel_err(flows, flows_ref) <= TOL
    sum_edges = ref.edge_is_sum[ref.down2up.astype(np.int64) - 1]
    assert rel_err(m.edge_aggr()[sum_edges], aggr_ref[sum_edges]) <= TOL
    assert rel_err(m.heap(), ref.heap) <= TOL

    # M-step
    oracle.em_update(ref, aggr_ref, 0.1, 0.3)
    m.lib.pcb_em_update(m.handle, 0.1, 0.3, None)
    p = api.vectorize_parameters(m)
    p_ref = oracle.vectorize(ref)
    assert np.abs(p - p_ref).max() <= TOL * max(1.0, np.abs(p_ref).max())
    assert np.abs(np.exp(p) - np.exp(p_ref)).max() <= TOL


def test_dense_and_sparse_paths_agree(oracle, monkeypatch):
    torch, api = _cuda()
    fc = random_hclt(15, 32, 4, 7)
    data, _ = random_data(64, fc.num_vars, 4, 3)
    m_dense = api.CuMetaBitsProbCircuit(fc)
    assert m_dense.info.num_dense_blocks > 0
    monkeypatch.setenv("PCB_DISABLE_DENSE", "1")
    m_sparse = api.CuMetaBitsProbCircuit(fc)
    assert m_sparse.info.num_dense_blocks == 0
    outs = []
    for m in (m_dense, m_sparse):
        api.em_step(m, data, pseudocount=0.1, inertia=0.5)
        outs.append((api.vectorize_parameters(m), m.edge_aggr()))
    assert np.abs(outs[0][0] - outs[1][0]).max() <= TOL
    assert rel_err(outs[0][1], outs[1][1]) <= TOL


def test_tensor_core_and_simt_dense_kernels_agree(monkeypatch):
    torch, api = _cuda()
    fc = random_hclt(9, 64, 4, 12)
    data, _ = random_data(300, fc.num_vars, 4, 5)
    outs = []
    for impl in ("tc", "simt"):
        monkeypatch.setenv("PCB_DENSE_IMPL", impl)
        m = api.CuMetaBitsProbCircuit(fc)
        assert m.info.num_dense_blocks > 0
        ll = torch.zeros(1, device=m.device)
        api.em_step(m, data, pseudocount=0.1, inertia=0.5, ll_sum=ll)
        outs.append((api.vectorize_parameters(m), m.edge_aggr(), ll.item()))
    assert abs(outs[0][2] - outs[1][2]) <= 1e-5 * abs(outs[1][2])
    assert np.abs(outs[0][0] - outs[1][0]).max() <= TOL
    assert rel_err(outs[0][1], outs[1][1]) <= TOL


def test_example_major_and_k_major_tensor_core_kernels_agree(monkeypatch):
    """The kernels that read the data-dependent operand example-major (pcb_dense_mn.cu, the default)
    against the K-major staging kernels of pcb_dense_tc.cu (PCB_TC_IMPL=km), ragged and full tiles,
    with and without column splits."""
    torch, api = _cuda()
    for fc, rows in ((random_hclt(6, 256, 3, 31), 300), (random_hclt(9, 80, 4, 32), 77)):
        data, _ = random_data(rows, fc.num_vars, int(fc.meta["num_cats"]), 5)
        outs = []
        for impl, nsplit in (("mn", "0"), ("km", "0"), ("mn", "1"), ("mn", "4")):
            monkeypatch.setenv("PCB_TC_IMPL", impl)
            monkeypatch.setenv("PCB_TC_NSPLIT", nsplit)
            m = api.CuMetaBitsProbCircuit(fc.copy())
            assert m.info.num_dense_blocks > 0
            ll = torch.zeros(1, device=m.device)
            ws = api.em_step(m, data, pseudocount=0.1, inertia=0.5, ll_sum=ll)
            outs.append((api.vectorize_parameters(m), m.edge_aggr(), ll.item(), m.flows(ws, rows)))
        assert np.isfinite(outs[0][2]) and np.isfinite(outs[0][0]).all()
        for o in outs[1:]:
            assert abs(o[2] - outs[0][2]) <= 1e-5 * abs(outs[0][2])
            assert np.abs(np.exp(o[0]) - np.exp(outs[0][0])).max() <= TOL
            assert rel_err(o[1], outs[0][1]) <= TOL
            assert rel_err(o[3], outs[0][3]) <= TOL


def test_k_split_of_small_dense_layers_agrees_with_the_unsplit_kernels(oracle, monkeypatch):
    """Layers of one or two blocks split the K range over 2 or 4 CTAs that hand their partial tiles over
    through a scratch slot (PCB_TC_KSPLIT forces the split, 1 turns it off): values, flows, statistics and
    the updated parameters against the unsplit kernels and the oracle; the second and third step replay
    the captured graph, i.e. run on the arrival counters the step before left behind."""
    torch, api = _cuda()
    for fc, rows, c in ((random_hclt(5, 256, 3, 41), 200, 3), (random_hclt(7, 128, 4, 42), 131, 4), (random_hclt(6, 64, 2, 43), 64, 2)):
        data, miss = random_data(rows, fc.num_vars, c, 6, 0.1)
        ref = fc.copy()
        mars_ref = oracle.forward(ref, data, miss=miss)
        flows_ref, _ = oracle.backward(ref, mars_ref)
        outs = []
        for ks in ("1", "2", "4"):
            monkeypatch.setenv("PCB_TC_KSPLIT", ks)
            m = api.CuMetaBitsProbCircuit(fc.copy())
            dd = api.DeviceData(data, m.device, miss)
            ll = torch.zeros(1, device=m.device)
            ws = api.em_step(m, dd, pseudocount=0.1, inertia=0.5, ll_sum=ll)
            first = (m.mars(ws, rows), m.flows(ws, rows), m.edge_aggr(), ll.item())
            for _ in range(2):
                api.em_step(m, dd, pseudocount=0.1, inertia=0.5, ll_sum=ll)
            outs.append(first + (api.vectorize_parameters(m), ll.item()))
            _lib_check_status(m)
        assert np.abs(outs[0][0] - mars_ref).max() <= TOL * max(1.0, np.abs(mars_ref).max())
        for o in outs:
            assert np.isfinite(o[3]) and np.isfinite(o[5])
            assert np.abs(o[0] - mars_ref).max() <= TOL * max(1.0, np.abs(mars_ref).max())
            assert rel_err(o[1], flows_ref) <= TOL
            assert rel_err(o[2], outs[0][2]) <= TOL
            assert abs(o[5] - outs[0][5]) <= 1e-5 * abs(outs[0][5])
            assert np.abs(np.exp(o[4]) - np.exp(outs[0][4])).max() <= TOL


def _lib_check_status(m):
    from lvd_pg_b200 import _lib
    _lib.check(m.lib.pcb_circuit_status(m.handle))


def test_em_steps_track_oracle_with_row_ids(oracle):
    torch, api = _cuda()
    fc = random_hclt(10, 16, 3, 5)
    data, _ = random_data(300, fc.num_vars, 3, 9)
    ref = fc.copy()
    m = api.CuMetaBitsProbCircuit(fc)
    dd = api.DeviceData(data, m.device)
    rng = np.random.default_rng(0)
    ll_dev = torch.zeros(1, device=m.device)
    # the second identical call captures the step as a CUDA graph, later ones replay it: every step
    # brings its own row ids
    for step in range(5):
        ids = (rng.permutation(300)[:128] + 1).astype(np.int32)
        ll_ref, _ = oracle.em_step(ref, data, row_ids=ids, pseudocount=0.1, inertia=0.9)
        api.em_step(m, dd, torch.from_numpy(ids).to(m.device), pseudocount=0.1, inertia=0.9, ll_sum=ll_dev)
        assert abs(ll_dev.item() - ll_ref) <= TOL * abs(ll_ref)
        p, p_ref = api.vectorize_parameters(m), oracle.vectorize(ref)
        assert np.abs(np.exp(p) - np.exp(p_ref)).max() <= TOL


@pytest.mark.parametrize("impl", ["atomic", "sorted"])
@pytest.mark.parametrize("cats,rows,missing", [(3, 77, 0.3), (40, 300, 0.0), (256, 2500, 0.1)])
def test_leaf_statistics_kernels_agree_with_oracle(oracle, monkeypatch, impl, cats, rows, missing):
    """Both leaf-statistics kernels (shared-memory histogram with atomics, sorted segments) against the
    oracle: few and many categories, missing values, more rows than one block slice, example weights."""
    torch, api = _cuda()
    monkeypatch.setenv("PCB_LEAF_FLOW_IMPL", impl)
    fc = random_hclt(5, 16, cats, 21)
    data, miss = random_data(rows, fc.num_vars, cats, 4, missing)
    w = np.random.default_rng(8).uniform(0.5, 1.5, rows).astype(np.float32)
    for weights in (None, w):
        m = api.CuMetaBitsProbCircuit(fc.copy())
        dd = api.DeviceData(data, m.device, miss)
        ws, B = api.forward(m, dd)
        api.backward(m, ws, None if weights is None else torch.from_numpy(weights).to(m.device))
        heap = m.heap()
        ref = fc.copy()
        mars = oracle.forward(ref, data, miss=miss)
        flows, _ = oracle.backward(ref, mars)
        oracle.input_flows(ref, flows, data, miss=miss, weights=weights)
        scale = max(1e-6, float(np.abs(ref.heap).max()))
        assert np.abs(heap - ref.heap).max() <= TOL * scale


def test_params_roundtrip_and_errors(oracle):
    torch, api = _cuda()
    from lvd_pg_b200._lib import PcbError
    fc = simple3(False)
    m = api.CuMetaBitsProbCircuit(fc)
    assert api.num_parameters(m) == 32
    p = api.vectorize_parameters(m)
    assert np.array_equal(p, oracle.vectorize(fc))
    q = p + 0.25
    api.update_parameters(m, q)
    assert np.array_equal(api.vectorize_parameters(m), q)
    with pytest.raises(AssertionError):
        api.update_parameters(m, q[:-1])
    ws = m.workspace(4)
    with pytest.raises(PcbError):  # backward without forward
        api.backward(m, ws)
    bad = fc.copy()
    bad.up_prime[0] = 99
    with pytest.raises(PcbError):
        api.CuMetaBitsProbCircuit(bad)
