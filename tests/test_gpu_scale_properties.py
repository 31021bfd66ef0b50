"""Size-independent properties of the CUDA path at a workload far beyond what the oracle can follow:
an image HCLT with 256 latents and 256 categories (the block shape of the headline workload, cut
to 96 variables), batch 2048.  No oracle involved: the checks are identities of the algorithm."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _setup(monkeypatch=None, env=None):
    import torch
    from lvd_pg_b200 import api, synth
    assert torch.cuda.is_available()
    if env:
        for k, v in env.items():
            monkeypatch.setenv(k, v)
    images, fc = synth.image_hclt(256, 4096, 32, 2.0, 3, "cuda", num_vars=96)
    m = api.CuMetaBitsProbCircuit(fc, 0)
    dd = api.DeviceData(images, torch.device("cuda", 0))
    return torch, api, fc, m, dd


def _group_sums(fc, m, api):
    """Sum of probabilities of every sum group and of every leaf categorical."""
    p = np.exp(np.asarray(api.vectorize_parameters(m), np.float64))
    n_inner = int(m.info.num_inner_params)
    inner = p[:n_inner]
    leaf = p[n_inner:].reshape(-1, 256)
    return inner, leaf, 256


def test_flow_conservation_and_normalisation():
    torch, api, fc, m, dd = _setup()
    ids = torch.arange(1, 2049, dtype=torch.int32, device="cuda")
    ws, B = api.forward(m, dd, ids)
    api.backward(m, ws)
    flows = m.flows(ws, B)          # [B, N]
    mars = m.mars(ws, B)
    assert np.isfinite(mars[:, -1]).all()
    # the root carries flow 1 for every example and every variable's leaves share exactly that flow
    assert np.allclose(flows[:, -1], 1.0, atol=1e-5)
    ids_in = np.asarray(fc.input_node_ids) - 1
    var = np.asarray(fc.node_var)[ids_in]
    for v in (1, 7, 96):
        tot = flows[:, ids_in[var == v]].sum(axis=1)
        assert np.abs(tot - 1.0).max() <= 2e-4, (v, np.abs(tot - 1.0).max())
    # leaf statistics: the flow slots of a variable's leaves add up to the number of examples
    heap = m.heap()
    hs = np.asarray(fc.node_heap_start)[ids_in] - 1
    for v in (1, 50):
        s = sum(heap[h + 256:h + 513].sum() for h in hs[var == v])
        assert abs(s - B) <= 2e-4 * B, (v, s)
    # edge statistics: all edge flows out of the root's block add up to the batch size
    agg = m.edge_aggr()
    assert agg.sum() > 0
    # one EM step keeps every sum group and every leaf normalised
    ll = torch.zeros(1, device="cuda")
    api.em_step(m, dd, ids, pseudocount=0.1, inertia=0.9, ll_sum=ll)
    inner, leaf, k = _group_sums(fc, m, api)
    assert np.abs(leaf.sum(axis=1) - 1.0).max() <= 1e-4
    blocks = inner.reshape(-1, k)   # every sum node of this circuit has k edges, consecutive in the flat order
    assert np.abs(blocks.sum(axis=1) - 1.0).max() <= 1e-4
    assert abs(ll.item() - mars[:, -1].sum()) <= 1e-4 * abs(ll.item())


def test_full_batch_em_is_monotone_and_graph_replay_matches_plain_launches(monkeypatch):
    torch, api, fc, m, dd = _setup()
    ids = torch.arange(1, 2049, dtype=torch.int32, device="cuda")
    ll = torch.zeros(1, device="cuda")
    lls = []
    for _ in range(5):   # steps 3.. replay the captured graph
        api.em_step(m, dd, ids, pseudocount=0.1, inertia=0.0, ll_sum=ll)
        lls.append(ll.item())
    assert all(b >= a - 1e-4 * abs(a) for a, b in zip(lls, lls[1:])), lls   # EM on a fixed batch never loses likelihood
    p_graph = np.asarray(api.vectorize_parameters(m))
    # the same five steps with plain launches, no side stream, no dependent launches
    torch2, api2, fc2, m2, dd2 = _setup(monkeypatch, {"PCB_NO_GRAPH": "1", "PCB_NO_PDL": "1", "PCB_NO_SIDE_STREAM": "1"})
    lls2 = []
    for _ in range(5):
        api2.em_step(m2, dd2, ids, pseudocount=0.1, inertia=0.0, ll_sum=ll)
        lls2.append(ll.item())
    p_plain = np.asarray(api2.vectorize_parameters(m2))
    assert np.allclose(lls, lls2, rtol=1e-5)
    assert np.abs(np.exp(p_graph) - np.exp(p_plain)).max() <= 1e-4


def test_row_range_and_row_ids_agree():
    torch, api, fc, m, dd = _setup()
    ll_a, ll_b = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    ids = torch.arange(101, 101 + 1024, dtype=torch.int32, device="cuda")
    p0 = np.asarray(api.vectorize_parameters(m)).copy()
    api.em_step(m, dd, ids, pseudocount=0.1, inertia=0.9, ll_sum=ll_a)
    pa = np.asarray(api.vectorize_parameters(m)).copy()
    api.update_parameters(m, p0)
    api.em_step(m, dd, None, row_start=101, B=1024, pseudocount=0.1, inertia=0.9, ll_sum=ll_b)
    pb = np.asarray(api.vectorize_parameters(m))
    assert abs(ll_a.item() - ll_b.item()) <= 1e-5 * abs(ll_a.item())
    assert np.abs(np.exp(pa) - np.exp(pb)).max() <= 1e-5
