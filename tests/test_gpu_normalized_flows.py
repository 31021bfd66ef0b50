"""pcb_normalized_flows (per_sample_normalized_flows, queries/flow.jl:417-612) against the oracle: with the
circuit's own parameters (the ordinary passes, tensor-core blocks included) and with one parameter
vector per data row (the gather passes)."""
import numpy as np
import pytest

from tests.helpers import random_data, random_hclt, simple3
from tests.test_gpu_kld_sample import _param_sets

pytestmark = pytest.mark.gpu
TOL = 1e-4

# row counts that are / are not multiples of four take the 16-byte and the scalar normalising kernel
CASES = [("simple3", lambda: simple3(False, 5, 0), 5, 9), ("hclt_k4", lambda: random_hclt(9, 4, 3, 1), 3, 36),
         ("hclt_k16_dense", lambda: random_hclt(8, 16, 4, 2), 4, 70), ("hclt_k32_dense", lambda: random_hclt(5, 32, 3, 3), 3, 40)]


def _compare(got, want):
    assert got.shape == want.shape
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    assert not np.isnan(got).any() and not np.isnan(want).any()
    np.testing.assert_allclose(np.exp(got), np.exp(want), atol=TOL, rtol=0)
    big = want > np.log(1e-3)
    np.testing.assert_allclose(got[big], want[big], atol=5 * TOL, rtol=0)


@pytest.mark.parametrize("name,make,c,rows", CASES, ids=[x[0] for x in CASES])
def test_normalized_flows_with_the_circuits_parameters(oracle, name, make, c, rows):
    import torch
    from lvd_pg_b200 import api
    fc = make()
    data, _ = random_data(rows, fc.num_vars, c, 4)
    m = api.CuMetaBitsProbCircuit(fc)
    want = oracle.per_sample_normalized_flows(fc, data)
    aggr_before, heap_before = m.edge_aggr().copy(), m.heap().copy()
    got = api.per_sample_normalized_flows(m, data, batch_size=32).cpu().numpy()
    _compare(got, want)
    # the call leaves the statistics alone (the reference hands edge_aggr = nothing)
    assert np.array_equal(m.edge_aggr(), aggr_before) and np.array_equal(m.heap(), heap_before)
    _compare(api.per_sample_normalized_flows(m, data, batch_size=30).cpu().numpy(), want)   # a batch that ends inside a quad
    # every sum node's shares add up to one (up to the 1e-8 guards)
    ni = m.num_inner_params
    e2p = m.edge2param.astype(np.int64)
    sums = np.zeros((rows, fc.num_nodes + 1))
    sel = np.nonzero(e2p > 0)[0]
    np.add.at(sums.T, fc.up_parent[sel].astype(np.int64), np.exp(got[:, e2p[sel] - 1]).T)
    parents = np.unique(fc.up_parent[sel])
    assert ni == len(sel)
    touched = sums[:, parents]
    assert np.all((np.abs(touched - 1.0) <= 1e-3) | (touched <= 1e-6))   # a node without flow keeps log(1e-8)


@pytest.mark.parametrize("name,make,c,rows", CASES[:3], ids=[x[0] for x in CASES[:3]])
def test_normalized_flows_with_per_row_parameters(oracle, name, make, c, rows):
    import torch
    from lvd_pg_b200 import api
    fc = make()
    rows = min(rows, 24)
    data, _ = random_data(rows, fc.num_vars, c, 7)
    m = api.CuMetaBitsProbCircuit(fc)
    params = _param_sets(oracle, fc, rows, 11)            # [rows, P] normalised log-parameters
    dparams = api.colmajor(params, m.device)
    got = api.per_sample_normalized_flows(m, data, dparams, batch_size=16).cpu().numpy()
    _compare(got, oracle.per_sample_normalized_flows(fc, data, params))
    # identical rows of parameters = the circuit's own parameters
    same = np.tile(oracle.vectorize(fc), (rows, 1))
    a = api.per_sample_normalized_flows(m, data, api.colmajor(same, m.device), batch_size=16).cpu().numpy()
    b = api.per_sample_normalized_flows(m, data, batch_size=16).cpu().numpy()
    _compare(a, b)


def test_normalize_params_and_column_mapping(oracle):
    """pcb_normalize_params (misc.jl:448-480, both directions) and pcb_map_param_columns
    (utils/map_params.jl:128-146) against the numpy restatement."""
    import torch
    from lvd_pg_b200 import api
    fc = random_hclt(7, 8, 3, 5)
    m = api.CuMetaBitsProbCircuit(fc)
    P = api.num_parameters(m)
    rng = np.random.default_rng(3)
    for S in (1, 5, 200):
        params = rng.normal(-1.0, 1.0, (S, P)).astype(np.float32)
        d = api.colmajor(params, m.device)
        want = oracle.normalize_params(fc, params)
        got = api.normalize_params(m, d).cpu().numpy()
        np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
        back = api.normalize_params(m, d, undo=True).cpu().numpy()
        np.testing.assert_allclose(back, oracle.normalize_params(fc, want, undo=True), rtol=1e-5, atol=1e-5)
    # column mapping: a random partial injection of columns
    S = 33
    src = rng.normal(size=(S, 50)).astype(np.float32)
    ids_src = (rng.permutation(50)[:20] + 1).astype(np.int32)
    ids_dst = (rng.permutation(P)[:20] + 1).astype(np.int32)
    dst = api.colmajor(np.zeros((S, P), np.float32), m.device)
    api.map_pc_parameters(dst, api.colmajor(src, m.device), torch.from_numpy(ids_dst).to(m.device),
                          torch.from_numpy(ids_src).to(m.device))
    want = np.zeros((S, P), np.float32)
    want[:, ids_dst - 1] = src[:, ids_src - 1]
    np.testing.assert_array_equal(dst.cpu().numpy(), want)


def test_normalized_flows_onto_a_latent_circuit(oracle):
    """normalized_flows_with_prealloc (utils/cuda_preallocation.jl:287-304) with the identity mapping of
    the sum parameters of a circuit onto a copy of itself: map, clamp to [-20, 0], normalise."""
    import torch
    from lvd_pg_b200 import api
    fc = random_hclt(6, 8, 3, 9)
    m = api.CuMetaBitsProbCircuit(fc)
    data, _ = random_data(20, fc.num_vars, 3, 2)
    ni = m.num_inner_params
    ids = torch.arange(1, ni + 1, dtype=torch.int32, device=m.device)
    got = api.normalized_flows(m, m, data, (ids, ids), batch_size=8).cpu().numpy()
    nf = oracle.per_sample_normalized_flows(fc, data)
    pz = np.zeros_like(nf)
    pz[:, :ni] = nf[:, :ni]
    want = oracle.normalize_params(fc, np.clip(pz, -20.0, 0.0))
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("S", [1, 7, 130])
def test_conditioned_td_prob(oracle, S):
    """pcb_cond_td_prob (queries/td_prob.jl:161-291): random marks on inner nodes, random node_probs."""
    import torch
    from lvd_pg_b200 import api
    fc = random_hclt(8, 6, 5, 12)
    m = api.CuMetaBitsProbCircuit(fc)
    N = fc.num_nodes
    rng = np.random.default_rng(S)
    inner = np.nonzero(fc.node_kind != 0)[0]
    marked = rng.choice(inner, size=len(inner) // 3, replace=False)
    Z1, Z2 = 4, 6
    mv, mc = np.zeros(N, np.int32), np.zeros(N, np.int32)
    mv[marked] = rng.integers(1, Z1 + 1, len(marked))
    mc[marked] = rng.integers(1, Z2 + 1, len(marked))
    mv[N - 1], mc[N - 1] = 1, 1                      # the root, so that something flows from the top
    node_probs = rng.random((S, Z1, Z2)).astype(np.float32)
    want, _ = oracle.conditioned_td_prob(fc, mv, mc, node_probs)
    got = api.conditioned_td_prob(m, torch.from_numpy(mv).to(m.device), torch.from_numpy(mc).to(m.device),
                                  api.colmajor(node_probs, m.device)).cpu().numpy()
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-6)
