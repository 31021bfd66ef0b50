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
    got = api.per_sample_normalized_flows(m, data, batch_size=32).cpu().numpy()
    _compare(got, want)
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
