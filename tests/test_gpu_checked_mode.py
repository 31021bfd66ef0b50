"""Checked mode (PCB_CHECKED=1 when the circuit is created): every pass first validates what the batch
brings as indices (row ids, observed categories) with a kernel that touches only what it has found in
range, waits for it, and refuses the pass with the first finding; no kernel of the pass is launched on
a bad index, so these tests make no out-of-range access on the GPU.  The reference reads both under
@inbounds (queries/likelihood.jl:14, regularization/reg_likelihood.jl:16-49)."""
import numpy as np
import pytest

from tests.helpers import random_data, random_hclt

pytestmark = pytest.mark.gpu


def _cuda():
    import torch
    from lvd_pg_b200 import _lib, api
    assert torch.cuda.is_available()
    return torch, api, _lib


def test_checked_mode_passes_good_batches_and_refuses_bad_ones(oracle, monkeypatch):
    torch, api, _lib = _cuda()
    monkeypatch.setenv("PCB_CHECKED", "1")
    fc = random_hclt(9, 16, 5, 3)
    rows = 120
    data, miss = random_data(rows, fc.num_vars, 5, 4, 0.1)
    ref = fc.copy()
    m = api.CuMetaBitsProbCircuit(fc)
    dd = api.DeviceData(data, m.device, miss)
    ll = torch.zeros(1, device=m.device)

    # good batches: the checked step is the ordinary step
    ids = (np.random.default_rng(0).permutation(rows)[:64] + 1).astype(np.int32)
    ll_ref, _ = oracle.em_step(ref, data, miss=miss, row_ids=ids, pseudocount=0.1, inertia=0.5)
    api.em_step(m, dd, torch.from_numpy(ids).to(m.device), pseudocount=0.1, inertia=0.5, ll_sum=ll)
    assert abs(ll.item() - ll_ref) <= 1e-4 * abs(ll_ref)
    p_after = api.vectorize_parameters(m).copy()
    assert np.abs(np.exp(p_after) - np.exp(oracle.vectorize(ref))).max() <= 1e-4

    # a row id below 1 and one past the last row: refused, parameters and statistics untouched
    for bad in (0, rows + 1, -5):
        ids_bad = ids.copy()
        ids_bad[17] = bad
        with pytest.raises(_lib.PcbError) as e:
            api.em_step(m, dd, torch.from_numpy(ids_bad).to(m.device), pseudocount=0.1, inertia=0.5, ll_sum=ll)
        assert e.value.code == 1 and "example 17" in str(e.value) and f"row {bad}" in str(e.value)
        assert np.array_equal(api.vectorize_parameters(m), p_after)
    with pytest.raises(_lib.PcbError):
        api.forward(m, dd, torch.from_numpy(np.array([1, 2, rows + 7], np.int32)).to(m.device))

    # an observed value that the variable's leaves have no category for (a missing cell may hold anything)
    data_bad = data.copy()
    cell = np.argwhere(miss == 0)[5]
    data_bad[cell[0], cell[1]] = 5
    hidden = np.argwhere(miss != 0)[0]
    data_bad[hidden[0], hidden[1]] = 200
    dd_bad = api.DeviceData(data_bad, m.device, miss)
    with pytest.raises(_lib.PcbError) as e:
        api.forward(m, dd_bad)
    assert e.value.code == 1 and f"variable {cell[1] + 1}" in str(e.value) and "value 5" in str(e.value)

    # the context is intact and the circuit goes on
    ll_ref2, _ = oracle.em_step(ref, data, miss=miss, row_ids=ids, pseudocount=0.1, inertia=0.5)
    api.em_step(m, dd, torch.from_numpy(ids).to(m.device), pseudocount=0.1, inertia=0.5, ll_sum=ll)
    assert abs(ll.item() - ll_ref2) <= 1e-4 * abs(ll_ref2)
    _lib.check(m.lib.pcb_circuit_status(m.handle))
