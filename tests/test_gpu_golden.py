"""The CUDA library against the committed golden vectors, through the C ABI."""
import numpy as np
import pytest

from tests.helpers import GOLDEN_CASES, flat_stats, load_golden, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden(name):
    import torch
    from lvd_pg_b200 import api
    g, fc = load_golden(name)
    m = api.CuMetaBitsProbCircuit(fc)
    rows = g["data"].shape[0]
    ll = torch.empty(rows, device=m.device)
    ws, B = api.forward(m, g["data"], ll_out=ll)
    assert rel_err(ll.cpu().numpy(), g["ll"]) <= 1e-5
    api.backward(m, ws)
    stats = flat_stats(fc, m.edge_aggr(), m.heap(), m.edge2param)
    assert rel_err(stats, g["stats"]) <= 1e-4
    m.lib.pcb_em_update(m.handle, float(g["pseudocount"]), float(g["inertia"]), None)
    assert np.abs(api.vectorize_parameters(m) - g["new_theta"]).max() <= 1e-4
    k, reuse = api.kld(m, g["theta"].astype(np.float32), g["theta2"].astype(np.float32))
    assert abs(k.item() - g["kld"]) <= 1e-4 * max(1.0, abs(g["kld"]))
    g1, g2 = api.kld_backward(m, reuse=reuse)
    ni = int(g["num_inner"])
    assert rel_err(g1.cpu().numpy()[0, :ni], g["kld_grad1"][:ni], 1e-3) <= 1e-4
    assert rel_err(g2.cpu().numpy()[0, :ni], g["kld_grad2"][:ni], 1e-3) <= 1e-4
