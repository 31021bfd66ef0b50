"""The allocation-free hard-sampling entry point (pcb_sample_hard_static).

It exists for hosts that own all device memory themselves (CUDA.jl's pool, a serving arena): the
library must then not call cudaMalloc.  The tests drive it through the C ABI with caller-made
buffers only and check that it reproduces pcb_sample_hard exactly, twice in a row (the static
scratch keeps the first call's contents), that free device memory does not move across a call, and
that an oversized request is refused.  The file name sorts last so that a run stopping at the first
failure has already run every other test."""
import numpy as np
import pytest

from lvd_pg_b200 import structures as st
from tests.helpers import random_hclt

pytestmark = pytest.mark.gpu


def _two_calls(oracle, fc, sizes):
    import torch
    from lvd_pg_b200 import api
    m = api.CuMetaBitsProbCircuit(fc)
    flat = oracle.vectorize(fc)
    params = torch.from_numpy(flat).to(m.device).view(-1, 1).contiguous()   # [P, Sp = 1]
    rng = np.random.default_rng(8)
    for call, S in enumerate(sizes):          # second call: fewer samples over a dirty scratch
        shp = api.noise_shapes(m, S)
        u_sum = torch.from_numpy(rng.random(shp[0], dtype=np.float32)).to(m.device)
        u_leaf = torch.from_numpy(rng.random(shp[1], dtype=np.float32)).to(m.device)
        x_out = torch.full((fc.num_vars, S), -7, dtype=torch.int32, device=m.device)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(m.device)[0]
        x = api.sample_static(m, params, u_sum, u_leaf, x_out)
        torch.cuda.synchronize()
        # the first call in a process makes the CUDA runtime load the module that holds the array
        # (that is the runtime placing the library image, not an allocation by the call); from the
        # second call on, free device memory must not move at all
        if call > 0:
            assert torch.cuda.mem_get_info(m.device)[0] == free_before, f"call {call}: device memory moved"
        x = x.cpu().numpy()
        want = api.sample(m, params.t(), u_sum, u_leaf).cpu().numpy()
        assert np.array_equal(x, want), f"call {call}"
        assert np.array_equal(x, oracle.sample_hard(fc, flat, u_sum.cpu().numpy(), u_leaf.cpu().numpy(), S))
    return m, params


def test_static_scratch_sampling_matches_the_workspace_variant(oracle):
    import torch
    from lvd_pg_b200 import _lib
    fc = random_hclt(24, 32, 4, 21)
    m, params = _two_calls(oracle, fc, (300, 77))
    # beyond the static limit: S * (V + 2) > 2^20 words is refused before anything is launched
    S_big = (1 << 20) // (fc.num_vars + 2) + 1
    dummy = torch.zeros(4, device=m.device)
    with pytest.raises(_lib.PcbError) as e:
        _lib.check(m.lib.pcb_sample_hard_static(m.handle, params.data_ptr(), 1, dummy.data_ptr(), dummy.data_ptr(),
                                                S_big, dummy.data_ptr(), None))
    assert e.value.code == 4 and "static scratch" in str(e.value)


def test_walk_stacks_in_the_static_array(oracle):
    """A circuit with more than 12 286 variables: one warp's stack no longer fits 48 KB of shared
    memory, so the walk really runs on the static array (two calls, the second over what the first
    left there)."""
    V = 12400
    rng = np.random.default_rng(0)
    parent = st.root_tree_at_center(V, st.random_spanning_tree(V, rng))
    fc = st.hclt_flat(parent, 2, 2, seed=1)
    assert fc.num_vars + 2 > 48 * 1024 // 4
    _two_calls(oracle, fc, (6, 3))
