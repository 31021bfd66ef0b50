"""Failure handling that involves a GPU, without faulting, trapping or hanging one: a bounded device
wait that runs out (nothing arrives at the barrier; the kernel gives up, reports and returns), and
the host-side poll / bounded wait / abort of the communicator on a single healthy rank."""
import ctypes as C

import numpy as np
import pytest

from tests.helpers import random_data, random_hclt

pytestmark = pytest.mark.gpu


def _cuda():
    import torch
    from lvd_pg_b200 import _lib, api
    assert torch.cuda.is_available()
    return torch, api, _lib


def test_bounded_wait_runs_out_reports_and_leaves_the_context_usable(oracle):
    torch, api, _lib = _cuda()
    lib = _lib.lib()
    status, after, ms, prod = C.c_int32(-1), C.c_int32(-1), C.c_float(0), C.c_uint32(0)
    polls = 1 << 16
    _lib.check(lib.pcb_selftest_wait_limit(0, polls, C.byref(status), C.byref(after), C.byref(ms), C.byref(prod)))
    assert status.value == 1            # the status word a circuit reports through pcb_circuit_status
    assert after.value == 2             # the kernel went on past the lost wait and returned by itself
    assert prod.value == 1 << 24
    lost_wait_s = ms.value * 1e-3 * prod.value / polls
    print(f"{polls} polls took {ms.value:.3f} ms -> a lost signal holds a production kernel {lost_wait_s:.2f} s")
    assert 0.0 < lost_wait_s < 60.0     # long enough for any healthy copy, short enough to end by itself
    # the context is intact: a forward pass on the same device still matches the oracle
    fc = random_hclt(9, 4, 3, 1)
    data, _ = random_data(40, fc.num_vars, 3, 5)
    m = api.CuMetaBitsProbCircuit(fc)
    ll = torch.empty(40, device=m.device)
    api.forward(m, api.DeviceData(data, m.device), ll_out=ll)
    ref = oracle.forward(fc, data)[:, -1]
    assert np.abs(ll.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    _lib.check(lib.pcb_circuit_status(m.handle))


def test_comm_poll_wait_abort_on_one_rank():
    torch, api, _lib = _cuda()
    fc = random_hclt(24, 32, 8, 3)
    data, _ = random_data(4096, fc.num_vars, 8, 7)
    m = api.CuMetaBitsProbCircuit(fc)
    dd = api.DeviceData(data, m.device)
    m.comm_poll()                                   # no communicator: nothing to report
    m.attach_comm(api.comm_unique_id(), 0, 1)
    ll = torch.zeros(1, device=m.device)
    api.em_step(m, dd, None, 1, 2048, 0.1, 0.9, 0.0, None, ll)
    m.comm_poll()
    m.comm_wait(20.0)                               # healthy: returns as soon as the stream has drained
    assert np.isfinite(float(ll.item())) and float(ll.item()) < 0
    # a wait whose limit is shorter than the work queued behind it: the communicator is aborted, the
    # kernels (all this circuit's own, there is no collective on one rank) finish normally
    for i in range(200):
        api.em_step(m, dd, None, 1 + (i % 2) * 2048, 2048, 0.1, 0.9, 0.0, None, ll)
    with pytest.raises(_lib.PcbError) as e:
        m.comm_wait(0.0)
    assert e.value.code == 3 and "aborted" in str(e.value)
    torch.cuda.synchronize()
    with pytest.raises(_lib.PcbError) as e:         # steps refuse until the dead communicator is dropped
        api.em_step(m, dd, None, 1, 2048, 0.1, 0.9, 0.0, None, ll)
    assert e.value.code == 5
    with pytest.raises(_lib.PcbError):
        m.comm_poll()
    m.detach_comm()
    m.comm_poll()
    api.em_step(m, dd, None, 1, 2048, 0.1, 0.9, 0.0, None, ll)
    torch.cuda.synchronize()
    assert np.isfinite(float(ll.item()))
    _lib.check(m.lib.pcb_circuit_status(m.handle))
