"""CUDA path vs the CPU oracle: KLD, its gradient, Adam, hard and soft sampling."""
import numpy as np
import pytest

from lvd_pg_b200 import structures as st
from lvd_pg_b200.circuit import compile_circuit
from tests.helpers import random_hclt, rel_err, simple3

pytestmark = pytest.mark.gpu
TOL = 1e-4


def _cuda():
    import torch
    from lvd_pg_b200 import api
    assert torch.cuda.is_available()
    return torch, api


def _param_sets(oracle, fc, S, seed):
    """S random normalised parameter sets in the circuit's flat order."""
    rng = np.random.default_rng(seed)
    base = oracle.vectorize(fc)
    out = np.zeros((S, base.shape[0]), np.float32)
    m = np.zeros_like(base)
    v = np.zeros_like(base)
    for s in range(S):
        theta = (base + rng.normal(0, 0.7, base.shape[0])).astype(np.float32)
        # lr = 0 Adam step == pure re-normalisation of every group and leaf
        oracle.adam_step(fc, theta, np.zeros_like(base), m, v, 1, lr=0.0)
        out[s] = theta
    return out


CASES = [("simple3", lambda: simple3(False, 5, 0), 2), ("hclt_k8", lambda: random_hclt(9, 8, 3, 1), 1),
         ("hclt_k32", lambda: random_hclt(14, 32, 2, 2), 5), ("hclt_k16_S40", lambda: random_hclt(8, 16, 4, 3), 40)]


@pytest.mark.parametrize("name,make,S", CASES, ids=[c[0] for c in CASES])
def test_kld_forward_backward(oracle, name, make, S):
    torch, api = _cuda()
    fc = make()
    p1, p2 = _param_sets(oracle, fc, S, 1), _param_sets(oracle, fc, S, 2)
    m = api.CuMetaBitsProbCircuit(fc)
    k, reuse = api.kld(m, p1, p2)
    klds_ref, ek_ref = oracle.kld(fc, p1, p2)
    assert rel_err(k.cpu().numpy(), klds_ref[:, -1]) <= TOL
    klds, ek = api.kld_matrices(m, reuse)
    assert rel_err(klds, klds_ref) <= TOL
    # edge values e^{p1} (k + p1 - p2) cancel, so they are compared on a coarser absolute floor
    assert rel_err(ek, ek_ref, 1e-2) <= TOL
    g1, g2 = api.kld_backward(m, reuse=reuse)
    ref = oracle.kld_backward(fc, p1, p2, klds_ref, ek_ref)
    assert rel_err(g1.cpu().numpy(), ref["param_grads1"], 1e-2) <= TOL
    assert rel_err(g2.cpu().numpy(), ref["param_grads2"]) <= TOL


def test_kld_closed_forms():
    """Known answers of VariationalJuice.jl/test/queries/kld_tests.jl:31-46,103-108."""
    torch, api = _cuda()
    fc = simple3(False, 5, 0)
    m = api.CuMetaBitsProbCircuit(fc)
    pars = api.vectorize_parameters(m)
    p1 = np.tile(pars, (2, 1))
    p2 = p1.copy()
    k, _ = api.kld(m, p1, p2)
    assert np.allclose(k.cpu().numpy(), 0.0, atol=1e-6)
    p1[:, :2] = np.log(np.array([[0.2, 0.8], [0.5, 0.5]], np.float32))
    p2[:, :2] = np.log(np.array([[0.4, 0.6], [0.9, 0.1]], np.float32))
    k, reuse = api.kld(m, p1, p2)
    k = k.cpu().numpy()
    assert np.isclose(k[0], 0.2 * np.log(0.2 / 0.4) + 0.8 * np.log(0.8 / 0.6), rtol=1e-5)
    assert np.isclose(k[1], 0.5 * np.log(0.5 / 0.9) + 0.5 * np.log(0.5 / 0.1), rtol=1e-5)
    g1, g2 = api.kld_backward(m, reuse=reuse)
    g1, g2 = g1.cpu().numpy(), g2.cpu().numpy()
    assert np.isclose(g1[0, 0], 0.2 * (np.log(0.2) - np.log(0.4) + 1), rtol=1e-5)
    assert np.isclose(g2[0, 0], -0.2, rtol=1e-5)
    assert np.isclose(g1[0, 1], 0.8 * (np.log(0.8) - np.log(0.6) + 1), rtol=1e-5)
    assert np.isclose(g2[0, 1], -0.8, rtol=1e-5)


def test_adam_step_matches_oracle(oracle):
    torch, api = _cuda()
    fc = random_hclt(10, 16, 3, 4)
    m = api.CuMetaBitsProbCircuit(fc)
    q, p = _param_sets(oracle, fc, 1, 5)[0], _param_sets(oracle, fc, 1, 6)[0]
    theta = torch.from_numpy(q.copy()).to(m.device)
    opt = api.Adam(m, lr=1e-2)
    th_ref, m_ref, v_ref = q.copy(), np.zeros_like(q), np.zeros_like(q)
    for t in range(1, 4):
        k, reuse = api.kld(m, theta, p)
        g1, _ = api.kld_backward(m, reuse=reuse)
        klds_ref, ek_ref = oracle.kld(fc, th_ref, p)
        gref = oracle.kld_backward(fc, th_ref, p, klds_ref, ek_ref)["param_grads1"][0]
        assert rel_err(g1.cpu().numpy()[0], gref) <= TOL
        opt.step(theta, g1, sign=-1.0)
        oracle.adam_step(fc, th_ref, gref, m_ref, v_ref, t, lr=1e-2, sign=-1.0)
        assert np.abs(theta.cpu().numpy() - th_ref).max() <= TOL


FUSED_CASES = [("hclt_k16_c3", lambda: random_hclt(12, 16, 3, 9)),          # leaves by thread, chunks of equal sums
               ("hclt_k64_binary", lambda: random_hclt(24, 64, 2, 2)),     # the shape of the variational configuration
               ("hclt_k5_c7", lambda: random_hclt(9, 5, 7, 4)),            # leaves by warp, chunks that mix nodes
               ("hclt_k160_c2", lambda: random_hclt(3, 160, 2, 5)),        # groups wider than the registers hold
               ("simple3", lambda: simple3(False, 5, 0)),
               ("fixed_leaves", lambda: compile_circuit(st.fully_factorized_categorical_fixed(3, 8)))]


@pytest.mark.parametrize("name,make", FUSED_CASES, ids=[c[0] for c in FUSED_CASES])
def test_fused_kld_adam_steps_match_oracle(oracle, name, make):
    """pcb_kld_adam_step: five steps (the second captures the chain as a CUDA graph, the later ones
    replay it) against kld + kld_backward + Adam of the oracle, then a re-seeded step count."""
    torch, api = _cuda()
    fc = make()
    m = api.CuMetaBitsProbCircuit(fc)
    q, p = _param_sets(oracle, fc, 1, 5)[0], _param_sets(oracle, fc, 1, 6)[0]
    theta = torch.from_numpy(q.copy()).to(m.device)
    opt = api.KldAdam(m, theta, torch.from_numpy(p).to(m.device), lr=1e-2)
    th_ref, m_ref, v_ref = q.copy(), np.zeros_like(q), np.zeros_like(q)
    for t in range(1, 6):
        kl = opt.step().item()
        klds_ref, ek_ref = oracle.kld(fc, th_ref, p)
        gref = oracle.kld_backward(fc, th_ref, p, klds_ref, ek_ref)["param_grads1"][0]
        oracle.adam_step(fc, th_ref, gref, m_ref, v_ref, t, lr=1e-2, sign=-1.0)
        assert abs(kl - klds_ref[0, -1]) <= TOL * max(1.0, abs(klds_ref[0, -1])), t
        assert np.abs(np.exp(theta.cpu().numpy()) - np.exp(th_ref)).max() <= TOL, t
    # a caller that restarts its count (new optimiser state) is followed
    opt.m.zero_(); opt.v.zero_(); opt.t = 0
    m_ref[:] = 0; v_ref[:] = 0
    for t in range(1, 3):
        opt.step()
        klds_ref, ek_ref = oracle.kld(fc, th_ref, p)
        gref = oracle.kld_backward(fc, th_ref, p, klds_ref, ek_ref)["param_grads1"][0]
        oracle.adam_step(fc, th_ref, gref, m_ref, v_ref, t, lr=1e-2, sign=-1.0)
        assert np.abs(np.exp(theta.cpu().numpy()) - np.exp(th_ref)).max() <= TOL, t


SAMPLE_CASES = [("simple3", lambda: simple3(False, 5, 0), 64, 1), ("hclt_k8", lambda: random_hclt(9, 8, 3, 1), 50, 1),
                ("hclt_k64_binary", lambda: random_hclt(24, 64, 2, 2), 200, 1),
                ("hclt_k16_persample", lambda: random_hclt(7, 16, 6, 3), 33, 33),
                ("fixed_leaves", lambda: compile_circuit(st.fully_factorized_categorical_fixed(3, 8)), 40, 1)]


@pytest.mark.parametrize("name,make,S,Sp", SAMPLE_CASES, ids=[c[0] for c in SAMPLE_CASES])
def test_hard_sampling_bit_exact(oracle, name, make, S, Sp):
    torch, api = _cuda()
    fc = make()
    m = api.CuMetaBitsProbCircuit(fc)
    reg_dev = m.sum_regions()
    reg_ref, R = oracle.sum_regions(fc)
    assert np.array_equal(reg_dev, reg_ref) and R == m.info.num_sum_regions
    params = _param_sets(oracle, fc, Sp, 7)
    rng = np.random.default_rng(5)
    shp = api.noise_shapes(m, S)
    u_sum, u_leaf = rng.random(shp[0], dtype=np.float32), rng.random(shp[1], dtype=np.float32)
    u_leaf[0, 0, :] = 0.5   # ties: identical noise on every category of one leaf
    x = api.sample(m, params, u_sum, u_leaf).cpu().numpy()
    x_ref = oracle.sample_hard(fc, params, u_sum, u_leaf, S)
    assert x.dtype == np.int32 and np.array_equal(x, x_ref)
    assert (x >= 0).all()


@pytest.mark.parametrize("noise", [False, True])
def test_soft_sampling_matches_oracle(oracle, noise):
    torch, api = _cuda()
    fc = random_hclt(9, 8, 3, 1)
    m = api.CuMetaBitsProbCircuit(fc)
    S = 8
    params = _param_sets(oracle, fc, S, 9)
    rng = np.random.default_rng(2)
    u = rng.random((S, m.num_inner_params), dtype=np.float32) if noise else None
    out = api.gumbel_sample(m, params, fc.num_vars, 3, temperature=0.7, no_gumbel=not noise, u=u).cpu().numpy()
    ref, aux = oracle.sample_soft(fc, params, u, 0.7, S, 3)
    assert rel_err(out, ref) <= TOL
    assert np.allclose(out.sum(2), 1.0, atol=1e-4)  # every variable's relaxed marginal sums to one


def test_fp32_preselection_never_changes_a_sample():
    """The hard sampler picks every arg-max from fp32 keys with an error bound and falls back to the fp64
    keys only among the entries that bound cannot separate; PCB_SAMPLE_EXACT_KEYS=1 turns the bound off
    (all keys in fp64).  Both must give the same samples: 32768 samples of the 784-variable circuit
    (1.7e9 keys), uniform noise; then noise quantised to eighths on uniform parameters, where most
    arg-maxes are exact ties that the lowest index has to win; then noise next to one and next to zero."""
    import os
    torch, api = _cuda()
    from lvd_pg_b200 import synth
    q, _ = synth.config4()
    fast = api.CuMetaBitsProbCircuit(q, 0)
    os.environ["PCB_SAMPLE_EXACT_KEYS"] = "1"
    try:
        exact = api.CuMetaBitsProbCircuit(q, 0)
    finally:
        del os.environ["PCB_SAMPLE_EXACT_KEYS"]
    theta = torch.from_numpy(np.asarray(api.vectorize_parameters(fast), np.float32)).to(fast.device)
    g = torch.Generator(device=fast.device).manual_seed(11)

    def same(S, u_sum, u_leaf, params):
        a = api.sample(fast, params, u_sum, u_leaf)
        b = api.sample(exact, params, u_sum, u_leaf)
        assert torch.equal(a, b)
        return a

    S = 32768
    shp_s, shp_l = api.noise_shapes(fast, S)
    u_sum = torch.rand(shp_s, generator=g, device=fast.device)
    u_leaf = torch.rand(shp_l, generator=g, device=fast.device)
    same(S, u_sum, u_leaf, theta)
    del u_sum, u_leaf
    S = 2048
    shp_s, shp_l = api.noise_shapes(fast, S)
    u_sum = torch.rand(shp_s, generator=g, device=fast.device)
    u_leaf = torch.rand(shp_l, generator=g, device=fast.device)
    flat = torch.zeros_like(theta)   # unnormalised, all equal: the keys differ by the noise alone
    x = same(S, torch.floor(u_sum * 8) / 8, torch.floor(u_leaf * 8) / 8, flat)
    assert int((x == 0).sum()) > 0
    same(S, 1.0 - u_sum * 1e-6, 1.0 - u_leaf * 1e-6, theta)      # u next to one: inner = -log x next to zero
    same(S, u_sum * 1e-6, u_leaf * 1e-6, theta)                  # u next to zero
    tiny = theta.clone()
    tiny[::3] = float("-inf")                                     # impossible edges and categories
    same(S, u_sum, u_leaf, tiny)
