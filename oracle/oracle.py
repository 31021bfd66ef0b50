"""ctypes front-end of the CPU oracle (oracle/pc_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by `__graft_entry__.smoke()` and by the
`cpu_baseline` / `--impl reference` legs of bench.py.  The product package never imports it.

All matrices are handed back as numpy arrays of shape [B, N] in Fortran order (the
reference's column-major layout), so `mars[b, n]` reads like the Julia code (0-based).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


VARIANTS = {
    "f32": "libpc_oracle.so",           # the reference's Float32 arithmetic (the parity checker)
    "f64": "libpc_oracle64.so",         # the EM path in double on the same fp32 parameters ("exact")
    "native": "libpc_oracle_native.so",  # f32 built -march=native on the machine that times it
}


def build(force: bool = False, variant: str = "f32") -> str:
    name = VARIANTS[variant]
    path = os.path.join(_HERE, name)
    src = os.path.join(_HERE, "pc_oracle.c")
    hdrs = [os.path.join(_HERE, "..", "include", h) for h in ("pcb200.h", "pcb200_gumbel.h")]
    stale = (not os.path.exists(path)) or any(
        os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(path) for p in [src] + hdrs)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", name], check=True, stdout=subprocess.DEVNULL)
    return path


def _load(variant: str):
    l = C.CDLL(build(variant=variant))
    l.orc_num_threads.restype = C.c_int
    l.orc_real_bytes.restype = C.c_int
    l.orc_gumbel_key.restype = C.c_double
    l.orc_log.restype = C.c_double
    return l


def lib():
    global _LIB
    if _LIB is None:
        _LIB = _load("f32")
    return _LIB


def use_native_build() -> None:
    """Switch this process to the -march=native build (compiled on this machine on first use):
    what the benchmark's CPU arm times.  Results are the same arithmetic (no fast-math)."""
    global _LIB
    build(force=True, variant="native")   # never trust a copy built on another machine
    _LIB = _load("native")


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f(shape):
    return np.zeros(shape, dtype=np.float32, order="F")


def gumbel_key(logp: float, u: float) -> float:
    return float(lib().orc_gumbel_key(C.c_float(logp), C.c_float(u)))


def det_log(x: float) -> float:
    return float(lib().orc_log(C.c_double(x)))


def num_threads() -> int:
    return int(lib().orc_num_threads())


def set_num_threads(n: int) -> None:
    lib().orc_set_num_threads(C.c_int(n))


def set_row_block(n: int) -> None:
    """Rows per block of the forward / backward loops (1..16, default 16)."""
    lib().orc_set_row_block(C.c_int(n))


def counts(fc):
    d = fc.desc()
    a, b, g = C.c_uint32(), C.c_uint32(), C.c_uint32()
    lib().orc_counts(C.byref(d), C.byref(a), C.byref(b), C.byref(g))
    return a.value, b.value, g.value


def meta(fc):
    d = fc.desc()
    ni, nl, ng = counts(fc)
    e2p = np.zeros(fc.num_edges, np.uint32)
    p2e = np.zeros(ni, np.uint32)
    p2g = np.zeros(ni, np.uint32)
    cum = np.zeros(len(fc.input_node_ids), np.uint32)
    lib().orc_meta(C.byref(d), _p(e2p), _p(p2e), _p(p2g), _p(cum))
    return {"edge2param": e2p, "param2edge": p2e, "param2group": p2g, "innode2ncumparam": cum,
            "num_inner_params": ni, "num_input_params": nl, "num_param_groups": ng}


def vectorize(fc) -> np.ndarray:
    d = fc.desc()
    ni, nl, _ = counts(fc)
    out = np.zeros(ni + nl, np.float32)
    lib().orc_vectorize(C.byref(d), _p(fc.up_logp), _p(fc.heap), _p(out))
    return out


def update_parameters(fc, params) -> None:
    d = fc.desc()
    params = np.ascontiguousarray(params, np.float32)
    lib().orc_update_parameters(C.byref(d), _p(fc.up_logp), _p(fc.heap), _p(params))


def _data_args(data, miss, row_ids, row_start, B):
    data = np.asfortranarray(data, dtype=np.uint8)
    miss = None if miss is None else np.asfortranarray(miss, dtype=np.uint8)
    rid = None if row_ids is None else np.ascontiguousarray(row_ids, np.int32)
    if B is None:
        B = len(rid) if rid is not None else data.shape[0] - (row_start - 1)
    return data, miss, rid, int(B)


def forward(fc, data, row_ids=None, row_start=1, B=None, miss=None, want_edge_mars=False):
    d = fc.desc()
    data, miss, rid, B = _data_args(data, miss, row_ids, row_start, B)
    mars = _f((B, fc.num_nodes))
    em = _f((B, fc.num_edges)) if want_edge_mars else None
    lib().orc_forward(C.byref(d), _p(fc.up_logp), _p(fc.heap), _p(data), _p(miss),
                      C.c_uint64(data.shape[0]), _p(rid), C.c_uint32(row_start), C.c_uint32(B),
                      _p(mars), _p(em))
    return (mars, em) if want_edge_mars else mars


def backward(fc, mars, edge_aggr=None, want_edge_flows=False):
    d = fc.desc()
    B = mars.shape[0]
    flows = _f((B, fc.num_nodes))
    ef = _f((B, fc.num_edges)) if want_edge_flows else None
    if edge_aggr is None:
        edge_aggr = np.zeros(fc.num_edges, np.float32)
    lib().orc_backward(C.byref(d), _p(fc.up_logp), _p(np.asfortranarray(mars)), C.c_uint32(B),
                       _p(flows), _p(ef), _p(edge_aggr))
    return (flows, ef, edge_aggr) if want_edge_flows else (flows, edge_aggr)


def input_flows(fc, flows, data, row_ids=None, row_start=1, miss=None, weights=None):
    d = fc.desc()
    data, miss, rid, B = _data_args(data, miss, row_ids, row_start, flows.shape[0])
    w = None if weights is None else np.ascontiguousarray(weights, np.float32)
    lib().orc_input_flows(C.byref(d), _p(fc.heap), _p(np.asfortranarray(flows)), _p(data), _p(miss),
                          C.c_uint64(data.shape[0]), _p(rid), C.c_uint32(row_start), C.c_uint32(B), _p(w))


def _soft(soft):
    """[rows, V, C] per-category log-weights in the reference's column-major layout."""
    return None if soft is None else np.asfortranarray(soft, dtype=np.float32)


def forward_ex(fc, data=None, soft=None, row_ids=None, row_start=1, B=None, miss=None, soft_reg=0.0, soft_reg_width=1):
    """eval_circuit with soft evidence (init_mar!_with_reg_cat_kernel, reg_likelihood.jl:51-91) or with
    soft-regularised leaves (soft_loglikelihood, reg_likelihood.jl:4-14)."""
    d = fc.desc()
    soft = _soft(soft)
    if data is None:
        rows = soft.shape[0]
        rid = None if row_ids is None else np.ascontiguousarray(row_ids, np.int32)
        B = int(B if B is not None else (len(rid) if rid is not None else rows - (row_start - 1)))
    else:
        data, miss, rid, B = _data_args(data, miss, row_ids, row_start, B)
        rows = data.shape[0]
    mars = _f((B, fc.num_nodes))
    lib().orc_forward_ex(C.byref(d), _p(fc.up_logp), _p(fc.heap), _p(data), _p(miss), _p(soft), C.c_uint64(rows),
                         _p(rid), C.c_uint32(row_start), C.c_uint32(B), C.c_float(soft_reg), C.c_int32(soft_reg_width),
                         _p(mars), None)
    return mars


def backward_ex(fc, mars, head_roots, head_mask, row_ids=None, row_start=1, edge_aggr=None):
    """multi_head_flows_circuit (src-jl/multi_head_pc/flow.jl:178-195): head_roots 1-based node ids,
    head_mask [rows, H]."""
    d = fc.desc()
    B = mars.shape[0]
    flows = _f((B, fc.num_nodes))
    if edge_aggr is None:
        edge_aggr = np.zeros(fc.num_edges, np.float32)
    roots = np.ascontiguousarray(head_roots, np.uint32)
    mask = np.asfortranarray(head_mask, dtype=np.float32)
    rid = None if row_ids is None else np.ascontiguousarray(row_ids, np.int32)
    lib().orc_backward_ex(C.byref(d), _p(fc.up_logp), _p(np.asfortranarray(mars)), C.c_uint32(B), _p(flows), None,
                          _p(edge_aggr), _p(roots), C.c_uint32(len(roots)), _p(mask), C.c_uint64(mask.shape[0]),
                          _p(rid), C.c_uint32(row_start))
    return flows, edge_aggr


def multihead_lls(fc, mars, head_roots, head_mask=None, row_ids=None, row_start=1):
    """extract_lls_from_root_nodes (src-jl/multi_head_pc/bit_circuit.jl:95-109)."""
    d = fc.desc()
    B = mars.shape[0]
    roots = np.ascontiguousarray(head_roots, np.uint32)
    mask = None if head_mask is None else np.asfortranarray(head_mask, dtype=np.float32)
    rid = None if row_ids is None else np.ascontiguousarray(row_ids, np.int32)
    lls = _f((B,)) if mask is not None else _f((B, len(roots)))
    lib().orc_multihead_lls(C.byref(d), _p(np.asfortranarray(mars)), C.c_uint32(B), _p(roots), C.c_uint32(len(roots)),
                            _p(mask), C.c_uint64(0 if mask is None else mask.shape[0]), _p(rid), C.c_uint32(row_start),
                            _p(lls))
    return lls


def input_flows_ex(fc, flows, data=None, soft=None, row_ids=None, row_start=1, miss=None, weights=None, soft_reg=0.0,
                   soft_reg_width=1):
    """input_flows_circuit_with_reg(_cat) (reg_flow.jl:24-82) into fc.heap."""
    d = fc.desc()
    soft = _soft(soft)
    B = flows.shape[0]
    if data is None:
        rows = soft.shape[0]
        rid = None if row_ids is None else np.ascontiguousarray(row_ids, np.int32)
    else:
        data, miss, rid, B = _data_args(data, miss, row_ids, row_start, B)
        rows = data.shape[0]
    w = None if weights is None else np.ascontiguousarray(weights, np.float32)
    lib().orc_input_flows_ex(C.byref(d), _p(fc.heap), _p(np.asfortranarray(flows)), _p(data), _p(miss), _p(soft),
                             C.c_uint64(rows), _p(rid), C.c_uint32(row_start), C.c_uint32(B), _p(w),
                             C.c_float(soft_reg), C.c_int32(soft_reg_width))


def em_step_ex(fc, data=None, soft=None, head_roots=None, head_mask=None, row_ids=None, row_start=1, B=None,
               pseudocount=0.1, inertia=0.0, miss=None, weights=None, edge_aggr=None, clear_rate=0.0, soft_reg=0.0,
               soft_reg_width=1):
    """Per-batch body of mini_batch_em_with_reg (reg_em.jl:273-301) on soft evidence / soft-regularised
    leaves, or of mini_batch_em_for_multihead_pc (src-jl/multi_head_pc/em.jl:58-83) when head_roots is
    given.  Mutates fc.up_logp and fc.heap; returns (sum of batch LLs, edge_aggr before the update)."""
    if edge_aggr is None:
        edge_aggr = np.zeros(fc.num_edges, np.float32)
    clear_flows(fc, edge_aggr, clear_rate)
    mars = forward_ex(fc, data, soft, row_ids, row_start, B, miss, soft_reg, soft_reg_width)
    if head_roots is not None:
        flows, edge_aggr = backward_ex(fc, mars, head_roots, head_mask, row_ids, row_start, edge_aggr)
        ll = float(multihead_lls(fc, mars, head_roots, head_mask, row_ids, row_start).astype(np.float64).sum())
    else:
        flows, edge_aggr = backward(fc, mars, edge_aggr)
        ll = float(mars[:, -1].astype(np.float64).sum())
    input_flows_ex(fc, flows, data, soft, row_ids, row_start, miss, weights, soft_reg, soft_reg_width)
    aggr_before = edge_aggr.copy()
    em_update(fc, edge_aggr, pseudocount, inertia)
    return ll, aggr_before


def per_sample_normalized_flows(fc, data, params=None):
    """per_sample_normalized_flows (queries/flow.jl:417-494) for small cases: every row is evaluated with
    its own parameter vector (params [rows, P]) by the forward / backward passes above, the edge flows
    are normalised per sum node as map_flows_kernel does (flow.jl:496-528: log(flow / (1e-8 + sum) + 1e-8))
    and the leaf parameters as map_input_flows_kernel does (flow.jl:549-593: log(flow / sum), the whole
    flow of a leaf going to the observed category, fixable_categorical_dist.jl:162-176)."""
    data = np.asfortranarray(data, dtype=np.uint8)
    rows = data.shape[0]
    ni, nl, _ = counts(fc)
    e2p = meta(fc)["edge2param"].astype(np.int64)            # 1-based parameter id per up edge, 0 for product edges
    out = np.zeros((rows, ni + nl), np.float32)
    sum_edges = np.nonzero(e2p > 0)[0]
    for r in range(rows):
        g = fc if params is None else fc.copy()
        if params is not None:
            update_parameters(g, np.ascontiguousarray(params[r], np.float32))
        mars = forward(g, data, row_start=r + 1, B=1)
        flows, ef, _ = backward(g, mars, want_edge_flows=True)
        ef = ef[0].astype(np.float32)
        group = np.full(fc.num_nodes + 1, np.float32(1e-8), np.float32)
        np.add.at(group, fc.up_parent[sum_edges].astype(np.int64), ef[sum_edges])
        with np.errstate(divide="ignore", invalid="ignore"):
            out[r, e2p[sum_edges] - 1] = np.log(ef[sum_edges] / group[fc.up_parent[sum_edges].astype(np.int64)]
                                                + np.float32(1e-8))
            pos = ni
            for nid in fc.input_node_ids.astype(np.int64):
                if fc.node_fixed[nid - 1]:
                    continue
                C_ = int(fc.node_num_cats[nid - 1])
                f = np.float32(flows[0, nid - 1])
                e = np.zeros(C_, np.float32)
                e[int(data[r, int(fc.node_var[nid - 1]) - 1])] = f
                out[r, pos:pos + C_] = np.log(e / e.sum(dtype=np.float32))
                pos += C_
    return out


def normalize_params(fc, params, undo=False):
    """normalize_params (misc.jl:363-392, 405-480) on [S, P] parameter sets; returns a new array."""
    out = np.array(params, np.float32, copy=True)
    ni, nl, _ = counts(fc)
    pos = ni
    for nid in fc.input_node_ids.astype(np.int64):
        if fc.node_fixed[nid - 1]:
            continue
        C_ = int(fc.node_num_cats[nid - 1])
        blk = out[:, pos:pos + C_]
        if undo:
            with np.errstate(invalid="ignore"):
                blk[...] = np.where(blk > 0, np.log(blk + np.float32(1e-6), where=blk > 0, out=np.zeros_like(blk)), blk)
        else:
            e = np.exp(blk)
            blk[...] = e / e.sum(1, keepdims=True, dtype=np.float32)
        pos += C_
    m = meta(fc)
    p2g = m["param2group"].astype(np.int64)
    tot = np.zeros((out.shape[0], p2g.max() + 1 if ni else 1), np.float32)
    np.add.at(tot.T, p2g, np.exp(out[:, :ni]).T)
    out[:, :ni] -= np.log(tot[:, p2g])
    return out


def conditioned_td_prob(fc, marked_var, marked_cat, node_probs):
    """conditioned_td_prob (queries/td_prob.jl:161-291) edge by edge in down order, then
    gumbel_input_sample_down with the circuit's own leaf parameters (queries/sample.jl:233-296);
    small cases only.  marked_* are [N] (0 = unmarked, else 1-based), node_probs [S, Z1, Z2]."""
    S = node_probs.shape[0]
    N = fc.num_nodes
    td = np.zeros((S, N), np.float32)
    for de in range(fc.num_edges):
        e = int(fc.down2up[de]) - 1
        parent, prime, sub = int(fc.up_parent[e]) - 1, int(fc.up_prime[e]) - 1, int(fc.up_sub[e])
        if marked_var[parent] > 0:
            td[:, parent] = node_probs[:, marked_var[parent] - 1, marked_cat[parent] - 1]
        etd = td[:, parent].copy()
        if fc.edge_is_sum[e]:
            etd = etd * np.exp(np.float32(fc.up_logp[e]))
        if sub != 0:
            td[:, sub - 1] += etd
        td[:, prime] += etd
    cmax = int(fc.node_num_cats.max())
    out = np.zeros((S, fc.num_vars, cmax), np.float32)
    for nid in fc.input_node_ids.astype(np.int64):
        C_ = int(fc.node_num_cats[nid - 1])
        hs = int(fc.node_heap_start[nid - 1]) - 1
        out[:, int(fc.node_var[nid - 1]) - 1, :C_] += td[:, [nid - 1]] * np.exp(fc.heap[hs:hs + C_])[None, :]
    return out, td


def clear_flows(fc, edge_aggr, rate=0.0):
    d = fc.desc()
    lib().orc_clear_flows(C.byref(d), _p(edge_aggr), _p(fc.heap), C.c_float(rate))


def em_update(fc, edge_aggr, pseudocount, inertia):
    d = fc.desc()
    lib().orc_em_update(C.byref(d), _p(fc.up_logp), _p(edge_aggr), _p(fc.heap),
                        C.c_float(pseudocount), C.c_float(inertia))


def em_step(fc, data, row_ids=None, row_start=1, B=None, pseudocount=0.1, inertia=0.0, miss=None,
            weights=None, edge_aggr=None, clear_rate=0.0):
    """Per-batch body of mini_batch_em_with_reg (regularization/reg_em.jl:273-301).
    Mutates fc.up_logp and fc.heap; returns (sum of batch LLs, edge_aggr before the update)."""
    if edge_aggr is None:
        edge_aggr = np.zeros(fc.num_edges, np.float32)
    clear_flows(fc, edge_aggr, clear_rate)
    mars = forward(fc, data, row_ids, row_start, B, miss)
    flows, edge_aggr = backward(fc, mars, edge_aggr)
    input_flows(fc, flows, data, row_ids, row_start, miss, weights)
    ll = float(mars[:, -1].astype(np.float64).sum())
    aggr_before = edge_aggr.copy()
    em_update(fc, edge_aggr, pseudocount, inertia)
    return ll, aggr_before


def kld(fc, params1, params2):
    d = fc.desc()
    p1 = np.asfortranarray(np.atleast_2d(params1), np.float32)
    p2 = np.asfortranarray(np.atleast_2d(params2), np.float32)
    S = p1.shape[0]
    klds = _f((S, fc.num_nodes))
    ek = _f((S, fc.num_edges))
    lib().orc_kld(C.byref(d), _p(p1), _p(p2), C.c_uint32(S), _p(klds), _p(ek))
    return klds, ek


def kld_backward(fc, params1, params2, klds, edge_klds):
    d = fc.desc()
    p1 = np.asfortranarray(np.atleast_2d(params1), np.float32)
    p2 = np.asfortranarray(np.atleast_2d(params2), np.float32)
    S, P = p1.shape
    grads = _f((S, fc.num_nodes))
    eg1, eg2 = _f((S, fc.num_edges)), _f((S, fc.num_edges))
    g1, g2 = _f((S, P)), _f((S, P))
    lib().orc_kld_backward(C.byref(d), _p(p1), _p(p2), C.c_uint32(S), _p(np.asfortranarray(klds)),
                           _p(np.asfortranarray(edge_klds)), _p(grads), _p(eg1), _p(eg2), _p(g1), _p(g2))
    return {"grads": grads, "edge_grads1": eg1, "edge_grads2": eg2, "param_grads1": g1, "param_grads2": g2}


def adam_step(fc, theta, grad, m, v, t, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, sign=-1.0):
    d = fc.desc()
    for a in (theta, m, v):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    grad = np.ascontiguousarray(grad, np.float32)
    lib().orc_adam_step(C.byref(d), _p(theta), _p(grad), _p(m), _p(v), C.c_int32(t), C.c_float(lr),
                        C.c_float(beta1), C.c_float(beta2), C.c_float(eps), C.c_float(sign))


def sum_regions(fc):
    d = fc.desc()
    reg = np.zeros(fc.num_nodes, np.uint32)
    R = C.c_uint32()
    lib().orc_sum_regions(C.byref(d), _p(reg), C.byref(R))
    return reg, R.value


def sample_hard(fc, params, u_sum, u_leaf, S):
    """params [Sp, P]; u_sum [S, R, kmax], u_leaf [S, V, cmax] C-order. Returns x [S, V] int32."""
    d = fc.desc()
    p = np.asfortranarray(np.atleast_2d(params), np.float32)
    u_sum = np.ascontiguousarray(u_sum, np.float32)
    u_leaf = np.ascontiguousarray(u_leaf, np.float32)
    x = np.zeros((S, fc.num_vars), np.int32, order="F")
    lib().orc_sample_hard(C.byref(d), _p(fc.heap), _p(p), C.c_uint32(p.shape[0]), _p(u_sum), _p(u_leaf),
                          C.c_uint32(S), C.c_uint32(u_sum.shape[2]), C.c_uint32(u_leaf.shape[2]), _p(x))
    return x


def sample_soft(fc, params, u, temperature, S, cmax):
    d = fc.desc()
    p = np.asfortranarray(np.atleast_2d(params), np.float32)
    ni, _, ng = counts(fc)
    uu = None if u is None else np.asfortranarray(u, np.float32)
    ep, cp, td = _f((S, ni)), _f((S, ng)), _f((S, fc.num_nodes))
    out = _f((S, fc.num_vars, cmax))
    lib().orc_sample_soft(C.byref(d), _p(fc.heap), _p(p), C.c_uint32(p.shape[0]), _p(uu),
                          C.c_float(temperature), C.c_uint32(S), C.c_uint32(cmax), _p(ep), _p(cp), _p(td), _p(out))
    return out, {"edge_probs": ep, "cum_probs": cp, "td_probs": td}


class Exact:
    """The EM path of the oracle evaluated in float64 (libpc_oracle64.so) on the same fp32
    parameters: mars, flows, statistics and the updated parameters as the exact arithmetic gives
    them.  Two fp32 implementations that sum in different orders (the reference's own atomics do)
    differ from each other by rounding that grows with the magnitude of the log-values; both are
    compared with this.  Holds its own float64 copies of the parameters (`up_logp`, `heap`)."""

    def __init__(self, fc):
        self.fc = fc
        self.lib = _load("f64")
        assert self.lib.orc_real_bytes() == 8
        self.up_logp = fc.up_logp.astype(np.float64)
        self.heap = fc.heap.astype(np.float64)

    def forward(self, data, row_ids=None, row_start=1, B=None, miss=None):
        d = self.fc.desc()
        data, miss, rid, B = _data_args(data, miss, row_ids, row_start, B)
        mars = np.zeros((B, self.fc.num_nodes), np.float64, order="F")
        self.lib.orc_forward(C.byref(d), _p(self.up_logp), _p(self.heap), _p(data), _p(miss),
                             C.c_uint64(data.shape[0]), _p(rid), C.c_uint32(row_start), C.c_uint32(B), _p(mars), None)
        return mars

    def backward(self, mars, edge_aggr=None):
        d = self.fc.desc()
        B = mars.shape[0]
        flows = np.zeros((B, self.fc.num_nodes), np.float64, order="F")
        if edge_aggr is None:
            edge_aggr = np.zeros(self.fc.num_edges, np.float64)
        self.lib.orc_backward(C.byref(d), _p(self.up_logp), _p(np.asfortranarray(mars)), C.c_uint32(B),
                              _p(flows), None, _p(edge_aggr))
        return flows, edge_aggr

    def input_flows(self, flows, data, row_ids=None, row_start=1, miss=None, weights=None):
        d = self.fc.desc()
        data, miss, rid, B = _data_args(data, miss, row_ids, row_start, flows.shape[0])
        w = None if weights is None else np.ascontiguousarray(weights, np.float64)
        self.lib.orc_input_flows(C.byref(d), _p(self.heap), _p(np.asfortranarray(flows)), _p(data), _p(miss),
                                 C.c_uint64(data.shape[0]), _p(rid), C.c_uint32(row_start), C.c_uint32(B), _p(w))

    def clear_flows(self, edge_aggr, rate=0.0):
        d = self.fc.desc()
        self.lib.orc_clear_flows(C.byref(d), _p(edge_aggr), _p(self.heap), C.c_double(rate))

    def em_update(self, edge_aggr, pseudocount, inertia):
        d = self.fc.desc()
        self.lib.orc_em_update(C.byref(d), _p(self.up_logp), _p(edge_aggr), _p(self.heap),
                               C.c_double(pseudocount), C.c_double(inertia))

    def em_step(self, data, row_ids=None, row_start=1, B=None, pseudocount=0.1, inertia=0.0, miss=None,
                weights=None, edge_aggr=None, clear_rate=0.0):
        if edge_aggr is None:
            edge_aggr = np.zeros(self.fc.num_edges, np.float64)
        self.clear_flows(edge_aggr, clear_rate)
        mars = self.forward(data, row_ids, row_start, B, miss)
        flows, edge_aggr = self.backward(mars, edge_aggr)
        self.input_flows(flows, data, row_ids, row_start, miss, weights)
        ll = float(mars[:, -1].sum())
        aggr_before = edge_aggr.copy()
        self.em_update(edge_aggr, pseudocount, inertia)
        return ll, aggr_before

    def vectorize(self) -> np.ndarray:
        """Flat parameters (misc.jl:42-68 order) as float64."""
        fc = self.fc
        inner = self.up_logp[fc.edge_is_sum]
        leaves = []
        for nid in fc.input_node_ids.astype(np.int64):
            if not fc.node_fixed[nid - 1]:
                hs = int(fc.node_heap_start[nid - 1]) - 1
                leaves.append(self.heap[hs:hs + int(fc.node_num_cats[nid - 1])])
        return np.concatenate([inner] + leaves) if leaves else inner.copy()
