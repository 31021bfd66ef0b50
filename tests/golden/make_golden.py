"""Generates tests/golden/*.npz: known answers computed independently of both the CPU oracle and
the CUDA library, by evaluating the circuit's node graph recursively in float64 with torch and
differentiating it with autograd.

Identities used (they hold for any smooth, decomposable circuit):
  * d log p(x) / d logp_e of a sum edge  = the edge's flow for that example
    (VariationalJuice.jl/src/queries/flow.jl:53-60), so the gradient summed over a batch is
    edge_aggr; d log p(x) / d logp_leaf[x_v] = the leaf's flow (fixable_categorical_dist.jl:121-130).
  * the M-step is the closed form of reg_em.jl:292-299 applied to those statistics.
  * the KLD recursion of queries/kld.jl:71-133 evaluated on the graph; its autograd gradient
    w.r.t. the sum-edge log-params of both arguments equals edge_grads1 / edge_grads2
    (kld.jl:278-279).

Run `python tests/golden/make_golden.py` from the repository root to regenerate.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from lvd_pg_b200 import structures as st  # noqa: E402
from lvd_pg_b200.circuit import Input, Product, Sum, compile_circuit  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def graph_nodes(root):
    seen, out, stack = set(), [], [root]
    while stack:
        n = stack.pop()
        if id(n) in seen:
            continue
        seen.add(id(n))
        out.append(n)
        if not isinstance(n, Input):
            stack.extend(n.children)
    return out


def flat_index_of_params(root):
    """Map every parameter array of the graph to its positions in the flat parameter vector by
    compiling a copy whose parameters are unique marker values."""
    nodes = [n for n in graph_nodes(root) if isinstance(n, Sum) or (isinstance(n, Input) and not n.fixed)]
    saved = [n.logps.copy() for n in nodes]
    marker = 1.0
    for n in nodes:
        n.logps = (marker + np.arange(n.logps.shape[0])).astype(np.float32)
        marker += n.logps.shape[0]
    fc = compile_circuit(root)
    flat = []
    is_sum = fc.edge_is_sum
    flat.extend(fc.up_logp[is_sum].tolist())
    for nid in fc.input_node_ids:
        if not fc.node_fixed[nid - 1]:
            hs = fc.node_heap_start[nid - 1] - 1
            flat.extend(fc.heap[hs:hs + fc.node_num_cats[nid - 1]].tolist())
    pos = {float(v): i for i, v in enumerate(flat)}
    index = {}
    for n, s in zip(nodes, saved):
        # single-child sums are not materialised: their parameter has no flat slot
        index[id(n)] = np.array([pos.get(float(v), -1) for v in n.logps], np.int64)
        n.logps = s
    return index, len(flat)


def torch_params(root):
    return {id(n): torch.tensor(n.logps.astype(np.float64), requires_grad=True)
            for n in graph_nodes(root) if not isinstance(n, Product)}


def log_likelihood(root, params, row):
    memo = {}

    def ev(n):
        if id(n) in memo:
            return memo[id(n)]
        if isinstance(n, Input):
            v = params[id(n)][int(row[n.var - 1])]
        elif isinstance(n, Product):
            v = sum(ev(c) for c in n.children)
        else:
            v = torch.logsumexp(torch.stack([ev(c) + params[id(n)][j] for j, c in enumerate(n.children)]), 0)
        memo[id(n)] = v
        return v

    return ev(root)


def kld_graph(root, p1, p2):
    memo = {}

    def ev(n):
        if id(n) in memo:
            return memo[id(n)]
        if isinstance(n, Input):
            v = torch.zeros((), dtype=torch.float64) if n.fixed else (p1[id(n)].exp() * (p1[id(n)] - p2[id(n)])).sum()
        elif isinstance(n, Product):
            v = sum(ev(c) for c in n.children)
        else:
            a, b = p1[id(n)], p2[id(n)]
            v = sum(a[j].exp() * (ev(c) + a[j] - b[j]) for j, c in enumerate(n.children))
        memo[id(n)] = v
        return v

    return ev(root)


def scatter(index, params_like, P, fn):
    out = np.zeros(P, np.float64)
    for key, idx in index.items():
        vals = fn(key)
        ok = idx >= 0
        out[idx[ok]] = vals[ok]
    return out


def make_case(name, root, data, pseudocount=0.1, inertia=0.3, seed=0, **extra):
    index, P = flat_index_of_params(root)
    params = torch_params(root)
    lls, grad = [], np.zeros(P, np.float64)
    for row in data:
        for t in params.values():
            t.grad = None
        ll = log_likelihood(root, params, row)
        ll.backward()
        lls.append(ll.item())
        grad += scatter(index, params, P, lambda k: (params[k].grad.numpy() if params[k].grad is not None
                                                     else np.zeros(params[k].shape[0])))
    theta = scatter(index, params, P, lambda k: params[k].detach().numpy())
    # closed-form M-step on the statistics
    new_theta = theta.copy()
    for n in graph_nodes(root):
        if isinstance(n, Product) or (isinstance(n, Input) and n.fixed):
            continue
        idx = index[id(n)]
        if (idx < 0).any() or idx.shape[0] < 1:
            continue
        cnt = idx.shape[0]
        if isinstance(n, Sum):
            if cnt == 1:
                continue
            a = grad[idx] + pseudocount / cnt
            new = a / a.sum()
        else:
            node_flow = grad[idx].sum() + pseudocount
            new = (grad[idx] + pseudocount / cnt) / node_flow
        new_theta[idx] = np.log(inertia * np.exp(theta[idx]) + (1 - inertia) * new)
    # KLD against a perturbed, re-normalised copy
    rng = np.random.default_rng(seed)
    p1 = {k: v.detach().clone().requires_grad_(True) for k, v in params.items()}
    p2 = {}
    for k, v in params.items():
        z = v.detach().numpy() + rng.normal(0, 0.5, v.shape[0])
        p2[k] = torch.tensor(z - np.log(np.exp(z).sum()), requires_grad=True)
    kl = kld_graph(root, p1, p2)
    kl.backward()
    theta2 = scatter(index, p2, P, lambda k: p2[k].detach().numpy())
    g1 = scatter(index, p1, P, lambda k: p1[k].grad.numpy() if p1[k].grad is not None else np.zeros(p1[k].shape[0]))
    g2 = scatter(index, p2, P, lambda k: p2[k].grad.numpy() if p2[k].grad is not None else np.zeros(p2[k].shape[0]))
    fc = compile_circuit(root)
    np.savez(os.path.join(HERE, name + ".npz"), data=data.astype(np.uint8), theta=theta, ll=np.array(lls),
             stats=grad, new_theta=new_theta, pseudocount=pseudocount, inertia=inertia, theta2=theta2,
             kld=kl.item(), kld_grad1=g1, kld_grad2=g2, num_inner=fc.num_inner_params, **extra)
    print(name, "P =", P, "rows =", len(data), "LL[0] =", lls[0], "KLD =", kl.item())


def main():
    rng = np.random.default_rng(2024)
    make_case("simple3", st.simple_3vars_circuit(num_cats=5, fixed=False, rng=rng),
              rng.integers(0, 5, (6, 3)))
    parent = st.root_tree_at_center(6, st.random_spanning_tree(6, rng))
    make_case("hclt_v6_k3_c4", st.hclt_graph(parent, 4, 3, rng), rng.integers(0, 4, (9, 6)),
              parent=parent, num_cats=4, k=3)
    parent = st.root_tree_at_center(5, [(0, 1), (1, 2), (2, 3), (3, 4)])
    make_case("hclt_chain5_k2_c2", st.hclt_graph(parent, 2, 2, rng), rng.integers(0, 2, (16, 5)),
              parent=parent, num_cats=2, k=2)


if __name__ == "__main__":
    main()
