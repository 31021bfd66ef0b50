"""Circuit structures: the reference's hand-built test circuits, Chow-Liu trees and HCLTs.

HCLT construction follows `hclt_from_clt`
(VariationalJuice.jl/src/structures/hclts.jl:100-145): every CLT variable y gets k leaves
L_y[j]; an inner CLT node with children x_1..x_m gets, for every latent state c of its parent,
the sum  S_y[c] = sum_j theta_y[c, j] * (prod_i child_i[j]) * L_y[j];  only S_root[0] is used.
hclts.jl:133 re-creates the k products inside the comprehension for each of the k sums; they
are value-identical, so the compiled form built here shares them (a sum edge carries the
pair (prime, sub) directly when its product has two children, as the reference's SumEdge
does, queries/likelihood.jl:30-36).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from .circuit import (PCB_INPUT, PCB_PRODUCT, PCB_SUM, TAG_FIRST, TAG_LAST, TAG_ONLYSUB,
                      FlatCircuit, Input, Product, Sum, compile_circuit, multiply, summate)


# ---------------------------------------------------------------------------------------------
# hand-built circuits of VariationalJuice.jl/test/helpers/simple_circuits.jl
# ---------------------------------------------------------------------------------------------
def _loguniform(n):
    return np.full(n, -np.log(n), np.float32)


def _perturbed(rng, n, perturbation):
    """init_params(d, perturbation), nodes/fixable_categorical_dist.jl:33-43."""
    if rng is None:
        return _loguniform(n)
    u = 1.0 - perturbation + rng.random(n) * 2.0 * perturbation
    return np.log(u / u.sum()).astype(np.float32)


def simple_3vars_circuit(num_cats: int = 5, fixed: bool = True, rng=None, perturbation: float = 0.4):
    """simple_circuits.jl:4-14: a 2-component mixture of fully factorised 3-variable leaves."""
    def leaf(v):
        lp = _loguniform(num_cats) if fixed else _perturbed(rng, num_cats, perturbation)
        return Input(v, lp, fixed)
    n11, n21, n31 = leaf(1), leaf(2), leaf(3)
    n12, n22, n32 = leaf(1), leaf(2), leaf(3)
    pc = Sum([multiply(n11, n21, n31), multiply(n12, n22, n32)], _perturbed(rng, 2, perturbation))
    return pc


def simple_multihead_circuit(num_cats: int = 5, heads: int = 2, rng=None, perturbation: float = 0.4):
    """simple_circuits.jl:54-66: `heads` mixtures over the same two fully factorised products."""
    def leaf(v):
        return Input(v, _perturbed(rng, num_cats, perturbation), False)
    n1 = multiply(leaf(1), leaf(2), leaf(3))
    n2 = multiply(leaf(1), leaf(2), leaf(3))
    return [Sum([n1, n2], _perturbed(rng, 2, perturbation)) for _ in range(heads)]


def fully_factorized_categorical_fixed(num_vars: int = 3, num_cats: int = 8, eps: float = 1e-6):
    """simple_circuits.jl:40-52: per variable a sum over near-one-hot fixed leaves."""
    sums = []
    for i in range(1, num_vars + 1):
        ins = []
        for j in range(num_cats):
            p = np.full(num_cats, eps / num_cats)
            p[j] += 1 - eps
            ins.append(Input(i, np.log(p).astype(np.float32), True))
        sums.append(summate(*ins))
    return summate(multiply(*sums))


# ---------------------------------------------------------------------------------------------
# Chow-Liu trees
# ---------------------------------------------------------------------------------------------
def pairwise_mi(data: np.ndarray, num_cats: int, pseudocount: float = 0.1, device: str = "cpu",
                chunk: int = 256) -> np.ndarray:
    """Pairwise mutual information of categorical columns
    (VariationalJuice.jl/src/utils/information.jl:3-157: joint counts + pseudocount spread over
    the table, MI = sum p_xy log(p_xy / (p_x p_y))).  One-hot matmuls in torch, chunked."""
    import torch

    n, v = data.shape
    dev = torch.device(device)
    x = torch.as_tensor(np.ascontiguousarray(data), device=dev).long()
    onehot = torch.zeros(n, v * num_cats, dtype=torch.float32, device=dev)
    onehot.scatter_(1, x + torch.arange(v, device=dev)[None, :] * num_cats, 1.0)
    total = n + pseudocount
    single = (onehot.sum(0).view(v, num_cats) + pseudocount / num_cats) / total
    mi = torch.zeros(v, v, dtype=torch.float64, device=dev)
    for i0 in range(0, v, chunk):
        i1 = min(v, i0 + chunk)
        joint = onehot[:, i0 * num_cats:i1 * num_cats].T @ onehot  # [(i,c1), (j,c2)]
        joint = joint.view(i1 - i0, num_cats, v, num_cats).permute(0, 2, 1, 3)
        pxy = (joint + pseudocount / (num_cats * num_cats)) / total
        px = single[i0:i1, None, :, None]
        py = single[None, :, None, :]
        mi[i0:i1] = (pxy * (pxy.log() - px.log() - py.log())).sum((2, 3)).double()
    return mi.cpu().numpy()


def max_spanning_tree(weights: np.ndarray) -> List[Tuple[int, int]]:
    """Prim's algorithm on a dense symmetric weight matrix; returns V-1 undirected edges."""
    v = weights.shape[0]
    in_tree = np.zeros(v, bool)
    in_tree[0] = True
    best = weights[0].astype(np.float64).copy()
    best_from = np.zeros(v, np.int64)
    best[0] = -np.inf
    edges = []
    for _ in range(v - 1):
        j = int(np.argmax(best))
        edges.append((int(best_from[j]), j))
        in_tree[j] = True
        best[j] = -np.inf
        upd = (~in_tree) & (weights[j] > best)
        best[upd] = weights[j][upd]
        best_from[upd] = j
    return edges


def random_spanning_tree(v: int, rng) -> List[Tuple[int, int]]:
    """A seeded random spanning tree: node i (in a random order) attaches to a random earlier node."""
    perm = rng.permutation(v)
    edges = []
    for i in range(1, v):
        edges.append((int(perm[rng.integers(0, i)]), int(perm[i])))
    return edges


def root_tree_at_center(v: int, edges: Sequence[Tuple[int, int]]) -> np.ndarray:
    """Direct an undirected tree away from its centre, found by BFS
    (structures/customizable_hclt.jl:106-126: bfs_tree(MStree, center(MStree)[1])).
    Returns parent[v] with -1 at the root."""
    adj = [[] for _ in range(v)]
    for a, b in edges:
        adj[a].append(b)
        adj[b].append(a)

    def bfs(src):
        dist = np.full(v, -1, np.int64)
        par = np.full(v, -1, np.int64)
        dist[src] = 0
        q = [src]
        for u in q:
            for w in sorted(adj[u]):
                if dist[w] < 0:
                    dist[w] = dist[u] + 1
                    par[w] = u
                    q.append(w)
        return dist, par

    d0, _ = bfs(0)
    a = int(np.argmax(d0))
    da, pa = bfs(a)
    b = int(np.argmax(da))
    path = [b]
    while path[-1] != a:
        path.append(int(pa[path[-1]]))
    # the centre vertices are the middle of a longest path; take the smallest id like center()[1]
    mid = [path[(len(path) - 1) // 2], path[len(path) // 2]]
    centre = min(mid)
    _, parent = bfs(centre)
    return parent


def learn_clt(data: np.ndarray, num_cats: int, pseudocount: float = 0.1, device: str = "cpu") -> np.ndarray:
    mi = pairwise_mi(data, num_cats, pseudocount, device)
    np.fill_diagonal(mi, -np.inf)
    return root_tree_at_center(data.shape[1], max_spanning_tree(mi))


# ---------------------------------------------------------------------------------------------
# HCLT
# ---------------------------------------------------------------------------------------------
def _children_lists(parent: np.ndarray) -> List[List[int]]:
    ch: List[List[int]] = [[] for _ in range(len(parent))]
    for v, p in enumerate(parent):
        if p >= 0:
            ch[int(p)].append(v)
    return ch


def _post_order(parent: np.ndarray) -> List[int]:
    ch = _children_lists(parent)
    root = int(np.nonzero(parent < 0)[0][0])
    out, stack = [], [(root, 0)]
    while stack:
        v, i = stack.pop()
        if i < len(ch[v]):
            stack.append((v, i + 1))
            stack.append((ch[v][i], 0))
        else:
            out.append(v)
    return out


def _dirichlet_log(rng, rows: int, cols: int) -> np.ndarray:
    """log of `rows` independent Dirichlet(1,...,1) draws of dimension `cols`, fp32."""
    e = rng.standard_exponential((rows, cols), dtype=np.float32)
    np.maximum(e, np.float32(1e-30), out=e)
    tot = e.sum(1, keepdims=True, dtype=np.float64)
    np.log(e, out=e)
    e -= np.log(tot).astype(np.float32)
    return e


def hclt_graph(parent: np.ndarray, num_cats: int, k: int, rng=None):
    """Object-graph HCLT, literally hclts.jl:100-145 (with the duplicated products).  Small
    circuits only; used to cross-check `hclt_flat`."""
    v = len(parent)
    ch = _children_lists(parent)
    leaves = [[Input(y + 1, _dirichlet_log(rng, 1, num_cats)[0] if rng is not None
                     else _loguniform(num_cats)) for _ in range(k)] for y in range(v)]
    circuits: List[Optional[list]] = [None] * v
    for y in _post_order(parent):
        if not ch[y]:
            circuits[y] = leaves[y]
            continue
        cc = [circuits[x] for x in ch[y]]
        if len(cc) > 1:
            child = [summate(multiply(*[c[j] for c in cc])) for j in range(k)]
        else:
            child = cc[0]
        sums = []
        for _ in range(k):
            w = _dirichlet_log(rng, 1, k)[0] if rng is not None else _loguniform(k)
            sums.append(Sum([multiply(child[j], leaves[y][j]) for j in range(k)], w))
        circuits[y] = sums
    return circuits[_post_order(parent)[-1]][0]


def hclt_flat(parent: np.ndarray, num_cats: int, k: int, seed: Optional[int] = 0) -> FlatCircuit:
    """Compiled HCLT built directly as arrays (no per-node Python objects), block-contiguous:
    the k leaves, the k products and the k sums of a CLT variable occupy consecutive node ids,
    and the k*k edges of a sum block are consecutive with the child index fastest.
    Parameters: every sum group and every leaf ~ Dirichlet(1) from `seed` (uniform if None)."""
    parent = np.asarray(parent, np.int64)
    v = len(parent)
    ch = _children_lists(parent)
    order = _post_order(parent)
    root = order[-1]
    rng = np.random.default_rng(seed) if seed is not None else None
    assert ch[root], "an HCLT needs at least two variables"

    # ---- node ids (1-based), layers --------------------------------------------------------
    leaf_base = np.zeros(v, np.int64)
    prod_base = np.zeros(v, np.int64)
    sum_base = np.zeros(v, np.int64)
    out_base = np.zeros(v, np.int64)   # block a parent multiplies in: S_y if inner else L_y
    out_layer = np.zeros(v, np.int64)
    prod_layer = np.zeros(v, np.int64)
    sum_layer = np.zeros(v, np.int64)
    nid = 1
    for y in order:
        leaf_base[y] = nid
        nid += k
        if not ch[y]:
            out_base[y], out_layer[y] = leaf_base[y], 0
            continue
        lay = max(out_layer[x] for x in ch[y])
        if len(ch[y]) > 1:
            prod_base[y] = nid
            nid += k
            prod_layer[y] = lay + 1
            lay = lay + 1
        sum_base[y] = nid
        nid += 1 if y == root else k
        sum_layer[y] = lay + 1
        out_base[y], out_layer[y] = sum_base[y], sum_layer[y]
    n_nodes = nid - 1

    kind = np.zeros(n_nodes, np.uint8)
    var = np.zeros(n_nodes, np.uint32)
    ncat = np.zeros(n_nodes, np.uint32)
    hstart = np.zeros(n_nodes, np.uint32)
    fixed = np.zeros(n_nodes, np.uint8)
    hl = 2 * num_cats + 1
    heap = np.zeros(v * k * hl, np.float32)
    input_ids = np.zeros(v * k, np.uint32)
    hpos = 0
    for i, y in enumerate(order):
        sl = slice(leaf_base[y] - 1, leaf_base[y] - 1 + k)
        kind[sl] = PCB_INPUT
        var[sl] = y + 1
        ncat[sl] = num_cats
        hstart[sl] = hpos + 1 + np.arange(k) * hl
        lp = _dirichlet_log(rng, k, num_cats) if rng is not None else np.tile(_loguniform(num_cats), (k, 1))
        heap[hpos:hpos + k * hl].reshape(k, hl)[:, :num_cats] = lp
        input_ids[i * k:(i + 1) * k] = leaf_base[y] + np.arange(k)
        hpos += k * hl
        if ch[y]:
            if len(ch[y]) > 1:
                kind[prod_base[y] - 1:prod_base[y] - 1 + k] = PCB_PRODUCT
            kind[sum_base[y] - 1:sum_base[y] - 1 + (1 if y == root else k)] = PCB_SUM

    # ---- edge groups: (layer, first parent id, kind, y) ---------------------------------------
    groups = []
    for y in order:
        if not ch[y]:
            continue
        if len(ch[y]) > 1:
            groups.append((int(prod_layer[y]), int(prod_base[y]), 0, y))
        groups.append((int(sum_layer[y]), int(sum_base[y]), 1, y))
    groups.sort()
    sizes = []
    for _, _, gk, y in groups:
        if gk == 0:
            sizes.append(k * ((len(ch[y]) + 1) // 2))
        else:
            sizes.append((1 if y == root else k) * k)
    offs = np.concatenate([[0], np.cumsum(sizes)])
    n_edges = int(offs[-1])
    up_parent = np.zeros(n_edges, np.uint32)
    up_prime = np.zeros(n_edges, np.uint32)
    up_sub = np.zeros(n_edges, np.uint32)
    up_logp = np.zeros(n_edges, np.float32)
    up_tag = np.zeros(n_edges, np.uint8)
    up_ends = []
    # depth from the root of each CLT node's sums (every edge into a node precedes its out-edges)
    sum_dl = np.zeros(v, np.int64)
    for y in reversed(order):
        if not ch[y]:
            continue
        d_children = sum_dl[y] + (2 if len(ch[y]) > 1 else 1)
        for x in ch[y]:
            sum_dl[x] = d_children
    runs = []  # (down layer, prime base, up-edge ids ordered by prime)
    ar = np.arange(k)
    ar32 = np.arange(k, dtype=np.uint32)
    for gi, (lay, _, gk, y) in enumerate(groups):
        o = int(offs[gi])
        if gk == 0:
            m = len(ch[y])
            h = (m + 1) // 2
            idx = o + (ar[:, None] * h + np.arange(h)[None, :])          # [j, i]
            up_parent[idx] = (prod_base[y] + ar)[:, None]
            for i in range(h):
                up_prime[idx[:, i]] = out_base[ch[y][2 * i]] + ar
                if 2 * i + 1 < m:
                    up_sub[idx[:, i]] = out_base[ch[y][2 * i + 1]] + ar
                    up_tag[idx[:, i]] |= TAG_ONLYSUB
                runs.append((int(sum_dl[y]) + 2, int(out_base[ch[y][2 * i]]), idx[:, i].copy()))
            up_tag[idx[:, 0]] |= TAG_FIRST
            up_tag[idx[:, h - 1]] |= TAG_LAST
        else:
            r = 1 if y == root else k
            sl = slice(o, o + r * k)
            pb = prod_base[y] if len(ch[y]) > 1 else out_base[ch[y][0]]
            up_parent[sl].reshape(r, k)[:] = (sum_base[y] + np.arange(r, dtype=np.uint32))[:, None]
            up_prime[sl].reshape(r, k)[:] = (pb + ar32)[None, :]
            up_sub[sl].reshape(r, k)[:] = (leaf_base[y] + ar32)[None, :]
            if rng is not None:
                up_logp[sl].reshape(r, k)[:] = _dirichlet_log(rng, r, k)
            else:
                up_logp[sl] = -np.log(k)
            tg = up_tag[sl].reshape(r, k)
            tg[:, 0] |= TAG_FIRST
            tg[:, k - 1] |= TAG_LAST
            if r == 1:
                tg[:] |= TAG_ONLYSUB
            # down order of the block: by prime child j, then by parent c
            runs.append((int(sum_dl[y]) + 1, int(pb), (np.uint32(o) + (ar32[:, None] + np.arange(r, dtype=np.uint32)[None, :] * np.uint32(k))).reshape(-1)))
        if gi + 1 == len(groups) or groups[gi + 1][0] != lay:
            up_ends.append(int(offs[gi + 1]))
    runs.sort(key=lambda t: (t[0], t[1]))
    down2up = np.concatenate([np.asarray(r[2], dtype=np.uint32) for r in runs])
    down2up += np.uint32(1)
    down_ends, pos = [], 0
    for i, r in enumerate(runs):
        pos += len(r[2])
        if i + 1 == len(runs) or runs[i + 1][0] != r[0]:
            down_ends.append(pos)
    meta = {"kind": "hclt", "k": k, "num_cats": num_cats, "num_clt_inner": int(sum(1 for c in ch if c)),
            "clt_depth": int(sum_dl.max())}
    return FlatCircuit(kind, var, ncat, hstart, fixed, up_parent, up_prime, up_sub, up_logp, up_tag,
                       up_ends, down2up, down_ends, input_ids, heap, v, meta)
