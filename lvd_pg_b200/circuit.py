"""Compiled circuits in the reference's flattened order.

`FlatCircuit` holds what `BitsProbCircuit` holds on the Julia side (fields used at
VariationalJuice.jl/src/bits_circuit.jl:40-42,76-99): nodes in children-before-parent order
with the root last, up-edges grouped by layer with a parent's edges contiguous, the
down-edge permutation, the input-node list and the leaf heap.  All ids are 1-based.

`compile_circuit` turns a small node graph (`Input` / `Product` / `Sum`) into that form and
is what the tests use to restate the hand-built circuits of
VariationalJuice.jl/test/helpers/simple_circuits.jl.  The facts it reproduces are the ones
the reference's own tests pin: post-order numbering (test/queries/sample_tests.jl:136-144),
a product of m children stored as ceil(m/2) (prime, sub) edges
(test/queries/likelihood_tests.jl:28-31), non-materialised single-child nodes
(bits_circuit.jl:140-142), root edges last in up order and first in down order
(test/misc_tests.jl:27-30).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

PCB_INPUT, PCB_PRODUCT, PCB_SUM = 0, 1, 2
TAG_FIRST, TAG_LAST, TAG_PARTIAL, TAG_ONLYSUB, TAG_USER = 1, 2, 4, 8, 16


class PcbCircuitDesc(C.Structure):
    """ctypes mirror of `pcb_circuit_desc` (include/pcb200.h)."""

    _fields_ = [
        ("num_nodes", C.c_uint32),
        ("num_edges", C.c_uint32),
        ("num_up_layers", C.c_uint32),
        ("num_down_layers", C.c_uint32),
        ("num_input_nodes", C.c_uint32),
        ("num_vars", C.c_uint32),
        ("heap_len", C.c_uint64),
        ("node_kind", C.c_void_p),
        ("node_var", C.c_void_p),
        ("node_num_cats", C.c_void_p),
        ("node_heap_start", C.c_void_p),
        ("node_fixed", C.c_void_p),
        ("up_parent", C.c_void_p),
        ("up_prime", C.c_void_p),
        ("up_sub", C.c_void_p),
        ("up_logp", C.c_void_p),
        ("up_tag", C.c_void_p),
        ("up_layer_ends", C.c_void_p),
        ("down2up", C.c_void_p),
        ("down_layer_ends", C.c_void_p),
        ("input_node_ids", C.c_void_p),
        ("heap", C.c_void_p),
    ]


def _arr(a, dtype):
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


@dataclass
class FlatCircuit:
    node_kind: np.ndarray
    node_var: np.ndarray
    node_num_cats: np.ndarray
    node_heap_start: np.ndarray
    node_fixed: np.ndarray
    up_parent: np.ndarray
    up_prime: np.ndarray
    up_sub: np.ndarray
    up_logp: np.ndarray
    up_tag: np.ndarray
    up_layer_ends: np.ndarray
    down2up: np.ndarray
    down_layer_ends: np.ndarray
    input_node_ids: np.ndarray
    heap: np.ndarray
    num_vars: int
    meta: dict = field(default_factory=dict)

    def __post_init__(self):
        self.node_kind = _arr(self.node_kind, np.uint8)
        self.node_var = _arr(self.node_var, np.uint32)
        self.node_num_cats = _arr(self.node_num_cats, np.uint32)
        self.node_heap_start = _arr(self.node_heap_start, np.uint32)
        self.node_fixed = _arr(self.node_fixed, np.uint8)
        self.up_parent = _arr(self.up_parent, np.uint32)
        self.up_prime = _arr(self.up_prime, np.uint32)
        self.up_sub = _arr(self.up_sub, np.uint32)
        self.up_logp = _arr(self.up_logp, np.float32)
        self.up_tag = _arr(self.up_tag, np.uint8)
        self.up_layer_ends = _arr(self.up_layer_ends, np.uint32)
        self.down2up = _arr(self.down2up, np.uint32)
        self.down_layer_ends = _arr(self.down_layer_ends, np.uint32)
        self.input_node_ids = _arr(self.input_node_ids, np.uint32)
        self.heap = _arr(self.heap, np.float32)

    # -- counters (bits_circuit.jl:119-131) ------------------------------------------------
    @property
    def num_nodes(self) -> int:
        return int(self.node_kind.shape[0])

    @property
    def num_edges(self) -> int:
        return int(self.up_parent.shape[0])

    @property
    def edge_is_sum(self) -> np.ndarray:
        return self.node_kind[self.up_parent.astype(np.int64) - 1] == PCB_SUM

    @property
    def num_inner_params(self) -> int:
        return int(self.edge_is_sum.sum())

    @property
    def num_input_params(self) -> int:
        ids = self.input_node_ids.astype(np.int64) - 1
        return int((self.node_num_cats[ids] * (1 - self.node_fixed[ids])).sum())

    @property
    def num_parameters(self) -> int:
        return self.num_inner_params + self.num_input_params

    def desc(self) -> PcbCircuitDesc:
        """A descriptor whose pointers stay valid while `self` is alive."""
        d = PcbCircuitDesc()
        d.num_nodes = self.num_nodes
        d.num_edges = self.num_edges
        d.num_up_layers = int(self.up_layer_ends.shape[0])
        d.num_down_layers = int(self.down_layer_ends.shape[0])
        d.num_input_nodes = int(self.input_node_ids.shape[0])
        d.num_vars = int(self.num_vars)
        d.heap_len = int(self.heap.shape[0])
        for name in ("node_kind", "node_var", "node_num_cats", "node_heap_start", "node_fixed",
                     "up_parent", "up_prime", "up_sub", "up_logp", "up_tag", "up_layer_ends",
                     "down2up", "down_layer_ends", "input_node_ids", "heap"):
            setattr(d, name, getattr(self, name).ctypes.data)
        return d

    def copy(self) -> "FlatCircuit":
        kw = {k: (v.copy() if isinstance(v, np.ndarray) else v) for k, v in self.__dict__.items()}
        kw["meta"] = dict(self.meta)
        return FlatCircuit(**kw)


# ---------------------------------------------------------------------------------------------
# node graph
# ---------------------------------------------------------------------------------------------
class PCNode:
    pass


class Input(PCNode):
    """Categorical leaf over `var` (1-based) with values 0..C-1
    (FixableCategorical, nodes/fixable_categorical_dist.jl:4-31)."""

    def __init__(self, var: int, logps: Sequence[float], fixed: bool = False):
        self.var = int(var)
        self.logps = np.asarray(logps, dtype=np.float32)
        self.fixed = bool(fixed)


class Product(PCNode):
    def __init__(self, children: Sequence[PCNode]):
        self.children = list(children)


class Sum(PCNode):
    def __init__(self, children: Sequence[PCNode], logps: Optional[Sequence[float]] = None):
        self.children = list(children)
        if logps is None:
            logps = np.full(len(self.children), -np.log(len(self.children)), dtype=np.float32)
        self.logps = np.asarray(logps, dtype=np.float32)
        assert self.logps.shape[0] == len(self.children)


def multiply(*children: PCNode) -> Product:
    return Product(children)


def summate(*children: PCNode) -> Sum:
    return Sum(children)


def compile_circuit(root: PCNode, collapse_elements: bool = True, return_ids: bool = False):
    """Flatten a node graph the way `BitsProbCircuit(pc)` does (see module docstring).  With
    `return_ids` also returns {id(node): 1-based node id} of the materialised nodes."""

    def resolve(n: PCNode) -> PCNode:
        # a non-root inner node with one child is not materialised
        while n is not root and not isinstance(n, Input) and len(n.children) == 1:
            n = n.children[0]
        return n

    def edge_children(n: PCNode):
        """[(prime, sub_or_None, logp)] of a materialised inner node."""
        out = []
        if isinstance(n, Sum):
            for ch, lp in zip(n.children, n.logps):
                r = resolve(ch)
                if collapse_elements and isinstance(r, Product) and len(r.children) == 2:
                    out.append((resolve(r.children[0]), resolve(r.children[1]), float(lp)))
                else:
                    out.append((r, None, float(lp)))
        else:
            ch = [resolve(c) for c in n.children]
            for i in range(0, len(ch), 2):
                out.append((ch[i], ch[i + 1] if i + 1 < len(ch) else None, 0.0))
        return out

    # iterative post-order over materialised nodes
    ids = {}
    order: List[PCNode] = []
    edges_of = {}
    stack = [(root, False)]
    while stack:
        n, done = stack.pop()
        if id(n) in ids:
            continue
        if done or isinstance(n, Input):
            ids[id(n)] = len(order) + 1
            order.append(n)
            continue
        if id(n) not in edges_of:
            edges_of[id(n)] = edge_children(n)
        stack.append((n, True))
        for prime, sub, _ in reversed(edges_of[id(n)]):
            if sub is not None and id(sub) not in ids:
                stack.append((sub, False))
            if id(prime) not in ids:
                stack.append((prime, False))

    N = len(order)
    kind = np.zeros(N, np.uint8)
    var = np.zeros(N, np.uint32)
    ncat = np.zeros(N, np.uint32)
    hstart = np.zeros(N, np.uint32)
    fixed = np.zeros(N, np.uint8)
    layer = np.zeros(N, np.int64)
    heap: List[np.ndarray] = []
    heap_len = 0
    input_ids = []
    num_vars = 0
    for i, n in enumerate(order):
        if isinstance(n, Input):
            kind[i] = PCB_INPUT
            var[i] = n.var
            ncat[i] = n.logps.shape[0]
            fixed[i] = n.fixed
            hstart[i] = heap_len + 1
            heap.append(n.logps)
            heap_len += n.logps.shape[0]
            if not n.fixed:  # C flow slots + the `missing` slot
                heap.append(np.zeros(n.logps.shape[0] + 1, np.float32))
                heap_len += n.logps.shape[0] + 1
            input_ids.append(i + 1)
            num_vars = max(num_vars, n.var)
        else:
            kind[i] = PCB_SUM if isinstance(n, Sum) else PCB_PRODUCT
            lay = 0
            for prime, sub, _ in edges_of[id(n)]:
                lay = max(lay, layer[ids[id(prime)] - 1])
                if sub is not None:
                    lay = max(lay, layer[ids[id(sub)] - 1])
            layer[i] = lay + 1

    up_parent, up_prime, up_sub, up_logp, up_tag, up_ends = [], [], [], [], [], []
    for lay in range(1, int(layer.max()) + 1 if N else 1):
        for i in np.nonzero(layer == lay)[0]:
            es = edges_of[id(order[i])]
            for j, (prime, sub, lp) in enumerate(es):
                up_parent.append(i + 1)
                up_prime.append(ids[id(prime)])
                up_sub.append(ids[id(sub)] if sub is not None else 0)
                up_logp.append(lp)
                up_tag.append((TAG_FIRST if j == 0 else 0) | (TAG_LAST if j == len(es) - 1 else 0))
        up_ends.append(len(up_parent))
    fc = finish_flat(kind, var, ncat, hstart, fixed, up_parent, up_prime, up_sub, up_logp, up_tag,
                     up_ends, input_ids, np.concatenate(heap) if heap else np.zeros(0, np.float32),
                     num_vars)
    return (fc, ids) if return_ids else fc


def compile_multihead(pcs: Sequence[PCNode], collapse_elements: bool = True):
    """`CuMultiHeadBitsProbCircuit(pcs)` (src-jl/multi_head_pc/bit_circuit.jl:14-56): the heads go
    under a fake root, a sum over them, so that one flat circuit holds all of them; the fake root's
    edges carry TAG_USER, which every top-down pass skips.  Returns (FlatCircuit, root_ids), root_ids
    the 1-based node ids of the heads in the order given."""
    fake = summate(*pcs)
    fc, ids = compile_circuit(fake, collapse_elements, return_ids=True)
    root_ids = []
    for pc in pcs:
        if id(pc) not in ids:
            raise ValueError("a head is not a materialised node of the flat circuit")
        root_ids.append(ids[id(pc)])
    sel = fc.up_parent == fc.num_nodes
    if not np.array_equal(np.sort(fc.up_prime[sel]), np.sort(np.asarray(root_ids, fc.up_prime.dtype))) or fc.up_sub[sel].any():
        raise ValueError("every head must be a child of the fake root by an edge of its own")
    fc.up_tag[sel] |= TAG_USER
    return fc, np.asarray(root_ids, np.uint32)


def finish_flat(kind, var, ncat, hstart, fixed, up_parent, up_prime, up_sub, up_logp, up_tag, up_ends,
                input_ids, heap, num_vars, meta=None) -> FlatCircuit:
    """Derive the down-edge order (grouped by layer from the root, by prime child within a
    layer) and its tags, then assemble a FlatCircuit."""
    up_parent = np.asarray(up_parent, np.int64)
    up_prime = np.asarray(up_prime, np.int64)
    up_sub = np.asarray(up_sub, np.int64)
    up_tag = np.asarray(up_tag, np.uint8).copy()
    N = len(kind)
    E = len(up_parent)
    # depth from the root: every edge into a node is processed before any edge out of it
    dl = np.zeros(N + 1, np.int64)
    order = np.argsort(-up_parent, kind="stable")  # parents in descending id
    # nodes are topologically numbered, so one pass over edges by descending parent id suffices
    # when done group by group; do it with a python loop over distinct parents for small
    # circuits and a vectorised relaxation for large ones.
    if E <= 200000:
        for e in order:
            d = dl[up_parent[e]] + 1
            if dl[up_prime[e]] < d:
                dl[up_prime[e]] = d
            if up_sub[e] and dl[up_sub[e]] < d:
                dl[up_sub[e]] = d
    else:
        changed = True
        while changed:
            d = dl[up_parent] + 1
            new = dl.copy()
            np.maximum.at(new, up_prime, d)
            m = up_sub > 0
            np.maximum.at(new, up_sub[m], d[m])
            changed = bool((new != dl).any())
            dl = new
    dlayer = dl[up_parent] + 1
    down_order = np.lexsort((np.arange(E), up_prime, dlayer))  # by layer, prime, up id
    down2up = down_order + 1
    dl_sorted = dlayer[down_order]
    down_ends = (np.nonzero(np.diff(dl_sorted))[0] + 1).tolist() + ([E] if E else [])
    # PARTIAL: a prime child whose incoming edges fall into several down layers;
    # ONLYSUB: the edge is the only one that writes flows[sub]
    if E:
        ref = np.bincount(np.concatenate([up_prime, up_sub[up_sub > 0]]), minlength=N + 1)
        lo = np.full(N + 1, np.iinfo(np.int64).max)
        hi = np.zeros(N + 1, np.int64)
        np.minimum.at(lo, up_prime, dlayer)
        np.maximum.at(hi, up_prime, dlayer)
        up_tag[(lo[up_prime] != hi[up_prime])] |= TAG_PARTIAL
        up_tag[(up_sub > 0) & (ref[up_sub] == 1)] |= TAG_ONLYSUB
    return FlatCircuit(kind, var, ncat, hstart, fixed, up_parent, up_prime, up_sub, up_logp, up_tag,
                       up_ends, down2up, down_ends, input_ids, heap, num_vars, meta or {})
