"""Reading and writing circuits as `.jpc` text files.

`.jpc` is the text format of ProbabilisticCircuits.jl (`JpcFormat`), which the reference reads with
`read(file, ProbCircuit, JpcFormat(), true)` (VariationalJuice.jl/src/transformations.jl:4-13) and
writes through `write(file, pc)` (src-jl/multi_head_pc/io.jl:1-9).  That package is a dependency the
reference does not vendor, so the grammar below is a restatement of its published format (version 0.4,
`io/jpc_io.jl`) and is NOT pinned against files the package wrote; only a round trip through this
module is tested.  The format, one node per line, children before parents, ids from 0:

    c <comment>
    jpc <number of nodes>
    C <id> <vtree id or -1> <variable, 1-based> <log-probability>+       categorical leaf
    I <id> <vtree id or -1> <variable> <value>                           indicator leaf
    L <id> <vtree id or -1> <signed literal>                             boolean literal
    P <id> <vtree id or -1> <number of children> <child id>+             product
    S <id> <vtree id or -1> <number of children> (<child id> <log-prob>)+  sum

Binomial leaves (`B`) have no counterpart in this library and are refused.  An indicator or a literal
becomes a fixed categorical leaf with probability one on its value (`num_cats` categories; 2 for
literals).
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np

from .circuit import Input, PCNode, Product, Sum, summate

HEADER = """c this file was saved by lvd_pg_b200.jpc in the format of ProbabilisticCircuits.jl
c ids of jpc nodes start at 0
c jpc nodes appear bottom-up, children before parents
c
c file syntax:
c jpc count-of-jpc-nodes
c L id-of-jpc-node id-of-vtree literal
c I id-of-jpc-node id-of-vtree variable indicator-value
c C id-of-jpc-node id-of-vtree variable {log-probability}+
c P id-of-product-jpc-node id-of-vtree number-of-children {child-id}+
c S id-of-sum-jpc-node id-of-vtree number-of-children {child-id log-probability}+
c
"""


def _fmt(x: float) -> str:
    return "-Inf" if x == -np.inf else repr(float(np.float32(x)))


def write_jpc(path: str, root: PCNode) -> int:
    """Writes the node graph under `root`; returns the number of nodes written."""
    ids: Dict[int, int] = {}
    lines: List[str] = []
    stack = [(root, False)]
    while stack:   # iterative post-order, every node once
        n, done = stack.pop()
        if id(n) in ids:
            continue
        if isinstance(n, Input) or done:
            nid = len(ids)
            ids[id(n)] = nid
            if isinstance(n, Input):
                lines.append(f"C {nid} -1 {n.var} " + " ".join(_fmt(v) for v in n.logps))
            elif isinstance(n, Product):
                lines.append(f"P {nid} -1 {len(n.children)} " + " ".join(str(ids[id(c)]) for c in n.children))
            else:
                lines.append(f"S {nid} -1 {len(n.children)} " +
                             " ".join(f"{ids[id(c)]} {_fmt(lp)}" for c, lp in zip(n.children, n.logps)))
            continue
        stack.append((n, True))
        for c in reversed(n.children):
            if id(c) not in ids:
                stack.append((c, False))
    with open(path, "w") as f:
        f.write(HEADER)
        f.write(f"jpc {len(lines)}\n")
        f.write("\n".join(lines) + "\n")
    return len(lines)


def _num(tok: str) -> float:
    t = tok.lower()
    if t in ("-inf", "-infinity"):
        return -np.inf
    return float(tok)


def read_jpc(path: str, num_cats: int = 2, fixed_inputs: bool = False) -> PCNode:
    """Reads a `.jpc` file into a node graph and returns its root (the last node).  `num_cats` sizes
    the leaves that indicator lines stand for; `fixed_inputs` marks categorical leaves as not learnable."""
    nodes: Dict[int, PCNode] = {}
    declared = None
    last = None
    with open(path) as f:
        for ln, raw in enumerate(f, 1):
            line = raw.strip()
            if not line or line.startswith("c"):
                continue
            tok = line.split()
            kind = tok[0]
            if kind == "jpc":
                declared = int(tok[1])
                continue
            nid = int(tok[1])
            if kind == "C":
                node = Input(int(tok[3]), [_num(t) for t in tok[4:]], fixed_inputs)
            elif kind == "I":
                var, val = int(tok[3]), int(tok[4])
                lp = np.full(max(num_cats, val + 1), -np.inf, np.float32)
                lp[val] = 0.0
                node = Input(var, lp, True)
            elif kind == "L":
                lit = int(tok[3])
                lp = np.array([-np.inf, 0.0] if lit > 0 else [0.0, -np.inf], np.float32)
                node = Input(abs(lit), lp, True)
            elif kind == "P":
                k = int(tok[3])
                if len(tok) != 4 + k:
                    raise ValueError(f"{path}:{ln}: product line with {len(tok) - 4} children, {k} declared")
                node = Product([nodes[int(t)] for t in tok[4:]])
            elif kind == "S":
                k = int(tok[3])
                if len(tok) != 4 + 2 * k:
                    raise ValueError(f"{path}:{ln}: sum line with {len(tok) - 4} tokens, {2 * k} expected")
                node = Sum([nodes[int(t)] for t in tok[4::2]], [_num(t) for t in tok[5::2]])
            elif kind == "B":
                raise NotImplementedError(f"{path}:{ln}: binomial leaves are not supported")
            else:
                raise ValueError(f"{path}:{ln}: unknown node kind {kind!r}")
            if nid in nodes:
                raise ValueError(f"{path}:{ln}: node id {nid} appears twice")
            nodes[nid] = node
            last = node
    if declared is not None and declared != len(nodes):
        raise ValueError(f"{path}: {declared} nodes declared, {len(nodes)} read")
    if last is None:
        raise ValueError(f"{path}: no nodes")
    return last


def write_mhpc(path: str, pcs: Sequence[PCNode]) -> int:
    """write_mhpc (src-jl/multi_head_pc/io.jl:1-3): the heads under one sum."""
    return write_jpc(path, summate(*pcs))


def read_mhpc(path: str, **kw) -> List[PCNode]:
    """read_mhpc (src-jl/multi_head_pc/io.jl:5-8): the children of the file's root."""
    return list(read_jpc(path, **kw).children)
