"""`.jpc` files: a round trip through lvd_pg_b200.jpc keeps the circuit (node order, edges, parameters),
and a file written by hand in the published syntax is read as the circuit it describes.  The format
itself is not pinned against ProbabilisticCircuits.jl, which the reference does not vendor."""
import numpy as np
import pytest

from lvd_pg_b200 import jpc, structures as st
from lvd_pg_b200.circuit import Input, compile_circuit, compile_multihead
from oracle import oracle as orc


def _same_flat(a, b):
    for f in ("node_kind", "node_var", "node_num_cats", "node_heap_start", "node_fixed", "up_parent", "up_prime",
              "up_sub", "up_tag", "up_layer_ends", "down2up", "down_layer_ends", "input_node_ids"):
        assert np.array_equal(getattr(a, f), getattr(b, f)), f
    np.testing.assert_array_equal(a.up_logp, b.up_logp)
    np.testing.assert_array_equal(a.heap, b.heap)


@pytest.mark.parametrize("make", [
    lambda: st.simple_3vars_circuit(num_cats=5, fixed=False, rng=np.random.default_rng(0)),
    lambda: st.hclt_graph(st.root_tree_at_center(7, st.random_spanning_tree(7, np.random.default_rng(1))), 3, 4,
                          np.random.default_rng(2)),
    lambda: st.fully_factorized_categorical_fixed(3, 8),
], ids=["simple3", "hclt_v7_k4", "fixed_leaves"])
def test_round_trip_keeps_the_flat_circuit(tmp_path, make):
    pc = make()
    path = str(tmp_path / "c.jpc")
    n = jpc.write_jpc(path, pc)
    assert n > 0
    back = jpc.read_jpc(path, fixed_inputs=_all_fixed(pc))   # the format has no "fixed" attribute
    _same_flat(compile_circuit(pc), compile_circuit(back))


def _all_fixed(pc):
    seen, stack, out = set(), [pc], []
    while stack:
        n = stack.pop()
        if id(n) in seen:
            continue
        seen.add(id(n))
        if isinstance(n, Input):
            out.append(n.fixed)
        else:
            stack.extend(n.children)
    return all(out)


def test_multihead_round_trip(tmp_path):
    pcs = st.simple_multihead_circuit(num_cats=5, heads=3, rng=np.random.default_rng(3))
    path = str(tmp_path / "mh.jpc")
    jpc.write_mhpc(path, pcs)
    back = jpc.read_mhpc(path)
    assert len(back) == 3
    a, ra = compile_multihead(pcs)
    b, rb = compile_multihead(back)
    _same_flat(a, b)
    assert ra.tolist() == rb.tolist()


def test_hand_written_file(tmp_path):
    # two variables, a mixture of two products of categorical leaves, one indicator, one literal
    text = """c hand-written
jpc 8
C 0 -1 1 -0.6931471805599453 -0.6931471805599453
C 1 -1 2 -1.6094379124341003 -0.2231435513142097
I 2 -1 1 1
L 3 -1 -2
P 4 -1 2 0 1
P 5 -1 2 2 3
S 6 -1 2 4 -0.35667494393873245 5 -1.2039728043259361
S 7 -1 1 6 0.0
"""
    path = tmp_path / "h.jpc"
    path.write_text(text)
    fc = compile_circuit(jpc.read_jpc(str(path), num_cats=2))
    data = np.array([[0, 0], [1, 1], [1, 0]], np.uint8)
    ll = orc.forward(fc, data)[:, -1]
    # P(x1, x2) = 0.7 * 0.5 * p2(x2) + 0.3 * [x1 = 1] * [x2 = 0]
    want = np.log([0.7 * 0.5 * 0.2, 0.7 * 0.5 * 0.8, 0.7 * 0.5 * 0.2 + 0.3])
    np.testing.assert_allclose(ll, want, rtol=1e-5)


def test_declared_count_is_checked(tmp_path):
    path = tmp_path / "bad.jpc"
    path.write_text("jpc 3\nC 0 -1 1 0.0\n")
    with pytest.raises(ValueError):
        jpc.read_jpc(str(path))
