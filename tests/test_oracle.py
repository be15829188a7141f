"""Pins the CPU checkers: the C restatement (oracle/ormi_oracle.c) against every known-answer test the
reference holds for the realize path, against the unmodified reference compiled into oracle/_ref, and
against the committed golden vectors; and the host-side autograd mirror against the reference's autograd."""
import math
import os

import numpy as np
import pytest

from ormi_b200 import graph as G
from ormi_b200 import workloads as W
from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
needs_ref = pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (needs the reference checkout)")


def port(*roots):
    return O.port_run(list(roots))[0]


def full(shape, v):
    return G.leaf(np.full(shape, v, dtype=np.float32))


# ---- known answers of ormi-core/csrc/tests/backend/cpu/test_jit.cpp (and its CUDA twin)
def test_jit_basic_execution():
    (c,) = port(G.add(full([4], 2.0), full([4], 3.0)))
    assert c.shape == (4,) and np.all(c == 5.0)


def test_jit_tape_chaining():
    (d,) = port(G.mul(G.add(full([2, 2], 2.0), full([2, 2], 3.0)), full([2, 2], 4.0)))
    assert np.all(d == 20.0)


def test_jit_broadcasting():
    (c,) = port(G.add(full([2, 3], 2.0), full([3], 5.0)))
    assert c.shape == (2, 3) and np.all(c == 7.0)


def test_jit_scalar():
    (c,) = port(G.add(full([2, 2], 10.0), full([], 3.0)))
    assert np.all(c == 13.0)


def test_jit_unary_math():
    (b,) = port(G.sin(full([2], 1.570796327)))
    assert np.allclose(b, 1.0, atol=1e-5)


# ---- ormi-core/csrc/tests/backend/cpu/kernels/reduce/test_sum.cpp
def test_sum_known_answers():
    a = G.leaf(np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32))
    (g, ax, kd) = port(G.sum_(a, [], False), G.sum_(a, [1], False), G.sum_(a, [0], True))
    assert g.shape == () and g == 21.0
    assert ax.tolist() == [6.0, 15.0]
    assert kd.shape == (1, 3) and kd.tolist() == [[5.0, 7.0, 9.0]]
    cube = G.leaf(np.arange(1, 9, dtype=np.float32).reshape(2, 2, 2))
    (m,) = port(G.sum_(cube, [0, 2], False))
    assert m.tolist() == [14.0, 22.0]


# ---- ormi-core/csrc/tests/core/test_ops.cpp
def test_ops_sums_and_matmuls():
    a = full([2, 3], 2.0)
    (flat, kept) = port(G.sum_(a, [], False), G.sum_(a, [], True))
    assert flat == 12.0 and kept.shape == (1, 1) and kept[0, 0] == 12.0
    (r,) = port(G.sum_(full([2, 3, 2], 1.0), [0, 2], False))
    assert r.tolist() == [4.0, 4.0, 4.0]
    (mm,) = port(G.matmul(full([2, 3], 2.0), full([3, 2], 3.0)))
    assert mm.shape == (2, 2) and np.all(mm == 18.0)
    (bm,) = port(G.matmul(full([2, 1, 2, 3], 1.5), full([1, 2, 3, 2], 2.0)))
    assert bm.shape == (2, 2, 2, 2) and np.all(bm == 9.0)
    with pytest.raises(RuntimeError):
        G.matmul(full([2, 3], 1.0), full([2, 2], 1.0))
    with pytest.raises(RuntimeError):
        G.matmul(full([3], 1.0), full([3], 1.0))
    with pytest.raises(RuntimeError):
        G.matmul(full([2, 2, 3], 1.0), full([3, 3, 2], 1.0))


# ---- ormi-core/csrc/tests/backend/cpu/kernels/blas/test_matmul.cpp
def test_matmul_kernel_known_answers():
    a = G.leaf(np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32))
    b = G.leaf(np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32))
    (c,) = port(G.matmul(a, b))
    assert c.reshape(-1).tolist() == [58.0, 64.0, 139.0, 154.0]
    # transposed strides {1, 3}: a [3,2] view of the same six numbers
    (ct,) = port(G.matmul(G.transpose(a, [1, 0]), G.leaf(np.array([[1, 2], [3, 4]], dtype=np.float32))))
    assert ct.reshape(-1).tolist() == [13.0, 18.0, 17.0, 24.0, 21.0, 30.0]
    # batched, B broadcast with stride 0
    a3 = G.leaf(np.arange(1, 13, dtype=np.float32).reshape(2, 2, 3))
    b2 = G.leaf(np.arange(1, 7, dtype=np.float32).reshape(1, 3, 2))
    (cb,) = port(G.matmul(a3, G.expand(b2, [2, 3, 2])))
    assert cb.reshape(-1).tolist() == [22.0, 28.0, 49.0, 64.0, 76.0, 100.0, 103.0, 136.0]


# ---- ormi-core/tests/test_tensor.py
def test_python_surface_known_answers():
    a, b = G.leaf([4.0, 6.0]), G.leaf([2.0, 3.0])
    outs = port(G.add(a, b), G.sub(a, b), G.mul(a, b), G.div(a, b), G.neg(a), G.pow_(a, G.const(2.0)))
    assert [o.tolist() for o in outs] == [[6.0, 9.0], [2.0, 3.0], [8.0, 18.0], [2.0, 2.0], [-4.0, -6.0], [16.0, 36.0]]
    m = G.leaf([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    (rs, tr) = port(G.reshape(m, [3, 2]), G.transpose(m, [1, 0]))
    assert rs.tolist() == [[1, 2], [3, 4], [5, 6]] and tr.tolist() == [[1, 4], [2, 5], [3, 6]]
    x, y = G.leaf([2.0, 3.0], True), G.leaf([4.0, 5.0], True)
    z = G.add(G.mul(x, y), x)
    G.compute_gradients(z)
    (dx, dy) = port(x.grad, y.grad)
    assert dx.tolist() == [5.0, 6.0] and dy.tolist() == [2.0, 3.0]


# ---- the restatement against the unmodified reference
def _softmax_case(R, C):
    x = G.leaf(W.normal(0, (R, C), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(1, (R, C)))
    y = W.softmax(x)
    return x, gy, y


@needs_ref
def test_port_matches_reference_bitwise_softmax_layernorm():
    x, gy, y = _softmax_case(48, 160)
    ref, _ = O.ref_run([(y, "value"), (x, "grad")], seeds=[(y, gy)], backward_root=y)
    y.grad = gy
    G.compute_gradients(y)
    mine = port(y, x.grad)
    assert all(np.array_equal(a, b) for a, b in zip(ref, mine))

    x = G.leaf(W.normal(0, (40, 96), math.sqrt(2.0)), True)
    g = G.leaf(W.uniform(2, (96,), 0.5, 1.5), True)
    b = G.leaf(W.normal(3, (96,), 0.1), True)
    gy = G.leaf(W.normal(1, (40, 96)))
    y = W.layernorm(x, g, b)
    outs = [(y, "value"), (x, "grad"), (g, "grad"), (b, "grad")]
    ref, _ = O.ref_run(outs, seeds=[(y, gy)], backward_root=y)
    y.grad = gy
    G.compute_gradients(y)
    mine = port(y, x.grad, g.grad, b.grad)
    assert all(np.array_equal(a, b_) for a, b_ in zip(ref, mine))


@needs_ref
def test_port_matches_reference_config1_and_mlp():
    a, b, c = (G.leaf(W.normal(i, (32, 128))) for i in range(3))
    y = W.fused_rowsum(a, b, c)
    ref, _ = O.ref_run([(y, "value")])
    assert np.array_equal(ref[0], port(y)[0])

    B, D, H = 16, 8, 32
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(np.zeros(H, np.float32), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(np.zeros(D, np.float32), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    outs = [(loss, "value")] + [(p, "grad") for p in (w1, b1, w2, b2)]
    ref, _ = O.ref_run(outs, backward_root=loss)
    G.compute_gradients(loss)
    mine = port(loss, w1.grad, b1.grad, w2.grad, b2.grad)
    for r, m in zip(ref, mine):     # SGEMM order differs between OpenBLAS and the k-ascending restatement
        assert np.abs(r - m).max() <= 1e-5 * max(1e-30, np.abs(r).max())


def _signature(c):
    return (c.op, c.n_parents, tuple(c.parents[:c.n_parents]), tuple(c.shape[:c.ndim]), tuple(c.strides[:c.ndim]),
            tuple(c.axes[:c.n_axes]), c.keepdims)


@needs_ref
@pytest.mark.parametrize("case", ["softmax", "layernorm", "mlp", "mixed"])
def test_autograd_mirror_builds_the_reference_graph(case):
    """ormi_b200.graph.compute_gradients must emit, node for node and in the same order, the graph the
    reference's compute_gradients emits (ormi-core/csrc/core/autograd.cpp:24-47)."""
    if case == "softmax":
        x, gy, y = _softmax_case(6, 10)
        params, root, seeds = [x], y, [(y, gy)]
    elif case == "layernorm":
        x = G.leaf(W.normal(0, (6, 10)), True)
        g, b = G.leaf(W.uniform(2, (10,), 0.5, 1.5), True), G.leaf(W.normal(3, (10,), 0.1), True)
        gy = G.leaf(W.normal(1, (6, 10)))
        root, params, seeds = W.layernorm(x, g, b), [x, g, b], None
        seeds = [(root, gy)]
    elif case == "mlp":
        x, t = G.leaf(W.normal(0, (6, 4))), G.leaf(W.normal(1, (6, 4)))
        w1, b1 = G.leaf(W.normal(2, (4, 8)), True), G.leaf(np.zeros(8, np.float32), True)
        w2, b2 = G.leaf(W.normal(3, (8, 4)), True), G.leaf(np.zeros(4, np.float32), True)
        root, params, seeds = W.mlp_loss(x, w1, b1, w2, b2, t), [w1, b1, w2, b2], []
    else:
        import make_golden
        root, params = make_golden.broadcast_views_forward()
        seeds = []
    outs = [(root, "value")] + [(p, "grad") for p in params]
    exp, n, origin, leaf_vals, out_index, _ = O.ref_export(outs, seeds=seeds, backward_root=root)
    for node, seed in seeds:
        node.grad = seed
    G.compute_gradients(root)
    arr, order, roots = G.flatten([root] + [p.grad for p in params], host_pointers=True)
    assert len(order) == n and roots == out_index
    for i in range(n):
        assert _signature(exp[i]) == _signature(arr[i]), f"node {i}"
        if origin[i] < 0 and exp[i].op == 0:   # a leaf the reference's autograd created: same constant
            assert np.all(order[i].data.host == np.float32(leaf_vals[i]))


def test_golden_vectors():
    """Outputs of the unmodified reference CPU backend, committed as fixtures (tests/golden/make_golden.py)."""
    import make_golden
    for name, build in make_golden.CASES.items():
        path = os.path.join(GOLDEN, name + ".npz")
        assert os.path.exists(path), f"{path} missing: run tests/golden/make_golden.py"
        want = np.load(path)
        roots = build()[0]
        got = port(*roots)
        for i, g in enumerate(got):
            w = want[f"out{i}"]
            if name.startswith("mlp"):
                assert np.abs(g - w).max() <= 1e-5 * np.abs(w).max()
            else:
                assert np.array_equal(g, w), f"{name} output {i}"
