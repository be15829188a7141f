"""Extension ops MAXIMUM, GE and MAX (no counterpart in the reference's OpEnum) plus the MEAN composition.

Nothing of the reference can pin these ops directly, so the chain is:
  1. the extended part of the oracle port against numpy, and against compositions the reference itself CAN
     evaluate (max(a, b) = (a + b + ((a - b)^2)^0.5) / 2; a stable softmax equals the plain one);
  2. the generated CUDA C (compiled for the CPU emulator here, for the B200 under ``-m gpu``) against the oracle port.
"""
import math

import numpy as np
import pytest

import emulator as E
from ormi_b200 import graph as G
from ormi_b200 import runtime as RT
from ormi_b200 import workloads as W
from oracle import oracle as O

PW_TOL, REDUCE_TOL = 1e-6, 1e-5
C = G.const


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(1e-30, np.abs(b).max()))


def graphs():
    """name -> (roots, numpy fp64 expectation or None)."""
    out = {}
    a_h, b_h = W.normal(0, (37, 200)), W.normal(1, (37, 200))
    row_h = W.normal(2, (200,))
    a, b, row = G.leaf(a_h), G.leaf(b_h), G.leaf(row_h)
    out["maximum_ge_broadcast"] = ([G.maximum(a, b), G.ge(a, b), G.maximum(a, row), G.maximum(a, C(0.25))],
                                   [np.maximum(a_h, b_h), (a_h >= b_h).astype(np.float32), np.maximum(a_h, row_h), np.maximum(a_h, 0.25)])
    x_h = W.normal(3, (24, 300), 3.0)
    x = G.leaf(x_h)
    out["max_every_kind"] = ([G.max_(x, [1], False), G.max_(x, [1], True), G.max_(x, [0], False), G.max_(x, [], False),
                              G.max_(G.mul(x, x), [1], True), G.mean(x, [1], True), G.mean(x, [0]), G.mean(x)],
                             [x_h.max(1), x_h.max(1, keepdims=True), x_h.max(0), x_h.max(), (x_h.astype(np.float64) ** 2).max(1, keepdims=True),
                              x_h.astype(np.float64).mean(1, keepdims=True), x_h.astype(np.float64).mean(0), x_h.astype(np.float64).mean()])
    t_h = W.normal(4, (5, 6, 7))
    t = G.leaf(t_h)
    # (a reduction over a transposed view is left out: the reference's SUM walk, which MAX shares, decodes coordinates from
    #  the view's strides and is wrong for views — the same divergence the SUM tests avoid)
    out["max_middle_axis"] = ([G.max_(t, [1], False), G.max_(t, [0, 2], True)], [t_h.max(1), t_h.max((0, 2), keepdims=True)])
    big_h = (W.normal(5, (16, 512)) * 30.0).astype(np.float32)           # exp overflows without the shift
    big = G.leaf(big_h)
    z = big_h.astype(np.float64) - big_h.astype(np.float64).max(1, keepdims=True)
    out["softmax_stable_large_logits"] = ([W.softmax_stable(big)], [np.exp(z) / np.exp(z).sum(1, keepdims=True)])
    return out


def backward_graphs():
    xs_h = W.normal(6, (24, 96), math.sqrt(2.0))
    xs, gy = G.leaf(xs_h, True), G.leaf(W.normal(7, (24, 96)))
    y = W.softmax_stable(xs)
    y.grad = gy
    G.compute_gradients(y)
    r_in = G.leaf(W.normal(8, (10, 64)), True)
    w = G.leaf(W.normal(9, (64,)), True)
    loss = G.sum_(G.mul(W.relu_max(G.mul(r_in, w)), G.max_(r_in, [1], True)), [], False)
    G.compute_gradients(loss)
    return {"softmax_stable_fwd_bwd": [y, xs.grad], "relu_and_rowmax_backward": [loss, r_in.grad, w.grad]}


@pytest.mark.parametrize("name", list(graphs()))
def test_oracle_extension_against_numpy(name):
    roots, want = graphs()[name]
    got, _ = O.port_run(roots)
    for g, w in zip(got, want):
        w = np.asarray(w)
        assert g.shape == w.shape
        assert rel(g, w) <= REDUCE_TOL


@pytest.mark.skipif(not O.ref_available(), reason="needs oracle/_ref (the reference compiled from its sources)")
def test_oracle_extension_against_reference_compositions():
    a_h, b_h = W.normal(0, (33, 65)), W.normal(1, (33, 65))
    a, b = G.leaf(a_h), G.leaf(b_h)
    d = G.sub(a, b)
    composed = G.mul(G.add(G.add(a, b), G.pow_(G.mul(d, d), C(0.5))), C(0.5))
    (ref_max,), _ = O.ref_run([(composed, "value")])
    (port_max,), _ = O.port_run([G.maximum(a, b)])
    assert rel(port_max, ref_max) <= 2 * PW_TOL
    x = G.leaf(W.normal(2, (24, 96), math.sqrt(2.0)))
    (ref_sm,), _ = O.ref_run([(W.softmax(x), "value")])
    (port_sm,), _ = O.port_run([W.softmax_stable(x)])
    assert rel(port_sm, ref_sm) <= REDUCE_TOL
    (ref_mean,), _ = O.ref_run([(G.mul(G.sum_(x, [1], True), C(1.0 / 96)), "value")])
    (port_mean,), _ = O.port_run([G.mean(x, [1], True)])
    np.testing.assert_array_equal(port_mean, ref_mean)


def test_autograd_rules_against_finite_differences():
    x_h = W.normal(11, (6, 9)).astype(np.float64)
    w_h = W.normal(12, (9,)).astype(np.float64)

    def f(xv, wv):
        return (np.maximum(xv * wv, 0.0) * xv.max(1, keepdims=True)).sum()
    x, w = G.leaf(x_h.astype(np.float32), True), G.leaf(w_h.astype(np.float32), True)
    loss = G.sum_(G.mul(W.relu_max(G.mul(x, w)), G.max_(x, [1], True)), [], False)
    G.compute_gradients(loss)
    (gx, gw), _ = O.port_run([x.grad, w.grad])
    eps = 1e-6
    num = np.zeros_like(x_h)
    for i in range(x_h.shape[0]):
        for j in range(x_h.shape[1]):
            p, m = x_h.copy(), x_h.copy()
            p[i, j] += eps
            m[i, j] -= eps
            num[i, j] = (f(p, w_h) - f(m, w_h)) / (2 * eps)
    assert rel(gx, num) <= 1e-4
    numw = np.array([(f(x_h, w_h + eps * np.eye(9)[j]) - f(x_h, w_h - eps * np.eye(9)[j])) / (2 * eps) for j in range(9)])
    assert rel(gw, numw) <= 1e-4


def _emulated(roots, tol):
    outs, plan = E.realize(roots)
    ref, _ = O.port_run(roots)
    for a, b in zip(outs, ref):
        assert a.shape == b.shape
        assert rel(a, b) <= tol
    return [s["what"].split("[")[0] if s["type"] == "kernel" else "gemm" for s in plan["steps"]]


@pytest.mark.parametrize("name", list(graphs()))
def test_generated_kernels_on_the_emulator(name):
    roots, _ = graphs()[name]
    _emulated(roots, REDUCE_TOL)


def test_stable_softmax_forward_backward_is_one_kernel():
    kinds = _emulated(backward_graphs()["softmax_stable_fwd_bwd"], REDUCE_TOL)
    assert kinds == ["rows"]
    _emulated(backward_graphs()["relu_and_rowmax_backward"], REDUCE_TOL)


def test_row_max_values_are_exact():
    x_h = W.normal(13, (9, 1000), 5.0)
    outs, _ = E.realize([G.max_(G.leaf(x_h), [1], False), G.max_(G.leaf(x_h), [0], False), G.max_(G.leaf(x_h), [], False)])
    np.testing.assert_array_equal(outs[0], x_h.max(1))
    np.testing.assert_array_equal(outs[1], x_h.max(0))
    np.testing.assert_array_equal(outs[2], x_h.max())


def test_full_size_schedule():
    fake = G.Node(G.OpEnum.LEAF, data=G.Buffer((16384, 4096), host=np.zeros(1, np.float32)), requires_grad=True)
    y = W.softmax_stable(fake)
    y.grad = G.Node(G.OpEnum.LEAF, data=G.Buffer((16384, 4096), host=np.zeros(1, np.float32)))
    G.compute_gradients(y)
    plan = RT.plan([y, fake.grad])
    assert not plan["error"]
    assert [s["what"].split("[")[0] for s in plan["steps"]] == ["rows"]
    assert plan["steps"][0]["bytes_read"] == 2 * 16384 * 4096 * 4


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(graphs()) + list(backward_graphs()))
def test_extension_ops_on_gpu(device, name):
    roots = graphs()[name][0] if name in graphs() else backward_graphs()[name]
    ref, _ = O.port_run(roots)
    for r, w in zip(roots, ref):
        g = device.numpy(r)
        assert g.shape == w.shape
        assert rel(g, w) <= REDUCE_TOL


@pytest.mark.gpu
def test_extension_ops_without_fusion_on_gpu(device):
    """One kernel per node (the generic reduction kernel carries the maximum too)."""
    device.set_option("fusion", "off")
    try:
        for name in ("max_every_kind", "softmax_stable_large_logits"):
            roots = graphs()[name][0]
            ref, _ = O.port_run(roots)
            for r, w in zip(roots, ref):
                assert rel(device.numpy(r), w) <= REDUCE_TOL
    finally:
        device.set_option("fusion", "on")


@pytest.mark.gpu
def test_stable_softmax_full_size_rows_on_gpu(device):
    """Full-size rows; sampled rows against fp64, and the size-independent properties: rows sum to one, the gradient rows
    sum to zero, the largest probability sits where the largest logit is."""
    R, Cn = 16384, 4096
    x_h, gy_h = W.normal(20, (R, Cn), 6.0), W.normal(21, (R, Cn))
    x, gy = device.leaf(x_h, requires_grad=True), device.leaf(gy_h)
    y = W.softmax_stable(x)
    y.grad = gy
    G.compute_gradients(y)
    device.realize([y, x.grad])
    y_h, dx_h = device.numpy(y), device.numpy(x.grad)
    assert np.abs(y_h.astype(np.float64).sum(1) - 1.0).max() <= 1e-5
    assert np.abs(dx_h.astype(np.float64).sum(1)).max() <= 1e-5
    np.testing.assert_array_equal(y_h.argmax(1), x_h.argmax(1))
    for r in (0, 1, R // 2, R - 1):
        z = x_h[r].astype(np.float64)
        p = np.exp(z - z.max())
        p /= p.sum()
        assert rel(y_h[r], p) <= REDUCE_TOL
        g = gy_h[r].astype(np.float64)
        assert rel(dx_h[r], p * (g - (p * g).sum())) <= 3 * REDUCE_TOL


def _random_graph(rng):
    unary = [G.neg, G.exp, G.sin, G.cos]
    binary = [G.add, G.sub, G.mul, G.maximum, G.ge]
    R, Cn = int(rng.integers(1, 9)), int(rng.choice([1, 4, 12, 33, 64, 130]))
    pool = [G.leaf(rng.uniform(-1.5, 1.5, size=s).astype(np.float32)) for s in ((R, Cn), (R, Cn), (Cn,), (R, 1), ())]
    for _ in range(int(rng.integers(3, 14))):
        u = rng.random()
        if u < 0.3:
            pool.append(unary[int(rng.integers(len(unary)))](pool[int(rng.integers(len(pool)))]))
        elif u < 0.7:
            x, y = pool[int(rng.integers(len(pool)))], pool[int(rng.integers(len(pool)))]
            try:
                pool.append(binary[int(rng.integers(len(binary)))](x, y))
            except RuntimeError:      # shapes that do not broadcast
                pass
        else:
            x = pool[int(rng.integers(len(pool)))]
            if len(x.shape) == 2 and x.op not in G.VIEW_OPS:
                axes = [[1], [0], []][int(rng.integers(3))]
                red = G.max_ if rng.random() < 0.6 else G.sum_
                pool.append(red(x, axes, bool(rng.integers(2))))
    return [n for n in pool[-3:] if not n.is_realized]


def test_random_graphs_with_extension_ops_on_the_emulator():
    rng = np.random.default_rng(4321)
    ran = 0
    for _ in range(25):
        roots = _random_graph(rng)
        if roots:
            _emulated(roots, 5 * REDUCE_TOL)
            ran += 1
    assert ran >= 15


@pytest.mark.gpu
def test_random_graphs_with_extension_ops_on_gpu(device):
    rng = np.random.default_rng(987)
    for _ in range(40):
        roots = _random_graph(rng)
        if not roots:
            continue
        ref, _ = O.port_run(roots)
        for r, w in zip(roots, ref):
            g = device.numpy(r)
            assert g.shape == w.shape
            assert rel(g, w) <= 5 * REDUCE_TOL
