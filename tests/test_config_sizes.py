"""Parity at the sizes the baseline configurations state, against the CPU oracle: the unmodified reference engine
(oracle/_ref, whose matmul is OpenBLAS' cblas_sgemm through the shim) for graphs with matmuls, the C restatement
(bit-identical to it on pointwise + sum graphs; tests/test_oracle.py pins that) for the rest.

Where the oracle would need minutes for the whole tensor, the comparison uses what the path's structure offers:
rows of softmax / layernorm are independent, so the oracle runs on the sampled rows alone and must reproduce those
rows of the full-size GPU result; column sums over all rows are compared on a 2048-row sub-problem realized on both
sides, and at full size through additivity over row blocks; for the largest matmul the oracle computes a block of rows.
Tolerances: fp32 pointwise 1e-6, fp32 reductions and FFMA matmul 1e-5, bf16 tensor-core matmul 2e-2, all as
max|gpu - cpu| <= tol * max|cpu| per tensor.
"""
import math

import numpy as np
import pytest

from ormi_b200 import graph as G
from ormi_b200 import workloads as W
from oracle import oracle as O

pytestmark = pytest.mark.gpu

REDUCE_TOL, BF16_TOL = 1e-5, 2e-2


def rel(a, b):
    return float(np.abs(a - b).max() / max(1e-30, np.abs(b).max()))


def oracle_matmul(a, b):
    """a @ b on the reference CPU backend (falls back to the restatement's plain loops when the library is absent)."""
    root = G.matmul(G.leaf(a), G.leaf(b))
    if O.ref_available():
        (c,), _ = O.ref_run([(root, "value")])
    else:
        (c,), _ = O.port_run([root])
    return c


def test_config0_fused_rowsum_4096x4096(device):
    """configs[0]: a, b, c [4096, 4096] ~ N(0, 1) from seeds 0, 1, 2; y = sum(relu(a*b + c) * exp(-|a|), axis=1)."""
    a, b, c = (W.normal(i, (4096, 4096)) for i in range(3))
    got = device.numpy(W.fused_rowsum(G.leaf(a), G.leaf(b), G.leaf(c)))
    (want,), _ = O.port_run([W.fused_rowsum(G.leaf(a), G.leaf(b), G.leaf(c))])
    assert got.shape == (4096,) and rel(got, want) <= REDUCE_TOL


def _softmax_graph(x, gy):
    y = W.softmax(x)
    y.grad = gy
    G.compute_gradients(y)
    return [y, x.grad]


def _layernorm_graph(x, gy, g, b):
    y = W.layernorm(x, g, b)
    y.grad = gy
    G.compute_gradients(y)
    return [y, x.grad, g.grad, b.grad]


def test_config1_softmax_layernorm_16384x4096(device):
    """configs[1] at full size: x [16384, 4096] ~ N(0, 2), g ~ U(0.5, 1.5), b ~ N(0, 0.1), upstream grad ~ N(0, 1)."""
    R, C = 16384, 4096
    xs, gys = W.normal(0, (R, C), math.sqrt(2.0)), W.normal(1, (R, C))
    gs, bs = W.uniform(2, (C,), 0.5, 1.5), W.normal(3, (C,), 0.1)
    rows = np.sort(np.random.default_rng(0).choice(R, 256, replace=False))

    sm = [device.numpy(n) for n in _softmax_graph(G.leaf(xs, True), G.leaf(gys))]
    want, _ = O.port_run(_softmax_graph(G.leaf(xs[rows], True), G.leaf(gys[rows])))
    assert rel(sm[0][rows], want[0]) <= REDUCE_TOL and rel(sm[1][rows], want[1]) <= REDUCE_TOL
    del sm

    ln = [device.numpy(n) for n in _layernorm_graph(G.leaf(xs, True), G.leaf(gys), G.leaf(gs, True), G.leaf(bs, True))]
    want, _ = O.port_run(_layernorm_graph(G.leaf(xs[rows], True), G.leaf(gys[rows]), G.leaf(gs, True), G.leaf(bs, True)))
    assert rel(ln[0][rows], want[0]) <= REDUCE_TOL and rel(ln[1][rows], want[1]) <= 2 * REDUCE_TOL
    # dg, db: a 2048-row sub-problem on both sides ...
    blocks = []
    for k in range(R // 2048):
        sub = slice(2048 * k, 2048 * (k + 1))
        outs = [device.numpy(n) for n in _layernorm_graph(G.leaf(xs[sub], True), G.leaf(gys[sub]), G.leaf(gs, True), G.leaf(bs, True))]
        blocks.append(outs[2:])
        if k == 3:
            want, _ = O.port_run(_layernorm_graph(G.leaf(xs[sub], True), G.leaf(gys[sub]), G.leaf(gs, True), G.leaf(bs, True)))
            for got, w in zip(outs, want):
                assert rel(got, w) <= 2 * REDUCE_TOL
    # ... and at full size through additivity: the column sums over 16384 rows are the sum of the eight blocks' sums
    for i in (0, 1):
        total = np.sum([blk[i].astype(np.float64) for blk in blocks], axis=0)
        assert rel(ln[2 + i], total) <= REDUCE_TOL


SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (8192, 1024, 8192)]


@pytest.mark.parametrize("mode,tol", [("fp32", REDUCE_TOL), ("bf16", BF16_TOL)])
@pytest.mark.parametrize("mnk", SHAPES)
def test_config2_matmul_sweep(mnk, mode, tol):
    """configs[2]: A, B ~ N(0, 1/sqrt(K)); fp32 on the FFMA path and bf16 on the tcgen05 path, against the oracle's
    matmul (cblas_sgemm of the reference CPU backend).  The GPU computes all of C; above 2^35 multiply-adds the oracle
    computes a block of 256 rows of it."""
    from ormi_b200.runtime import Device
    M, N, K = mnk
    a = W.normal(0, (M, K), 1 / math.sqrt(K))
    b = W.normal(1, (K, N), 1 / math.sqrt(K))
    dev = Device(0)
    try:
        dev.set_option("matmul", mode)
        got = dev.numpy(G.matmul(G.leaf(a), G.leaf(b)))
    finally:
        dev.close()
    rows = slice(0, M) if M * N * K <= 2 ** 35 else slice(M // 2 - 128, M // 2 + 128)
    want = oracle_matmul(a[rows], b)
    assert got.shape == (M, N) and rel(got[rows], want) <= tol


LR = 0.05


def _mlp_problem(B, D, H):
    return (W.normal(0, (B, D)), W.normal(1, (B, D)), W.kaiming_uniform(2, D, (D, H)), np.zeros(H, np.float32),
            W.kaiming_uniform(3, H, (H, D)), np.zeros(D, np.float32))


def _mlp_step(B, D, H):
    """loss, the four gradients, the four updated parameters."""
    xh, th, *ph = _mlp_problem(B, D, H)
    x, t = G.leaf(xh), G.leaf(th)
    params = [G.leaf(p, True) for p in ph]
    loss = W.mlp_loss(x, params[0], params[1], params[2], params[3], t)
    G.compute_gradients(loss)
    return [loss] + [p.grad for p in params] + [W.sgd_update(p, LR) for p in params]


def _mlp_step_oracle(B, D, H):
    """The same nine tensors from the reference engine: its own autograd builds the backward graph, its CPU backend
    realizes it; the SGD update p - lr * g is two fp32 operations and is applied with numpy."""
    if not O.ref_available():
        return O.port_run(_mlp_step(B, D, H))[0]
    xh, th, *ph = _mlp_problem(B, D, H)
    params = [G.leaf(p, True) for p in ph]
    loss = W.mlp_loss(G.leaf(xh), params[0], params[1], params[2], params[3], G.leaf(th))
    outs, _ = O.ref_run([(loss, "value")] + [(p, "grad") for p in params], backward_root=loss)
    grads = [g.reshape(p.shape) for g, p in zip(outs[1:], ph)]
    return [outs[0]] + grads + [p - np.float32(LR) * g for p, g in zip(ph, grads)]


def test_config3_mlp_step_fp32_full_batch(device):
    """configs[3]: one full training step at B = 8192, 1024 -> 4096 -> 1024, fp32 FFMA matmuls, against the oracle."""
    want = _mlp_step_oracle(8192, 1024, 4096)
    roots = _mlp_step(8192, 1024, 4096)
    device.realize(roots)
    got = [device.numpy(r) for r in roots]
    for g, w in zip(got[1:], want[1:]):
        assert g.shape == w.shape and rel(g, w) <= 3 * REDUCE_TOL
    # The loss is a sum of 8.4 million positive terms.  The oracle adds them one after the other in fp32: once the
    # running sum has passed 2^24 every term of about 3 is rounded to a multiple of 2, and the total ends up about one
    # per cent low.  The GPU adds them as a tree.  So the scalar is judged against an fp64 evaluation of the same
    # forward pass, with the oracle's value required to lie within its own error of it.
    xh, th, w1, b1, w2, b2 = (a.astype(np.float64) for a in _mlp_problem(8192, 1024, 4096))
    u = xh @ w1 + b1
    z = 0.79788456 * (u + 0.044715 * u ** 3)
    h = 0.5 * u * (1.0 + (1.0 - 2.0 / (np.exp(2.0 * z) + 1.0)))
    loss64 = float(np.mean((h @ w2 + b2 - th) ** 2))
    assert abs(float(got[0]) - loss64) <= 3 * REDUCE_TOL * loss64
    assert abs(float(want[0]) - loss64) <= 3e-2 * loss64


def test_config4_mlp_step_bf16_widths_at_1024_rows():
    """configs[4] widths 2048 -> 8192 -> 2048 with bf16 matmuls, fused epilogues and bf16 twins, at 1024 rows (one
    eighth of a rank's share at 8 GPUs), against the oracle's fp32 step."""
    from ormi_b200.runtime import Device
    want = _mlp_step_oracle(1024, 2048, 8192)
    dev = Device(0)
    try:
        dev.set_option("matmul", "bf16")
        roots = _mlp_step(1024, 2048, 8192)
        dev.realize(roots)
        got = [dev.numpy(r) for r in roots]
        assert dev.counter("gemm_launches") == 5 and dev.counter("cvt_launches") <= 3     # x, W1, W2 once each; h, g_out, du never
    finally:
        dev.close()
    for g, w in zip(got, want):
        assert g.shape == w.shape and rel(g, w) <= BF16_TOL
