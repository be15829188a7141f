"""Parity of the B200 backend with the CPU oracle, through the C ABI (ormi_b200.runtime.Device).

Tolerances (north star of the build): fp32 pointwise <= 1e-6, fp32 reductions and FFMA matmul <= 1e-5,
bf16 tensor-core matmul <= 2e-2 — all as max|gpu - cpu| / max|cpu| per tensor, because the oracle sums
serially in fp32 and an element-wise relative error is unbounded wherever a sum cancels.
"""
import ctypes
import os
import math

import numpy as np
import pytest

import make_golden
from ormi_b200 import graph as G
from ormi_b200 import workloads as W
from ormi_b200 import runtime as RT
from oracle import oracle as O

pytestmark = pytest.mark.gpu

POINTWISE_TOL, REDUCE_TOL, BF16_TOL = 1e-6, 1e-5, 2e-2


def rel(a, b):
    return float(np.abs(a - b).max() / max(1e-30, np.abs(b).max()))


def check(device, roots, tol):
    ref, _ = O.port_run(roots)
    got = [device.numpy(r) for r in roots]
    for g, r in zip(got, ref):
        assert g.shape == r.shape
        assert rel(g, r) <= tol, rel(g, r)
    return got


@pytest.mark.parametrize("name", list(make_golden.CASES))
def test_golden_cases(device, name):
    import os
    roots, _ = make_golden.CASES[name]()
    got = check(device, roots, REDUCE_TOL)
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", name + ".npz"))
    for i, g in enumerate(got):       # and against the stored outputs of the unmodified reference
        assert rel(g, want[f"out{i}"]) <= REDUCE_TOL


def test_reference_known_answers(device):
    full = lambda s, v: G.leaf(np.full(s, v, dtype=np.float32))
    cases = [
        (G.add(full([4], 2.0), full([4], 3.0)), 5.0),
        (G.mul(G.add(full([2, 2], 2.0), full([2, 2], 3.0)), full([2, 2], 4.0)), 20.0),
        (G.add(full([2, 3], 2.0), full([3], 5.0)), 7.0),
        (G.add(full([2, 2], 10.0), full([], 3.0)), 13.0),
        (G.matmul(full([2, 3], 2.0), full([3, 2], 3.0)), 18.0),
        (G.matmul(full([2, 1, 2, 3], 1.5), full([1, 2, 3, 2], 2.0)), 9.0),
        (G.sum_(full([2, 3], 2.0), [], True), 12.0),
        (G.sum_(full([2, 3, 2], 1.0), [0, 2], False), 4.0),
    ]
    device.realize([c for c, _ in cases])
    for c, want in cases:
        assert np.all(device.numpy(c) == want)
    a = G.leaf(np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32))
    b = G.leaf(np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32))
    assert device.numpy(G.matmul(a, b)).reshape(-1).tolist() == [58.0, 64.0, 139.0, 154.0]
    ct = G.matmul(G.transpose(a, [1, 0]), G.leaf(np.array([[1, 2], [3, 4]], dtype=np.float32)))
    assert device.numpy(ct).reshape(-1).tolist() == [13.0, 18.0, 17.0, 24.0, 21.0, 30.0]
    a3 = G.leaf(np.arange(1, 13, dtype=np.float32).reshape(2, 2, 3))
    b2 = G.leaf(np.arange(1, 7, dtype=np.float32).reshape(1, 3, 2))
    cb = G.matmul(a3, G.expand(b2, [2, 3, 2]))
    assert device.numpy(cb).reshape(-1).tolist() == [22.0, 28.0, 49.0, 64.0, 76.0, 100.0, 103.0, 136.0]
    x, y = G.leaf([2.0, 3.0], True), G.leaf([4.0, 5.0], True)
    z = G.add(G.mul(x, y), x)
    G.compute_gradients(z)
    assert device.numpy(x.grad).tolist() == [5.0, 6.0] and device.numpy(y.grad).tolist() == [2.0, 3.0]
    m = G.leaf([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    assert device.numpy(G.reshape(m, [3, 2])).tolist() == [[1, 2], [3, 4], [5, 6]]
    assert device.numpy(G.transpose(m, [1, 0])).tolist() == [[1, 4], [2, 5], [3, 6]]


def test_pointwise_chain_within_1e6(device):
    a, b = G.leaf(W.normal(0, (512, 1024))), G.leaf(W.uniform(1, (512, 1024), 0.5, 2.0))
    root = G.div(G.sub(G.exp(G.neg(G.mul(a, a))), G.sin(b)), G.add(G.log(b), G.const(3.0)))
    check(device, [root, G.cos(G.pow_(b, G.const(1.7)))], 2 * POINTWISE_TOL)


def test_config1_shape(device):
    a, b, c = (G.leaf(W.normal(i, (512, 4096))) for i in range(3))
    check(device, [W.fused_rowsum(a, b, c)], REDUCE_TOL)


@pytest.mark.parametrize("shape", [(512, 4096), (300, 1000), (64, 37), (33, 8192)])
def test_softmax_layernorm_forward_backward(device, shape):
    R, C = shape
    x = G.leaf(W.normal(0, (R, C), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(1, (R, C)))
    y = W.softmax(x)
    y.grad = gy
    G.compute_gradients(y)
    check(device, [y, x.grad], REDUCE_TOL)
    x = G.leaf(W.normal(0, (R, C), math.sqrt(2.0)), True)
    g, b = G.leaf(W.uniform(2, (C,), 0.5, 1.5), True), G.leaf(W.normal(3, (C,), 0.1), True)
    y = W.layernorm(x, g, b)
    y.grad = gy
    G.compute_gradients(y)
    check(device, [y, x.grad, g.grad, b.grad], 3 * REDUCE_TOL)


def test_mlp_training_step(device):
    B, D, H = 512, 128, 512
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(np.zeros(H, np.float32), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(np.zeros(D, np.float32), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    G.compute_gradients(loss)
    ups = [W.sgd_update(p, 0.1) for p in (w1, b1, w2, b2)]
    check(device, [loss] + ups + [w1.grad, w2.grad], 3 * REDUCE_TOL)


@pytest.mark.parametrize("mnk", [(128, 128, 128), (1024, 1024, 1024), (257, 130, 67), (8, 4096, 64), (2048, 64, 1500)])
def test_matmul_fp32_layouts(device, mnk):
    M, N, K = mnk
    a = W.normal(0, (M, K), 1 / math.sqrt(K))
    b = W.normal(1, (K, N), 1 / math.sqrt(K))
    want = (a.astype(np.float64) @ b.astype(np.float64))
    la, lb = G.leaf(a), G.leaf(b)
    lat, lbt = G.leaf(np.ascontiguousarray(a.T)), G.leaf(np.ascontiguousarray(b.T))
    for root in (G.matmul(la, lb), G.matmul(G.transpose(lat, [1, 0]), lb), G.matmul(la, G.transpose(lbt, [1, 0])),
                 G.matmul(G.transpose(lat, [1, 0]), G.transpose(lbt, [1, 0]))):
        assert rel(device.numpy(root), want) <= REDUCE_TOL


def test_full_size_row_kernels_against_fp64_on_sampled_rows(device):
    """configs[1] at full size [16384, 4096]: the oracle would need minutes, so rows are sampled and compared with
    an fp64 evaluation of the same formulas, plus the invariants that hold for every row."""
    R, C = 16384, 4096
    xs = W.normal(0, (R, C), math.sqrt(2.0))
    gys = W.normal(1, (R, C))
    x, gy = G.leaf(xs, True), G.leaf(gys)
    y = W.softmax(x)
    y.grad = gy
    G.compute_gradients(y)
    yv, dxv = device.numpy(y), device.numpy(x.grad)
    assert np.abs(yv.sum(axis=1, dtype=np.float64) - 1.0).max() < 1e-5
    assert np.abs(dxv.sum(axis=1, dtype=np.float64)).max() < 1e-4          # softmax gradients sum to zero per row
    rows = np.random.default_rng(0).choice(R, 64, replace=False)
    x64, g64 = xs[rows].astype(np.float64), gys[rows].astype(np.float64)
    e = np.exp(x64); s = e.sum(1, keepdims=True); y64 = e / s
    dx64 = y64 * (g64 - (g64 * y64).sum(1, keepdims=True))
    assert rel(yv[rows], y64) <= REDUCE_TOL and rel(dxv[rows], dx64) <= REDUCE_TOL

    g = G.leaf(W.uniform(2, (C,), 0.5, 1.5), True)
    b = G.leaf(W.normal(3, (C,), 0.1), True)
    x = G.leaf(xs, True)
    y = W.layernorm(x, g, b)
    y.grad = gy
    G.compute_gradients(y)
    yv, dxv, dgv, dbv = (device.numpy(n) for n in (y, x.grad, g.grad, b.grad))
    mu = x64.mean(1, keepdims=True); var = ((x64 - mu) ** 2).mean(1, keepdims=True); xh = (x64 - mu) / np.sqrt(var + 1e-5)
    g64v, b64v = g.data.host.astype(np.float64), b.data.host.astype(np.float64)
    assert rel(yv[rows], xh * g64v + b64v) <= REDUCE_TOL
    dxh = g64 * g64v
    dx64 = (dxh - dxh.mean(1, keepdims=True) - xh * (dxh * xh).mean(1, keepdims=True)) / np.sqrt(var + 1e-5)
    assert rel(dxv[rows], dx64) <= 2 * REDUCE_TOL
    assert rel(dbv, gys.sum(0, dtype=np.float64)) <= REDUCE_TOL               # column sums over all 16384 rows
    xh_all = (xs - xs.mean(1, keepdims=True, dtype=np.float64)) / np.sqrt(xs.var(1, keepdims=True, dtype=np.float64) + 1e-5)
    assert rel(dgv, (gys * xh_all).sum(0, dtype=np.float64)) <= REDUCE_TOL


def test_results_are_deterministic(device):
    outs = []
    for _ in range(2):
        x = G.leaf(W.normal(0, (777, 1536)), True)
        g, b = G.leaf(W.uniform(2, (1536,), 0.5, 1.5), True), G.leaf(W.normal(3, (1536,), 0.1), True)
        y = W.layernorm(x, g, b)
        G.compute_gradients(G.sum_(G.mul(y, y), [], False))
        outs.append([device.numpy(n) for n in (y, x.grad, g.grad, b.grad)])
    for a, b_ in zip(*outs):
        assert np.array_equal(a, b_)        # no atomics anywhere: bit-identical from run to run


def test_allocator_contract(device):
    """ormi-core/csrc/tests/core/test_allocator.cpp:12-47: same size gives the same block back, another size does not."""
    p1, p2 = device.alloc(1024), device.alloc(2048)
    assert p1 and p2 and p1 != p2
    device.free(p1, 1024)
    p3 = device.alloc(1024)
    assert p3 == p1
    p4 = device.alloc(2048)
    assert p4 != p3
    for p, n in ((p3, 1024), (p2, 2048), (p4, 2048)):
        device.free(p, n)
    host = np.arange(100, dtype=np.float32)
    buf = device.upload(host)
    assert np.array_equal(device.download(buf), host)


def test_plan_and_kernel_caches(device):
    def step():
        x = G.leaf(W.normal(0, (64, 256)), True)
        y = W.softmax(x)
        G.compute_gradients(G.sum_(G.mul(y, y), [], False))
        device.realize([y, x.grad])
    step()
    compiled, hits = device.counter("kernels_compiled"), device.counter("plan_cache_hits")
    step()
    assert device.counter("kernels_compiled") == compiled and device.counter("plan_cache_hits") == hits + 1


def test_views_and_edge_shapes(device):
    a = G.leaf(W.normal(0, (6, 10)))
    b = G.leaf(W.normal(1, (10, 6)))
    roots = [G.mul(G.transpose(a, [1, 0]), b),
             G.add(G.reshape(G.exp(a), [3, 20]), G.leaf(W.normal(2, (20,)))),
             G.transpose(G.add(a, a), [1, 0]),
             G.add(G.expand(G.leaf(W.normal(3, (6, 1))), [6, 10]), a),
             G.mul(G.transpose(G.exp(a), [1, 0]), b)]
    check(device, roots, 2 * POINTWISE_TOL)
    c = G.leaf(W.normal(0, (6, 5, 8)))
    e = G.exp(c)
    check(device, [G.sum_(e, [], False), G.sum_(e, [2], True), G.sum_(e, [0, 1], False), G.sum_(e, [1], False),
                   G.sum_(c, [0, 2], True)], REDUCE_TOL)
    w = G.leaf(W.normal(0, (2, 40000)))
    check(device, [G.sum_(G.mul(w, w), [1], False)], REDUCE_TOL)
    for n in (1, 3, 127, 1025):
        p, q = G.leaf(W.normal(0, (n,))), G.leaf(W.normal(1, (n,)))
        check(device, [G.div(G.sub(p, q), G.add(G.mul(q, q), G.const(1.0))), G.sum_(G.mul(p, q), [], False)], REDUCE_TOL)


def test_raw_buffer_sum_and_matmul_entry_points(device):
    """ormi_b200_sum / ormi_b200_matmul: the C counterparts of cuda::sum and cuda::matmul on raw buffers."""
    from ormi_b200._lib import lib, check as ok
    a = W.normal(0, (2, 3, 4))
    src = device.upload(a)
    out = device.buffer([3])
    shape = (ctypes.c_int32 * 3)(2, 3, 4); strides = (ctypes.c_int32 * 3)(12, 4, 1); axes = (ctypes.c_int32 * 2)(0, 2)
    ok(lib.ormi_b200_sum(device.handle, ctypes.c_void_p(src.dev_ptr), 3, shape, strides, axes, 2, ctypes.c_void_p(out.dev_ptr)))
    assert rel(device.download(out), a.sum(axis=(0, 2))) <= REDUCE_TOL
    A, B = W.normal(1, (5, 7)), W.normal(2, (7, 3))
    da, db, dc = device.upload(A), device.upload(B), device.buffer([5, 3])
    sa, sta = (ctypes.c_int32 * 2)(5, 7), (ctypes.c_int32 * 2)(7, 1)
    sb, stb = (ctypes.c_int32 * 2)(7, 3), (ctypes.c_int32 * 2)(3, 1)
    so = (ctypes.c_int32 * 2)(5, 3)
    ok(lib.ormi_b200_matmul(device.handle, ctypes.c_void_p(da.dev_ptr), 2, sa, sta, ctypes.c_void_p(db.dev_ptr), 2, sb, stb,
                            ctypes.c_void_p(dc.dev_ptr), 2, so))
    assert rel(device.download(dc), A @ B) <= REDUCE_TOL


@pytest.mark.parametrize("mnk", [(256, 256, 256), (1024, 1024, 1024), (300, 520, 200), (128, 2048, 4096), (4096, 256, 512)])
def test_matmul_bf16_tensor_core(mnk):
    """Opt-in tcgen05 path: bf16 operands, fp32 accumulation in tensor memory; tolerance 2e-2."""
    from ormi_b200.runtime import Device
    M, N, K = mnk
    dev = Device(0)
    try:
        dev.set_option("matmul", "bf16")
        a = W.normal(0, (M, K), 1 / math.sqrt(K))
        b = W.normal(1, (K, N), 1 / math.sqrt(K))
        want = a.astype(np.float64) @ b.astype(np.float64)
        la, lb = G.leaf(a), G.leaf(b)
        lat, lbt = G.leaf(np.ascontiguousarray(a.T)), G.leaf(np.ascontiguousarray(b.T))
        for root in (G.matmul(la, lb), G.matmul(G.transpose(lat, [1, 0]), lb), G.matmul(la, G.transpose(lbt, [1, 0])),
                     G.matmul(G.transpose(lat, [1, 0]), G.transpose(lbt, [1, 0]))):
            got = dev.numpy(root)
            assert rel(got, want) <= BF16_TOL, rel(got, want)
        # exact check: operands that are exactly representable in bf16 give the fp32 result of the same products
        ai = np.random.default_rng(0).integers(-4, 5, size=(M, K)).astype(np.float32)
        bi = np.random.default_rng(1).integers(-4, 5, size=(K, N)).astype(np.float32)
        got = dev.numpy(G.matmul(G.leaf(ai), G.leaf(bi)))
        assert np.array_equal(got, ai @ bi)
        assert dev.counter("gemm_launches") >= 5
    finally:
        dev.close()


def test_mlp_training_step_bf16_matmuls():
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        dev.set_option("matmul", "bf16")
        B, D, H = 1024, 256, 1024
        x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
        w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(np.zeros(H, np.float32), True)
        w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(np.zeros(D, np.float32), True)
        loss = W.mlp_loss(x, w1, b1, w2, b2, t)
        G.compute_gradients(loss)
        roots = [loss, w1.grad, b1.grad, w2.grad, b2.grad]
        ref, _ = O.port_run(roots)
        for r, w in zip(roots, ref):
            assert rel(dev.numpy(r), w) <= BF16_TOL
    finally:
        dev.close()


def test_mlp_trainer_matches_oracle_over_steps(device):
    """The repeated-step host loop (ormi_b200.train_step.MLPTrainer): three SGD steps against the oracle."""
    from ormi_b200.train_step import MLPTrainer
    B, D, H, lr = 256, 64, 256, 0.1
    x, t = W.normal(0, (B, D)), W.normal(1, (B, D))
    w1, b1 = W.kaiming_uniform(2, D, (D, H)), np.zeros(H, np.float32)
    w2, b2 = W.kaiming_uniform(3, H, (H, D)), np.zeros(D, np.float32)
    tr = MLPTrainer(device, x, t, w1, b1, w2, b2, lr=lr)
    params = [w1, b1, w2, b2]
    for _ in range(3):
        tr.step()
        leaves = [G.leaf(p, True) for p in params]
        loss = W.mlp_loss(G.leaf(x), leaves[0], leaves[1], leaves[2], leaves[3], G.leaf(t))
        G.compute_gradients(loss)
        outs, _ = O.port_run([loss] + [W.sgd_update(l, lr) for l in leaves])
        assert abs(tr.loss() - float(outs[0])) <= 3 * REDUCE_TOL * abs(float(outs[0]))
        params = [o for o in outs[1:]]
    for name, want in zip(tr.names, params):
        assert rel(tr.parameter(name).reshape(want.shape), want) <= 3 * REDUCE_TOL


@pytest.mark.parametrize("mode,tol", [("tf32", 2e-3), ("3xtf32", 3 * REDUCE_TOL)])
@pytest.mark.parametrize("mnk", [(512, 512, 512), (300, 520, 200), (1024, 256, 1024)])
def test_matmul_tf32_modes(mode, tol, mnk):
    """Opt-in fp32 matmul on the tensor cores: tf32 operands (about 1e-3), or the three-product 3xTF32 split (fp32-grade:
    the dropped lo*lo term is 2^-22 per product, but the tensor-core accumulator does not round to nearest, so the error
    grows with K — measured 3e-6 at K = 256, 1.4e-5 at K = 1024, 5e-5 at K = 4096 — which is why FFMA stays the default)."""
    from ormi_b200.runtime import Device
    M, N, K = mnk
    dev = Device(0)
    try:
        dev.set_option("matmul", mode)
        a = W.normal(0, (M, K), 1 / math.sqrt(K))
        b = W.normal(1, (K, N), 1 / math.sqrt(K))
        want = a.astype(np.float64) @ b.astype(np.float64)
        la, lbt = G.leaf(a), G.leaf(np.ascontiguousarray(b.T))
        for root in (G.matmul(la, G.leaf(b)), G.matmul(la, G.transpose(lbt, [1, 0]))):
            assert rel(dev.numpy(root), want) <= tol, rel(dev.numpy(root), want)
    finally:
        dev.close()


def test_wide_hidden_layer_schedule(device):
    """Rows of 8192 columns (1024 threads per row, staged operands) and a dynamic shared-memory size of exactly 48 KB:
    the shapes of one rank's share of the wide MLP at reduced batch."""
    B, D, H = 256, 2048, 8192
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(W.normal(4, (H,), 0.1), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(W.normal(5, (D,), 0.1), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    G.compute_gradients(loss)
    (want,), _ = O.port_run([loss])          # before the device realizes (and so cuts) parts of this graph
    check(device, [w1.grad, b1.grad, w2.grad, b2.grad], 3 * REDUCE_TOL)
    # the loss is a sum of 524288 positive terms: the oracle adds them serially in fp32 and is itself 2e-4 away from the
    # fp64 value, the tree sum on the GPU is not — so the scalar is compared with a bound that covers the oracle's error
    assert abs(float(device.numpy(loss)) - float(want)) <= 1e-3 * abs(float(want))


def test_scratch_buffers_are_reused_inside_one_realize():
    """Three column sums in a chain need three 1 MiB partial buffers with disjoint lifetimes: the executor takes each
    from the pool at its first step and returns it after its last, so a fresh context allocates that size once."""
    if os.environ.get("ORMI_B200_POOL_CANARY"):
        pytest.skip("counts bytes taken from the driver: guard zones add 256 to every block")
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        a, b, c = (dev.leaf(W.normal(i, (512, 1024))) for i in range(3))
        y1 = G.sum_(a, [0], False)
        y2 = G.sum_(G.mul(b, y1), [0], False)
        y3 = G.sum_(G.mul(c, y2), [0], False)
        plan = RT.plan([y3], host_pointers=False)
        temps = [bf["bytes"] for bf in plan["buffers"] if bf["kind"] == "temp"]
        assert temps == [1 << 20] * 3
        before = dev.counter("bytes_allocated")
        dev.realize([y3])
        grown = dev.counter("bytes_allocated") - before
        outs = 3 * 4096                                   # y1, y2, y3 are materialized and handed back
        assert grown == (1 << 20) + outs, grown
        (want,), _ = O.port_run([G.sum_(G.mul(G.leaf(W.normal(2, (512, 1024))), G.sum_(G.mul(G.leaf(W.normal(1, (512, 1024))),
                                 G.sum_(G.leaf(W.normal(0, (512, 1024))), [0], False)), [0], False)), [0], False)])
        assert rel(dev.numpy(y3), want) <= 3 * REDUCE_TOL
    finally:
        dev.close()


def test_limits_fail_loudly_on_the_device_path(device):
    a = G.leaf(np.zeros((0, 5), np.float32))
    with pytest.raises(RuntimeError, match="empty or negative dimension"):
        device.realize([G.add(a, a)])
    # the context is still usable afterwards
    b = G.leaf(np.full((4,), 2.0, np.float32))
    np.testing.assert_array_equal(device.numpy(G.mul(b, b)), np.full((4,), 4.0, np.float32))


@pytest.mark.parametrize("shape", [(1, 1), (1, 7), (7, 1), (3, 33), (33, 3), (2, 1025), (129, 5), (5, 12289)])
def test_ragged_shapes(device, shape):
    R, C = shape
    x = G.leaf(W.normal(0, (R, C)), True)
    g, b = G.leaf(W.uniform(1, (C,), 0.5, 1.5), True), G.leaf(W.normal(2, (C,), 0.1), True)
    y = W.layernorm(x, g, b)
    y.grad = G.leaf(W.normal(3, (R, C)))
    G.compute_gradients(y)
    check(device, [y, x.grad, g.grad, b.grad, W.softmax(x), G.sum_(x, [0], False), G.sum_(x, [1], True), G.sum_(x, [], False)], 5 * REDUCE_TOL)


def test_compiled_kernels_are_cached_on_disk(tmp_path, monkeypatch):
    """A second context (a new process would be the same) finds the cubins of the first on disk and does not call NVRTC."""
    import os
    from ormi_b200.runtime import Device
    monkeypatch.setenv("ORMI_B200_CACHE_DIR", str(tmp_path / "cubins"))
    x_h = W.normal(0, (48, 160), math.sqrt(2.0))

    def run():
        dev = Device(0)
        try:
            x = dev.leaf(x_h, requires_grad=True)
            y = W.softmax(x)
            y.grad = dev.leaf(W.normal(1, (48, 160)))
            G.compute_gradients(y)
            out = [dev.numpy(y).copy(), dev.numpy(x.grad).copy()]
            return out, dev.counter("nvrtc_compiles"), dev.counter("cubin_disk_hits")
        finally:
            dev.close()

    first, compiled1, hits1 = run()
    files = os.listdir(tmp_path / "cubins")
    assert compiled1 >= 1 and hits1 == 0 and len(files) == compiled1 and all(f.endswith(".cubin") for f in files)
    second, compiled2, hits2 = run()
    assert compiled2 == 0 and hits2 == compiled1
    for a, b in zip(first, second):
        np.testing.assert_array_equal(a, b)
    monkeypatch.setenv("ORMI_B200_CACHE_DIR", "off")
    _, compiled3, hits3 = run()
    assert compiled3 == compiled1 and hits3 == 0


def test_bounded_wait_gives_up_and_reports(device):
    """A device-side wait that nothing completes runs out after its limit: the kernel returns, the next sync reports it
    once, and the context keeps working.  (The same routine guards every mbarrier wait of the tensor-core GEMM.)"""
    import time
    from ormi_b200._lib import lib, check
    check(lib.ormi_b200_selftest_wait_timeout(device.handle, 50))
    t0 = time.perf_counter()
    with pytest.raises(RuntimeError, match="bounded device-side wait ran out \\(code 9"):
        device.sync()
    assert 0.03 <= time.perf_counter() - t0 <= 1.0
    device.sync()                                  # reported once; the word is clear again
    a = G.leaf(W.normal(0, (256, 512)))
    check_ = G.matmul(a, G.transpose(a, [1, 0]))
    (want,), _ = O.port_run([check_])
    assert rel(device.numpy(check_), want) <= REDUCE_TOL
    assert lib.ormi_b200_selftest_wait_timeout(device.handle, 5000) != 0      # limits outside 1..1000 ms are refused


def test_unaligned_caller_pointer_gets_scalar_kernels():
    """A device pointer that is not on a 16-byte boundary (a caller's own sub-buffer): the plan is generated without
    128-bit accesses or bulk copies and gives the same result; the aligned call right after uses the vector plan again."""
    from ormi_b200._lib import lib, check as ok
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        R, C = 96, 512
        host = W.normal(0, (R * C + 1,))
        base = dev.upload(host)
        out = dev.buffer([R])
        shape, strides, axes = (ctypes.c_int32 * 2)(R, C), (ctypes.c_int32 * 2)(C, 1), (ctypes.c_int32 * 1)(1)
        compiled = dev.counter("kernels_compiled")
        ok(lib.ormi_b200_sum(dev.handle, ctypes.c_void_p(base.dev_ptr + 4), 2, shape, strides, axes, 1, ctypes.c_void_p(out.dev_ptr)))
        want = host[1:].reshape(R, C).astype(np.float64).sum(axis=1)
        assert rel(dev.download(out), want) <= REDUCE_TOL
        ok(lib.ormi_b200_sum(dev.handle, ctypes.c_void_p(base.dev_ptr), 2, shape, strides, axes, 1, ctypes.c_void_p(out.dev_ptr)))
        assert rel(dev.download(out), host[:-1].reshape(R, C).astype(np.float64).sum(axis=1)) <= REDUCE_TOL
        assert dev.counter("kernels_compiled") == compiled + 2          # two different plans: scalar and vector
    finally:
        dev.close()


def test_pool_byte_cap_walks_the_out_of_memory_path():
    """"pool_limit_bytes": an allocation that would take the pool past the cap first gives the cached blocks back and
    then fails with the driver's out-of-memory text; the context keeps working; lifting the cap lifts the failure."""
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        dev.set_option("pool_limit_bytes", str(8 << 20))
        a = dev.alloc(3 << 20)
        b = dev.alloc(3 << 20)
        dev.free(b, 3 << 20)                                   # cached by the pool: still counts until it is trimmed
        trims = dev.counter("pool_trims")
        c = dev.alloc(4 << 20)                                 # 3 + 3 (cached) + 4 > 8: trim, then 3 + 4 fits
        assert dev.counter("pool_trims") == trims + 1
        with pytest.raises(RuntimeError, match="out of memory"):
            dev.alloc(2 << 20)                                 # 3 + 4 + 2 > 8 even after a trim
        x = G.leaf(np.full((16,), 3.0, np.float32))
        with pytest.raises(RuntimeError, match="out of memory"):
            dev.realize([G.mul(dev.leaf(W.normal(0, (1 << 19,))), dev.const(2.0))])
        dev.set_option("pool_limit_bytes", "0")
        np.testing.assert_array_equal(dev.numpy(G.mul(x, x)), np.full((16,), 9.0, np.float32))
        dev.free(a, 3 << 20)
        dev.free(c, 4 << 20)
    finally:
        dev.close()


def test_intermediates_free_reuses_blocks_inside_the_call():
    """"intermediates=free": a materialized node the caller does not hold is scratch of the realize call — its block is
    back in the pool for a later step of the same call — and does not come back realized.  Values are unchanged."""
    if os.environ.get("ORMI_B200_POOL_CANARY"):
        pytest.skip("counts bytes taken from the driver: guard zones add 256 to every block")
    from ormi_b200.runtime import Device
    a_h, b_h = W.normal(0, (512, 512), 0.05), W.normal(1, (512, 512), 0.05)
    got = {}
    for mode in ("keep", "free"):
        dev = Device(0)
        try:
            dev.set_option("intermediates", mode)
            a, b = dev.leaf(a_h), dev.leaf(b_h)
            p1 = G.matmul(a, b)
            e1 = G.exp(p1)
            p2 = G.matmul(e1, b)
            root = G.exp(p2)
            before = dev.counter("bytes_allocated")
            dev.realize([root])
            got[mode] = (dev.numpy(root), dev.counter("bytes_allocated") - before, [n.is_realized for n in (p1, e1, p2)])
        finally:
            dev.close()
    np.testing.assert_array_equal(got["keep"][0], got["free"][0])
    assert got["keep"][2] == [True, True, True] and got["free"][2] == [False, False, False]
    assert got["keep"][1] == 4 << 20 and got["free"][1] == 2 << 20      # the block of p1 serves p2, that of e1 the root


def test_pool_canary_reports_a_write_past_the_end_of_a_block():
    """"pool_canary": every block carries a guard zone that is read back when the block returns.  Odd-shaped graphs leave
    the zones alone (the generated kernels' bounds predicates hold); a write past the end of a block — made here through
    the ABI, inside the block's own allocation, so nothing faults — is reported by the call that returns the block."""
    import gc
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        dev.set_option("pool_canary", "on")
        for shape in ((5, 33), (7, 1001), (3, 4097), (130, 250)):
            x = dev.leaf(W.normal(0, shape), True)
            g, b = dev.leaf(W.normal(1, shape[-1:]), True), dev.leaf(W.normal(2, shape[-1:]), True)
            y = W.layernorm(x, g, b)
            y.grad = dev.leaf(W.normal(3, shape))
            G.compute_gradients(y)
            s = G.sum_(G.mul(x, x), [0], False)
            m = G.matmul(G.transpose(x, [1, 0]), y)
            dev.realize([y, x.grad, g.grad, b.grad, s, m])
            ref = W.normal(0, shape).astype(np.float64)
            np.testing.assert_allclose(dev.numpy(s), (ref * ref).sum(0), rtol=1e-5)
            del x, g, b, y, s, m
            gc.collect()
        dev.sync()
        assert dev.counter("canary_hits") == 0
        p = dev.alloc(1000)
        check_bytes = np.zeros(2, np.float32)
        dev.h2d(p + 1000, check_bytes)                          # 8 bytes past the end: inside the guard zone
        with pytest.raises(RuntimeError, match="guard zone behind a 1000-byte block"):
            dev.free(p, 1000)
        assert dev.counter("canary_hits") == 1
        q = dev.alloc(1000)                                     # the block is back in the pool and usable
        dev.free(q, 1000)
    finally:
        dev.close()


def test_captured_step_replays_with_new_input_contents():
    """Step capture: a softmax + layernorm forward/backward step and a matmul are recorded once and replayed with one call;
    the replays read the input buffers at their addresses (new contents give new results), rewrite the results in place,
    and keep every block they touch until the step is destroyed."""
    if os.environ.get("ORMI_B200_POOL_CANARY"):
        pytest.skip("a capture is refused while guard zones are on: their checks wait for the device")
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        R, C = 96, 520

        def graph(xn, gyn, gn, bn, an, wn):
            y = W.layernorm(xn, gn, bn)
            y.grad = gyn
            G.compute_gradients(y)
            return [y, xn.grad, gn.grad, bn.grad, G.matmul(an, wn)]

        def inputs(seed):
            return [W.normal(seed, (R, C), 1.5), W.normal(seed + 1, (R, C)), W.normal(seed + 2, (C,), 0.5, 1.0), W.normal(seed + 3, (C,)),
                    W.normal(seed + 4, (64, 72)), W.normal(seed + 5, (72, 40))]

        host = inputs(0)
        leaves = [dev.leaf(h, i in (0, 2, 3)) for i, h in enumerate(host)]
        roots = graph(*leaves)
        arr, order, ridx = G.flatten(roots, host_pointers=False, stop_at_realized=True)
        dev.ensure_on_device(order)
        arr, order, ridx = G.flatten(roots, host_pointers=False, stop_at_realized=True)
        template = bytes(arr)
        cridx = (ctypes.c_int * len(ridx))(*ridx)
        from ormi_b200._lib import lib, check

        def run():
            ctypes.memmove(arr, template, len(template))
            check(lib.ormi_b200_realize(dev.handle, arr, len(order), cridx, len(ridx)))
            return [(arr[i].data, arr[i].data_bytes) for i in ridx]

        for ptr, nbytes in run():                     # warm-up: kernels compiled, blocks cached by the pool
            dev.free(ptr, nbytes)
        dev.sync()
        held = dev.counter("bytes_allocated")
        with dev.capture() as step:
            outs = run()
            with pytest.raises(RuntimeError, match="not allowed while a step is being captured"):
                dev.sync()
        assert dev.counter("bytes_allocated") == held               # nothing was taken from the driver inside the capture
        launches = dev.counter("launches")

        def expect(hs):
            ref_leaves = [G.leaf(h, i in (0, 2, 3)) for i, h in enumerate(hs)]
            want, _ = O.port_run(graph(*ref_leaves))
            return want

        for seed in (0, 100, 200):
            hs = inputs(seed)
            for leaf, h in zip(leaves, hs):
                dev.h2d(leaf.data.dev_ptr, np.ascontiguousarray(h))
            step.launch()
            dev.sync()
            for (ptr, nbytes), want in zip(outs, expect(hs)):
                got = np.empty(want.size, np.float32)
                dev.d2h(got, ptr)
                assert np.abs(got - want.reshape(-1)).max() <= 2e-5 * max(1e-30, np.abs(want).max())
        assert dev.counter("launches") == launches                   # the replays went through the graph, not through realize
        assert dev.counter("graph_launches") == 3
        dev.free(*outs[0])                                           # a no-op while the step lives
        step.launch()
        dev.sync()
        step.destroy()
    finally:
        dev.close()


def test_softmax_and_layernorm_in_one_realize_call_match_the_separate_calls(device):
    """The benchmark step as one realize call (one fused kernel for both graphs + one finalize launch) against the two
    graphs realized in calls of their own: y and dx of both graphs bit for bit (the arithmetic of a row does not depend on
    what else the kernel computes), dg and db within the reduction tolerance (the blocks' row shares may differ)."""
    import bench as B
    R = 2048
    sm, ln, inputs = B.build_graphs(G, W, lambda a, rg=False: device.leaf(a, rg), rows=R)
    before = device.counter("launches")
    device.realize(sm + ln)
    assert device.counter("launches") == before + 2
    together = [device.numpy(n) for n in sm + ln]
    for n in sm + ln:
        n.data = None
    device.realize(sm)
    device.realize(ln)
    apart = [device.numpy(n) for n in sm + ln]
    for a, b in zip(together[:4], apart[:4]):
        np.testing.assert_array_equal(a, b)
    for a, b in zip(together[4:], apart[4:]):
        assert np.abs(a - b).max() <= REDUCE_TOL * np.abs(b).max()


def test_a_bf16_only_result_is_freed_once():
    """A root handed back as bf16 ONLY (ORMI_NODE_BF16) is an ordinary pool block for its owner: freeing it returns it once
    (it used to be registered as its own bf16 copy, so that freeing it freed it twice: two later allocations then shared
    one block)."""
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        dev.set_option("matmul", "bf16")
        B, D, H = 256, 128, 512
        x, w1, b1 = W.normal(0, (B, D)), W.kaiming_uniform(2, D, (D, H)), W.normal(4, (H,), 0.1)
        h = W.gelu_tanh(G.add(G.matmul(dev.leaf(x), dev.leaf(w1)), dev.leaf(b1)))
        h.bf16 = True
        dev.realize([h])
        assert h.bf16 and h.data.nbytes == B * H * 2
        ptr, nbytes = h.data.dev_ptr, h.data.nbytes
        h.data._release = None                      # freed by hand below
        dev.free(ptr, nbytes)                       # raised "returned twice" before the fix
        p1, p2 = dev.alloc(nbytes), dev.alloc(nbytes)
        assert p1 != p2
        dev.free(p1, nbytes)
        dev.free(p2, nbytes)
    finally:
        dev.close()
