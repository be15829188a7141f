"""Scheduler + code generator, checked on the CPU: every generated CUDA C kernel is compiled unchanged
against tests/cuda_emul.h, launched with its real geometry by tests/emulator.py, and compared with the
oracle.  No GPU needed; the same cases run on the B200 in tests/test_gpu_parity.py."""
import math

import numpy as np
import pytest

import emulator as E
import make_golden
from ormi_b200 import graph as G
from ormi_b200 import runtime as RT
from ormi_b200 import workloads as W
from oracle import oracle as O

POINTWISE_TOL = 1e-6     # |gpu - cpu| <= tol * max|cpu|  (fp32 pointwise)
REDUCE_TOL = 1e-5        # fp32 reductions and FFMA matmul


def compare(roots, tol):
    outs, plan = E.realize(roots)
    ref, _ = O.port_run(roots)
    for a, b in zip(outs, ref):
        assert a.shape == b.shape
        assert np.abs(a - b).max() <= tol * max(1e-30, np.abs(b).max()), np.abs(a - b).max() / np.abs(b).max()
    return plan


def kinds(plan):
    return [s["what"].split("[")[0] if s["type"] == "kernel" else "gemm" for s in plan["steps"]]


@pytest.mark.parametrize("name", list(make_golden.CASES))
def test_golden_cases_through_generated_kernels(name):
    roots, _ = make_golden.CASES[name]()
    compare(roots, REDUCE_TOL)


def test_fused_rowsum_is_one_kernel():
    a, b, c = (G.leaf(W.normal(i, (8, 4096))) for i in range(3))
    plan = compare([W.fused_rowsum(a, b, c)], REDUCE_TOL)
    assert kinds(plan) == ["rows"]
    step = plan["steps"][0]
    assert step["bytes_read"] == 3 * 8 * 4096 * 4 + 3 * 4      # a, b, c once each, plus the three rank-0 constants
    assert "V=4" in step["what"] and "stages=0,dyn" in step["what"]  # 128-bit direct loads, rows handed out dynamically


def test_softmax_forward_backward_is_one_kernel():
    x = G.leaf(W.normal(0, (24, 96), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(1, (24, 96)))
    y = W.softmax(x)
    y.grad = gy
    G.compute_gradients(y)
    plan = compare([y, x.grad], REDUCE_TOL)
    assert kinds(plan) == ["rows"]


@pytest.mark.parametrize("shape", [(12, 256), (7, 100), (3, 4096)])
def test_softmax_and_layernorm_realized_together_are_one_kernel(shape):
    """Both graphs of the benchmark step handed to ONE realize call: they share x, gy and the [rows, columns] domain, so
    the scheduler puts all six results (y, dx of the softmax; y, dx, dg, db of the layernorm) into one rows kernel that
    reads the inputs once, plus the finalize launch of the column partials."""
    R, C = shape
    x = G.leaf(W.normal(0, (R, C), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(1, (R, C)))
    y1 = W.softmax(x)
    y1.grad = gy
    G.compute_gradients(y1)
    dx1 = x.grad
    x.grad = None
    g, b = G.leaf(W.uniform(3, (C,), 0.5, 1.5), True), G.leaf(W.normal(4, (C,), 0.1), True)
    y2 = W.layernorm(x, g, b)
    y2.grad = gy
    G.compute_gradients(y2)
    plan = compare([y1, dx1, y2, x.grad, g.grad, b.grad], 2 * REDUCE_TOL)
    assert kinds(plan) == ["rows", "finalize"]
    assert "outs=FFFFCC" in plan["steps"][0]["what"]
    assert plan["steps"][0]["bytes_read"] <= 2 * R * C * 4 + 2 * C * 4 + 64    # x and gy once (not once per graph), g, b, constants


@pytest.mark.parametrize("shape", [(12, 256), (7, 100), (5, 37), (3, 1024), (2, 4096)])
def test_layernorm_forward_backward(shape):
    R, C = shape
    x = G.leaf(W.normal(0, (R, C), math.sqrt(2.0)), True)
    g, b = G.leaf(W.uniform(2, (C,), 0.5, 1.5), True), G.leaf(W.normal(3, (C,), 0.1), True)
    gy = G.leaf(W.normal(1, (R, C)))
    y = W.layernorm(x, g, b)
    y.grad = gy
    G.compute_gradients(y)
    plan = compare([y, x.grad, g.grad, b.grad], 2 * REDUCE_TOL)
    assert kinds(plan) == ["rows", "finalize"]       # y, dx, dg, db from one pass over x and gy; one launch adds up both partials


def test_mlp_step_schedule():
    B, D, H = 32, 16, 64
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(np.zeros(H, np.float32), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(np.zeros(D, np.float32), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    G.compute_gradients(loss)
    ups = [W.sgd_update(p, 0.1) for p in (w1, b1, w2, b2)]
    plan = compare([loss] + ups, 2 * REDUCE_TOL)
    k = kinds(plan)
    assert k.count("gemm") == 5
    assert len(k) <= 17, k    # 5 GEMMs + gelu, loss/grad/bias-grad, hidden grad, loss scale, 4 updates, 3 finalizes


def test_fusion_off_is_one_kernel_per_node():
    a, b = G.leaf(W.normal(0, (4, 8))), G.leaf(W.normal(1, (4, 8)))
    root = G.mul(G.add(a, b), G.exp(a))
    arr, order, roots = G.flatten([root], host_pointers=True)
    assert len(RT.plan([root])["steps"]) == 1


# ---------------------------------------------------------------------------- edge cases
def test_reference_known_answers_through_generated_kernels():
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
    outs, _ = E.realize([c for c, _ in cases])
    for o, (_, want) in zip(outs, cases):
        assert np.all(o == want)


def test_sums_every_kind():
    a = G.leaf(W.normal(0, (6, 5, 8)))
    roots = [G.sum_(a, [], False), G.sum_(a, [], True), G.sum_(a, [2], False), G.sum_(a, [1, 2], True),
             G.sum_(a, [0], False), G.sum_(a, [0, 1], False), G.sum_(a, [1], False), G.sum_(a, [0, 2], True)]
    compare(roots, REDUCE_TOL)
    e = G.exp(a)                                # the same, fused behind a producer
    roots = [G.sum_(e, [], False), G.sum_(e, [2], True), G.sum_(e, [0, 1], False), G.sum_(e, [1], False)]
    compare(roots, REDUCE_TOL)


def test_size_one_axes_and_rank0():
    a = G.leaf(W.normal(0, (1, 7, 1)))
    s = G.leaf(np.float32(3.0))
    roots = [G.sum_(a, [0], False), G.sum_(a, [0, 2], True), G.sum_(a, [1], False), G.mul(G.sum_(a, [], False), s),
             G.add(s, s), G.exp(G.neg(s))]
    compare(roots, REDUCE_TOL)


def test_views_as_operands():
    a = G.leaf(W.normal(0, (6, 10)))
    b = G.leaf(W.normal(1, (10, 6)))
    at = G.transpose(a, [1, 0])                                   # strided input
    r1 = G.mul(at, b)
    r2 = G.add(G.reshape(G.exp(a), [3, 20]), G.leaf(W.normal(2, (20,))))   # reshape of an un-realized node
    r3 = G.transpose(G.add(a, a), [1, 0])                         # root that is a view of an un-realized node
    r4 = G.add(G.expand(G.leaf(W.normal(3, (6, 1))), [6, 10]), a)
    r5 = G.mul(G.transpose(G.exp(a), [1, 0]), b)                  # permuted access to an un-realized node
    outs, plan = E.realize([r1, r2, r3, r4, r5])
    ref, _ = O.port_run([r1, r2, r3, r4, r5])
    for o, r in zip(outs, ref):
        assert np.abs(o - r).max() <= POINTWISE_TOL * np.abs(r).max()


def test_square_row_vector_is_not_mistaken_for_a_row_value():
    """[R] broadcast against [R, R] runs along columns; a row sum of shape [R] must not be fused as a per-row value."""
    x = G.leaf(W.normal(0, (8, 8)))
    s = G.sum_(x, [1], False)            # [8]
    compare([G.add(x, s)], REDUCE_TOL)   # x[i, j] + s[j]


def test_pointwise_tail_sizes():
    for n in (1, 3, 5, 127, 1000, 1025):
        a, b = G.leaf(W.normal(0, (n,))), G.leaf(W.normal(1, (n,)))
        compare([G.div(G.sub(a, b), G.add(G.mul(b, b), G.const(1.0))), G.sum_(G.mul(a, b), [], False)], REDUCE_TOL)


def test_wide_rows_fall_back_to_generic_sum():
    a = G.leaf(W.normal(0, (2, 40000)))
    plan = compare([G.sum_(G.mul(a, a), [1], False)], REDUCE_TOL)
    assert "generic_sum" in kinds(plan)


def test_matmul_layouts_and_gather():
    a = G.leaf(W.normal(0, (5, 7)))
    b = G.leaf(W.normal(1, (7, 3)))
    c = G.leaf(W.normal(2, (3, 7)))
    roots = [G.matmul(a, b), G.matmul(a, G.transpose(c, [1, 0])), G.matmul(G.transpose(b, [1, 0]), G.transpose(a, [1, 0])),
             G.matmul(G.expand(G.leaf(W.normal(3, (1, 7))), [5, 7]), b),                      # stride-0 rows
             G.matmul(G.expand(G.leaf(W.normal(4, (5, 1))), [5, 7]), b)]                      # stride-0 columns: gathered first
    compare(roots, REDUCE_TOL)


def test_random_graphs_against_oracle():
    rng = np.random.default_rng(1234)
    unary = [G.neg, G.exp, G.sin, G.cos]
    binary = [G.add, G.sub, G.mul]
    for trial in range(12):
        R, C = int(rng.integers(1, 9)), int(rng.choice([1, 4, 12, 33, 64]))
        pool = [G.leaf(rng.uniform(0.5, 1.5, size=s).astype(np.float32)) for s in ((R, C), (R, C), (C,), (R, 1), ())]
        for _ in range(int(rng.integers(3, 12))):
            if rng.random() < 0.35:
                pool.append(unary[int(rng.integers(len(unary)))](pool[int(rng.integers(len(pool)))]))
            elif rng.random() < 0.75:
                x, y = pool[int(rng.integers(len(pool)))], pool[int(rng.integers(len(pool)))]
                try:
                    pool.append(binary[int(rng.integers(len(binary)))](x, y))
                except RuntimeError:      # shapes that do not broadcast
                    pass
            else:
                x = pool[int(rng.integers(len(pool)))]
                if len(x.shape) == 2 and x.op not in G.VIEW_OPS:
                    axes = [[1], [0], []][int(rng.integers(3))]
                    pool.append(G.sum_(x, axes, bool(rng.integers(2))))
        roots = [n for n in pool[-3:] if not n.is_realized]
        if roots:
            compare(roots, 5 * REDUCE_TOL)


# ---------------------------------------------------------------------------- full-size schedules compile for sm_100a
def _fake(shape, rg=False):
    buf = G.Buffer(shape, host=np.zeros(1, np.float32))
    return G.Node(G.OpEnum.LEAF, data=buf, requires_grad=rg)


def test_full_size_schedules_compile_with_nvrtc():
    """The kernels of the benchmark configurations, generated at full size and compiled for sm_100a (no GPU needed)."""
    x, gy = _fake((16384, 4096), True), _fake((16384, 4096))
    y = W.softmax(x); y.grad = gy; G.compute_gradients(y)
    x2, g, b = _fake((16384, 4096), True), _fake((4096,), True), _fake((4096,), True)
    y2 = W.layernorm(x2, g, b); y2.grad = gy; G.compute_gradients(y2)
    a = [_fake((4096, 4096)) for _ in range(3)]
    plans = [RT.plan([y, x.grad]), RT.plan([y2, x2.grad, g.grad, b.grad]), RT.plan([W.fused_rowsum(*a)])]
    assert [len(p["steps"]) for p in plans] == [1, 2, 1]
    for p in plans:
        assert p["error"] == ""
        for s in p["steps"]:
            assert RT.compile_cubin(s["source"]) > 0
    # algorithmic traffic of the layernorm backward+forward kernel: x, gy in; y, dx out (+ small vectors and partials)
    big = plans[1]["steps"][0]
    assert big["bytes_read"] >= 2 * 16384 * 4096 * 4 and big["bytes_written"] >= 2 * 16384 * 4096 * 4


# ---------------------------------------------------------------------------- limits the backend states out loud
def test_empty_dimension_is_rejected_with_a_message():
    """A zero-sized dimension has no defined meaning in the reference (its broadcast rule turns (0, 5) + (5,) into
    (1, 5)); the backend refuses it instead of guessing."""
    a = G.leaf(np.zeros((0, 5), np.float32))
    for root in (G.add(a, a), G.sum_(a, [0], False), G.matmul(a, G.leaf(np.ones((5, 3), np.float32)))):
        assert "empty or negative dimension" in RT.plan([root])["error"]


def test_more_than_2_31_elements_is_rejected_with_a_message():
    """Index arithmetic is 32-bit like the reference's: a tensor of 2^31 elements is refused at plan time."""
    big = G.Node(G.OpEnum.LEAF, data=G.Buffer((1 << 16, 1 << 15), host=np.zeros(1, np.float32)))
    assert "2^31" in RT.plan([G.add(big, big)])["error"]
    ok = G.Node(G.OpEnum.LEAF, data=G.Buffer((1 << 15, 1 << 15), host=np.zeros(1, np.float32)))     # 2^30: the largest power of two
    assert not RT.plan([G.add(ok, ok)])["error"]
    # the last grid-stride step of a kernel may overshoot the end by a grid of vector accesses before its bound check:
    # sizes within 2^22 of 2^31 are refused too, and so is a strided view whose EXTENT (not its element count) gets there
    near = G.Node(G.OpEnum.LEAF, data=G.Buffer(((1 << 31) - 1024,), host=np.zeros(1, np.float32)))
    assert "2^31" in RT.plan([G.neg(near)])["error"]
    wide = G.Node(G.OpEnum.LEAF, data=G.Buffer((1 << 16, 1 << 15), host=np.zeros(1, np.float32)))
    wide.shape, wide.strides = [1 << 10, 1 << 10], [1 << 21, 1]                              # 2^20 elements spread over 2^31
    assert "spans 2^31" in RT.plan([G.sum_(G.transpose(wide, [1, 0]), [0], False)])["error"]


@pytest.mark.parametrize("shape", [(1, 1), (1, 7), (7, 1), (3, 33), (33, 3), (2, 1025), (129, 5)])
def test_ragged_shapes_softmax_layernorm_and_sums(shape):
    R, C = shape
    x = G.leaf(W.normal(0, (R, C)), True)
    g, b = G.leaf(W.uniform(1, (C,), 0.5, 1.5), True), G.leaf(W.normal(2, (C,), 0.1), True)
    y = W.layernorm(x, g, b)
    y.grad = G.leaf(W.normal(3, (R, C)))
    G.compute_gradients(y)
    compare([y, x.grad, g.grad, b.grad, W.softmax(x), G.sum_(x, [0], False), G.sum_(x, [1], True), G.sum_(x, [], False)], 5 * REDUCE_TOL)


# ---------------------------------------------------------------------------- "bf16" matmul arithmetic: fused epilogues, bf16 twins

BF16_TOL = 2e-2


def _mlp(B, D, H, bias_std=0.1):
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(W.normal(4, (H,), bias_std), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(W.normal(5, (D,), bias_std), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    G.compute_gradients(loss)
    return loss, (w1, b1, w2, b2)


def test_bf16_mlp_step_fuses_epilogues_and_writes_twins():
    """The training step in "bf16" arithmetic: GELU runs in the first GEMM's epilogue and leaves only a bf16 hidden
    activation, every in-plan matmul operand is written as bf16 by its producer (no conversion pass over it), the hidden
    gradient is never written as fp32, and the weight update of the first layer sits in the epilogue of its gradient GEMM."""
    loss, params = _mlp(256, 128, 512)
    ups = [W.sgd_update(p, 0.1) for p in params]
    plan = RT.plan([loss] + ups, options="matmul=bf16")
    assert not plan["error"]
    gemms = [s for s in plan["steps"] if s["type"] == "gemm"]
    assert len(gemms) == 5 and all(g["tc"] for g in gemms)
    first = gemms[0]
    assert "nodes=13" in first["epilogue"] and "outs=h" in first["epilogue"] and first["store_c"]      # h as bf16 only, x W1 kept for backward
    assert "expf" in first["epi_body"] and "ormi_store_bf16x4" in first["epi_body"]
    assert gemms[1]["a16"] >= 0                                     # h W2 reads the twin the epilogue wrote
    assert gemms[2]["a16"] >= 0                                     # g_out W2^T reads g_out's twin
    dw1 = [g for g in gemms if g["trans_a"] and not g["store_c"]]
    assert len(dw1) >= 1 and all("outs=F" in g["epilogue"] for g in dw1)   # W1 - lr * (x^T du): the product itself is never stored
    twins = [b for b in plan["buffers"] if b["kind"] == "twin16"]
    assert len(twins) == 3                                          # h, g_out, du
    assert not any("gelu" in s.get("what", "") for s in plan["steps"])
    kernels = [s for s in plan["steps"] if s["type"] == "kernel"]
    assert len(kernels) + len(gemms) <= 14
    # without the option the same graph keeps the fp32 schedule
    assert not any(s.get("tc") for s in RT.plan([loss] + ups)["steps"] if s["type"] == "gemm")


@pytest.mark.parametrize("bdh", [(256, 128, 512), (128, 136, 264)])
def test_bf16_mlp_step_on_the_emulator(bdh):
    loss, params = _mlp(*bdh)
    roots = [loss] + [p.grad for p in params] + [W.sgd_update(p, 0.1) for p in params]
    ref, _ = O.port_run(roots)
    outs, plan = E.realize(roots, options="matmul=bf16")
    assert sum(1 for s in plan["steps"] if s["type"] == "gemm" and s["tc"]) == 5
    for a, b in zip(outs, ref):
        assert a.shape == b.shape
        assert np.abs(a - b).max() <= BF16_TOL * max(1e-30, np.abs(b).max())


def test_bf16_matmul_chain_and_epilogue_operand_kinds():
    """A product that feeds the next matmul directly (bf16 twin written by the GEMM itself), and an epilogue with every
    operand kind: a bias row, a per-row column, a full matrix, a scalar."""
    M, K, N, P = 128, 128, 136, 128
    a, b, c = G.leaf(W.normal(0, (M, K), 0.1)), G.leaf(W.normal(1, (K, N), 0.1)), G.leaf(W.normal(2, (N, P), 0.1))
    bias, col, full = G.leaf(W.normal(3, (P,))), G.leaf(W.normal(4, (M, 1))), G.leaf(W.normal(5, (M, P)))
    y = G.matmul(G.matmul(a, b), c)
    root = G.mul(G.add(G.add(y, bias), G.mul(col, full)), G.const(0.5))
    ref, _ = O.port_run([root])
    outs, plan = E.realize([root], options="matmul=bf16")
    gemms = [s for s in plan["steps"] if s["type"] == "gemm"]
    assert [g["tc"] for g in gemms] == [True, True]
    assert "product=Fh" in gemms[0]["epilogue"] or "product=h" in gemms[0]["epilogue"]
    assert gemms[1]["a16"] >= 0 and not gemms[1]["store_c"] and len(plan["steps"]) == 2
    assert np.abs(outs[0] - ref[0]).max() <= BF16_TOL * np.abs(ref[0]).max()


def test_unaligned_inputs_get_scalar_kernels():
    """A caller's pointer that is not on a 16-byte boundary: the whole plan is generated without 128-bit accesses, bulk
    copies or the tensor-core kernel (the bit is part of the plan key)."""
    loss, params = _mlp(256, 128, 512)
    plan = RT.plan([loss, params[0].grad], options="matmul=bf16,aligned=0")
    assert not plan["error"]
    for s in plan["steps"]:
        if s["type"] == "kernel":
            assert "float4" not in s["source"].split("#endif")[-1] and s["dyn_smem"] == 0
        else:
            assert not s["tc"]
    x = G.leaf(W.normal(0, (64, 256)), True)
    y = W.softmax(x)
    outs, plan = E.realize([y], options="aligned=0")
    assert "V=1" in plan["steps"][0]["what"]
    ref, _ = O.port_run([y])
    assert np.abs(outs[0] - ref[0]).max() <= REDUCE_TOL * np.abs(ref[0]).max()


def test_registered_lowering_replaces_the_builtin_expression():
    """ormi_b200_set_lowering, the C side of the reference's CUDALoweringRegistry: the expression given for an op is what
    the fused kernels (and the guarded scalar kernel of ormi_b200_compile_source) evaluate, until it is taken back."""
    import ctypes
    from ormi_b200._lib import lib, check
    x = G.leaf(W.normal(0, (6, 40)))
    build = lambda: G.add(G.sin(x), G.sum_(G.sin(x), [1], True))
    try:
        check(lib.ormi_b200_set_lowering(int(G.OpEnum.SIN), b"cosf($0) * 2.0f"))
        outs, plan = E.realize([build()])
        assert "cosf(" in plan["steps"][0]["source"] and "sinf(" not in plan["steps"][0]["source"].split("#endif")[-1]
        c = 2.0 * np.cos(x.data.host.astype(np.float64))
        assert np.abs(outs[0] - (c + c.sum(axis=1, keepdims=True))).max() <= REDUCE_TOL * 100
        arr, order, roots = G.flatten([G.sin(x)], host_pointers=True)
        buf = ctypes.create_string_buffer(1 << 16)
        n = ctypes.c_size_t()
        check(lib.ormi_b200_compile_source(arr, len(order), roots[0], buf, len(buf), ctypes.byref(n), None, 0, None))
        assert b"cosf(val_LEAF_0) * 2.0f" in buf.value
        assert lib.ormi_b200_set_lowering(int(G.OpEnum.MATMUL), b"$0") != 0          # only pointwise ops have one
    finally:
        check(lib.ormi_b200_set_lowering(int(G.OpEnum.SIN), None))
    compare([build()], 2 * REDUCE_TOL)           # the stock sine again


def test_sum_over_a_view_with_few_outputs_uses_a_block_per_output():
    """A global (or near-global) sum whose operand is a view cannot take the fused templates; with few outputs each one
    gets a block whose threads stride over the reduced coordinates, not one thread walking them all."""
    a = W.normal(0, (64, 48))
    t = G.transpose(G.leaf(a), [1, 0])
    outs, plan = E.realize([G.sum_(t, [], False), G.sum_(t, [0], False)])
    whats = [s["what"] for s in plan["steps"]]
    assert any("generic_sum[out=1,red=3072,block]" in w for w in whats), whats
    assert abs(float(outs[0]) - a.sum(dtype=np.float64)) <= REDUCE_TOL * np.abs(a).sum()
    assert np.abs(outs[1] - a.sum(axis=1, dtype=np.float64)).max() <= REDUCE_TOL * np.abs(a).sum(axis=1).max()


def _bf16_words(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def test_first_class_bf16_tensors_cross_realize_calls():
    """ORMI_NODE_BF16: a root materialized as bf16 ONLY (no fp32 copy is written), handed back, and read by the matmuls
    of a later call as a bf16 tensor — the way the sharded trainer carries the hidden activation from one phase to the
    next.  Anything but a tensor-core matmul refuses such a tensor."""
    B, D, H = 256, 128, 512
    x, w1, b1, w2 = W.normal(0, (B, D)), W.kaiming_uniform(2, D, (D, H)), W.normal(4, (H,), 0.1), W.kaiming_uniform(3, H, (H, D))
    # call 1: h = gelu(x W1 + b1) as a bf16-only root
    h = W.gelu_tanh(G.add(G.matmul(G.leaf(x), G.leaf(w1)), G.leaf(b1)))
    h.bf16 = True
    (want_h,), _ = O.port_run([W.gelu_tanh(G.add(G.matmul(G.leaf(x), G.leaf(w1)), G.leaf(b1)))])
    outs, plan = E.realize([h], options="matmul=bf16")
    gemm = [s for s in plan["steps"] if s["type"] == "gemm"][0]
    assert len(plan["steps"]) == 1 and "outs=h" in gemm["epilogue"] and not gemm["store_c"]      # one kernel, nothing fp32 leaves it
    assert [r["bf16"] for r in plan["results"]] == [True]
    assert np.abs(outs[0] - want_h).max() <= BF16_TOL * np.abs(want_h).max()
    # call 2: the bf16 tensor as operand of two matmuls, plain and transposed
    h16 = G.Node(G.OpEnum.LEAF, data=G.Buffer((B, H), host=_bf16_words(outs[0])))
    h16.data.nbytes = B * H * 2
    h16.bf16 = True
    g = W.normal(5, (B, D))
    roots = [G.matmul(h16, G.leaf(w2)), G.matmul(G.transpose(h16, [1, 0]), G.leaf(g))]
    outs2, plan2 = E.realize(roots, options="matmul=bf16")
    gemms = [s for s in plan2["steps"] if s["type"] == "gemm"]
    assert all(s["tc"] and s["a16"] == s["a"] for s in gemms)                                    # read in place, no conversion
    assert np.abs(outs2[0] - outs[0] @ w2).max() <= BF16_TOL * np.abs(outs[0] @ w2).max()
    assert np.abs(outs2[1] - outs[0].T @ g).max() <= BF16_TOL * np.abs(outs[0].T @ g).max()
    # refused: pointwise work on a bf16 tensor, a bf16 root of another arithmetic, a shape the tensor cores do not take
    assert "bf16 tensor can only be" in RT.plan([G.exp(h16)], options="matmul=bf16")["error"]
    assert "need the" in RT.plan([G.matmul(h16, G.leaf(w2))])["error"]
    small = G.mul(G.leaf(W.normal(0, (4, 6))), G.leaf(W.normal(1, (4, 6))))
    small.bf16 = True
    assert "bf16 only when" in RT.plan([small], options="matmul=bf16")["error"]


def test_intermediates_free_makes_unheld_nodes_scratch():
    """With "intermediates=free" only roots (and KEEP nodes) come back; a materialized node nobody outside the call holds
    — the product x W1 that the backward epilogue reads again, for one — is a scratch buffer of the plan.  Same steps,
    same values."""
    loss, params = _mlp(256, 128, 512)
    roots = [loss] + [W.sgd_update(p, 0.1) for p in params]
    keep = RT.plan(roots, options="matmul=bf16")
    free = RT.plan(roots, options="matmul=bf16,intermediates=free")
    assert not keep["error"] and not free["error"]
    assert [s["type"] for s in keep["steps"]] == [s["type"] for s in free["steps"]]
    assert len(free["results"]) == len(roots) < len(keep["results"])
    dropped = {r["buffer"] for r in keep["results"]} - {r["buffer"] for r in free["results"]}
    assert dropped and all(free["buffers"][b]["kind"] == "temp" and keep["buffers"][b]["kind"] == "node" for b in dropped)
    a, _ = E.realize(roots, options="matmul=bf16")
    b, _ = E.realize(roots, options="matmul=bf16,intermediates=free")
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    # a node the caller keeps stays a result
    loss2, params2 = _mlp(64, 32, 64)
    hidden = loss2
    while hidden.op != G.OpEnum.MATMUL:
        hidden = hidden.parents[0]
    hidden.keep = True
    plan = RT.plan([loss2], options="intermediates=free")
    assert len(plan["results"]) == 2
