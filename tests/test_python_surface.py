"""The Python binding surface: ormi-core's own pybind11 module (built unchanged on top of the B200 backend) under
the ``Tensor`` layer of ormi_b200/tensor.py.

Without a GPU the module's CPU device runs (that is ormi-core's CPU backend, unmodified): these cases pin the host
logic of the Tensor layer.  With a GPU every case also runs on ``device="cuda"`` — graphs go through
``execute_graph`` -> the execute_jit seam -> ``ormi_b200_realize`` — and is compared with the CPU device of the
same module on identical inputs.  Topics follow ormi-core/tests/test_tensor.py:5-81.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

try:
    from ormi_b200.tensor import Tensor, DeviceMismatchError, backend
except ImportError as e:          # a checkout without the ormi-core sources cannot build the module
    pytest.skip(str(e), allow_module_level=True)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("ORMI_REFERENCE") or __import__("re").search(      # the ormi checkout, where there is one: the Makefile's default
    r"^REF\s*\?=\s*(\S+)", open(os.path.join(ROOT, "oracle", "Makefile")).read(), __import__("re").M).group(1)
DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
PW_TOL, REDUCE_TOL = 1e-6, 1e-5


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(1e-30, np.abs(b).max()))


@pytest.mark.parametrize("dev", DEVICES)
def test_leaf_attributes(dev):
    t = Tensor([[1.0, 2.0], [3.0, 4.0]], device=dev, requires_grad=True)
    assert t.shape == (2, 2) and t.requires_grad and t.op.name == "LEAF"
    assert t.device.type.name.lower() == dev
    assert t.grad is None
    np.testing.assert_array_equal(t.numpy(), [[1.0, 2.0], [3.0, 4.0]])
    assert "realized" in repr(t) and "LEAF" in repr(t)


@pytest.mark.parametrize("dev", DEVICES)
def test_arithmetic_and_scalar_promotion(dev):
    a, b = Tensor([8.0, 9.0, -3.0], device=dev), Tensor([2.0, 3.0, 4.0], device=dev)
    np.testing.assert_allclose((a + b).numpy(), [10.0, 12.0, 1.0])
    np.testing.assert_allclose((a - b).numpy(), [6.0, 6.0, -7.0])
    np.testing.assert_allclose((a * b).numpy(), [16.0, 27.0, -12.0])
    np.testing.assert_allclose((a / b).numpy(), [4.0, 3.0, -0.75])
    np.testing.assert_allclose((-a).numpy(), [-8.0, -9.0, 3.0])
    np.testing.assert_allclose((b ** 3.0).numpy(), [8.0, 27.0, 64.0])
    # a scalar on the left goes through the reflected operators
    np.testing.assert_allclose((1.0 + b).numpy(), [3.0, 4.0, 5.0])
    np.testing.assert_allclose((1.0 - b).numpy(), [-1.0, -2.0, -3.0])
    np.testing.assert_allclose((3.0 * b).numpy(), [6.0, 9.0, 12.0])
    np.testing.assert_allclose((12.0 / b).numpy(), [6.0, 4.0, 3.0])
    lazy = a * b + 1.0
    assert "lazy" in repr(lazy)
    lazy.realize()
    assert "realized" in repr(lazy)


@pytest.mark.parametrize("dev", DEVICES)
def test_matmul_and_operand_check(dev):
    a = Tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], device=dev)
    b = Tensor([[1.0, 0.0], [0.0, 1.0], [2.0, 2.0]], device=dev)
    c = a @ b
    assert c.shape == (2, 2)
    np.testing.assert_allclose(c.numpy(), [[7.0, 8.0], [16.0, 17.0]])
    with pytest.raises(TypeError):
        _ = a @ 3.0


@pytest.mark.parametrize("dev", DEVICES)
def test_views(dev):
    a = Tensor(np.arange(12, dtype=np.float32).reshape(3, 4), device=dev)
    np.testing.assert_array_equal(a.reshape((2, 6)).numpy(), np.arange(12).reshape(2, 6))
    np.testing.assert_array_equal(a.transpose().numpy(), np.arange(12).reshape(3, 4).T)
    row = Tensor([1.0, 2.0, 3.0, 4.0], device=dev)
    np.testing.assert_array_equal((a + row.expand((3, 4))).numpy(), np.arange(12).reshape(3, 4) + [1, 2, 3, 4])
    np.testing.assert_array_equal((a.transpose() * 2.0).numpy(), 2 * np.arange(12).reshape(3, 4).T)


@pytest.mark.parametrize("dev", DEVICES)
def test_backward_and_zero_grad(dev):
    a = Tensor([2.0, 3.0], device=dev, requires_grad=True)
    b = Tensor([4.0, 5.0], device=dev, requires_grad=True)
    z = a * b + a * a            # dz/da = b + 2a, dz/db = a
    z.backward()
    np.testing.assert_allclose(a.grad.numpy(), [8.0, 11.0])
    np.testing.assert_allclose(b.grad.numpy(), [2.0, 3.0])
    a.zero_grad()
    assert a.grad is None and b.grad is not None
    z.zero_grad_graph()
    assert b.grad is None
    with pytest.raises(RuntimeError):
        Tensor([1.0], device=dev).backward()


def test_device_errors():
    with pytest.raises(DeviceMismatchError):
        Tensor([1.0], device="tpu")
    with pytest.raises(DeviceMismatchError):
        Tensor([1.0], device=3)
    a = Tensor([1.0], device="cpu")
    assert a.device.type == backend.DeviceEnum.CPU and Tensor([1.0]).device.type == backend.DeviceEnum.CPU


def _softmax(x):
    e = x.exp()
    return e / e.sum([1], True)


def _layernorm(x, g, b, eps=1e-5):
    n = float(x.shape[1])
    mu = x.sum([1], True) / n
    d = x - mu
    var = (d * d).sum([1], True) / n
    return d / (var + eps) ** 0.5 * g + b


def _run_graphs(dev, seed=0):
    rng = np.random.default_rng(seed)
    R, C = 64, 96
    x_h = (rng.standard_normal((R, C)) * 1.5).astype(np.float32)
    g_h, b_h = rng.uniform(0.5, 1.5, C).astype(np.float32), (rng.standard_normal(C) * 0.1).astype(np.float32)
    w_h = (rng.standard_normal((C, 32)) / np.sqrt(C)).astype(np.float32)
    x, g, b = (Tensor(v, device=dev, requires_grad=True) for v in (x_h, g_h, b_h))
    w = Tensor(w_h, device=dev, requires_grad=True)
    loss = ((_layernorm(x, g, b) @ w) * _softmax(x @ w)).sum()
    loss.backward()
    return [t.numpy().copy() for t in (loss, x.grad, g.grad, b.grad, w.grad)]


def test_fused_graphs_on_cpu_device():
    """The CPU device of the module against numpy in fp64: the Tensor layer builds the graph it should."""
    rng = np.random.default_rng(0)
    x_h = (rng.standard_normal((64, 96)) * 1.5).astype(np.float32)
    y = _softmax(Tensor(x_h, device="cpu")).numpy()
    e = np.exp(x_h.astype(np.float64))
    assert rel(y, e / e.sum(1, keepdims=True)) <= REDUCE_TOL
    assert len(_run_graphs("cpu")) == 5


@pytest.mark.gpu
def test_fused_graphs_cuda_against_cpu_device():
    """layernorm -> matmul, softmax, a product, a global sum and the whole backward: the CUDA device of the module (the
    fusion scheduler behind execute_graph) against its CPU device (ormi-core's CPU backend) on the same inputs."""
    want, got = _run_graphs("cpu"), _run_graphs("cuda")
    for w, g in zip(want, got):
        assert w.shape == g.shape
        assert rel(g, w) <= 3 * REDUCE_TOL


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "ormi-core", "tests")), reason="needs the ormi checkout")
def test_ormi_core_python_tests_on_cpu_device():
    """ormi-core's own Python package and tests (read where they lie, CPU device only here) on top of the module built
    in this repository."""
    code = (
        "import sys; sys.dont_write_bytecode = True\n"
        f"sys.path[:0] = [{os.path.join(REF, 'ormi-core', 'src')!r}, {ROOT!r}]\n"
        "from ormi_b200 import tensor as T\n"
        "sys.modules['ormi_core._ext.ormi_backend'] = T.backend\n"
        "import pytest\n"
        f"sys.exit(pytest.main([{os.path.join(REF, 'ormi-core', 'tests', 'test_tensor.py')!r}, '-q', '-k', 'cpu', '-p', 'no:cacheprovider',"
        " '--rootdir', '/tmp', '-c', '/dev/null']))\n"
    )
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd="/tmp")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert " passed" in out.stdout


@pytest.mark.gpu
def test_example_scenarios_on_cuda():
    """The scenarios of ormi-core's example scripts (example/test_graph.py:5-15: a pointwise chain over an odd-sized
    [2029, 1202] tensor; example/test_matmul.py:7-18: a [2, 3] @ [3, 1] graph break), on device="cuda"."""
    rng = np.random.default_rng(5)
    x_h, w_h, b_h = (rng.random((2029, 1202)).astype(np.float32) for _ in range(3))
    X, Wt, b = (Tensor(v, device="cuda") for v in (x_h, w_h, b_h))
    Z = (Wt * (X ** 2.0)) + b
    Z.realize()
    assert rel(Z.numpy(), w_h.astype(np.float64) * x_h.astype(np.float64) ** 2 + b_h) <= PW_TOL
    Wm = Tensor(np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], dtype=np.float32), device="cuda")
    Xm = Tensor(np.array([[1.0], [2.0], [3.0]], dtype=np.float32), device="cuda")
    Zm = Wm @ Xm
    assert Zm.shape == (2, 1)
    np.testing.assert_array_equal(Zm.numpy(), [[14.0], [32.0]])


def test_backend_knobs_need_a_gpu_or_work():
    """set_option / counter reach the process-wide context of the CUDA device; without a GPU they fail loudly."""
    from ormi_b200 import tensor as T
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            T.set_option("matmul", "bf16")
        assert T.counter("launches") == -1


@pytest.mark.gpu
def test_matmul_mode_and_fusion_knobs_on_cuda():
    from ormi_b200 import tensor as T
    rng = np.random.default_rng(3)
    a_h = (rng.standard_normal((256, 512)) / np.sqrt(512)).astype(np.float32)
    b_h = (rng.standard_normal((512, 384)) / np.sqrt(512)).astype(np.float32)
    want = a_h.astype(np.float64) @ b_h.astype(np.float64)
    exact = (Tensor(a_h, device="cuda") @ Tensor(b_h, device="cuda")).numpy().copy()
    assert rel(exact, want) <= REDUCE_TOL
    T.set_option("matmul", "bf16")
    try:
        g0 = T.counter("gemm_launches")
        rounded = (Tensor(a_h, device="cuda") @ Tensor(b_h, device="cuda")).numpy().copy()
        assert T.counter("gemm_launches") == g0 + 1
        assert 1e-5 < rel(rounded, want) <= 2e-2              # bf16 operands: inside its own tolerance, not fp32-exact
    finally:
        T.set_option("matmul", "fp32")
    T.set_option("fusion", "off")
    try:
        l0 = T.counter("launches")
        x = Tensor(a_h, device="cuda")
        y = ((x * 2.0) + 1.0).exp().numpy()
        assert T.counter("launches") - l0 >= 3                   # one kernel per node, like the reference
        assert rel(y, np.exp(a_h.astype(np.float64) * 2 + 1)) <= PW_TOL
    finally:
        T.set_option("fusion", "on")
    with pytest.raises(RuntimeError):
        T.set_option("matmul", "fp64")


@pytest.mark.parametrize("dev", DEVICES)
def test_known_answers_of_the_reference_python_tests(dev):
    """The eight cases of ormi-core/tests/test_tensor.py:5-81 with their own numbers (that file is parametrised over
    "cpu" and "cuda" by ormi-core/tests/conftest.py:3-5; it cannot be read on a machine without the ormi checkout, so its
    known answers are restated here against the same extension module)."""
    t = Tensor([1.0, 2.0, 3.0], device=dev, requires_grad=True)                       # initialization
    assert t.shape == (3,) and t.requires_grad is True and t.device.type.name.lower() == dev
    np.testing.assert_allclose(t.numpy(), [1.0, 2.0, 3.0])
    a, b = Tensor([4.0, 6.0], device=dev), Tensor([2.0, 3.0], device=dev)               # binary operations
    for got, want in (((a + b), [6.0, 9.0]), ((a - b), [2.0, 3.0]), ((a * b), [8.0, 18.0]), ((a / b), [2.0, 2.0]),
                      ((-a), [-4.0, -6.0]), ((a ** 2.0), [16.0, 36.0])):
        np.testing.assert_allclose(got.numpy(), want)
    c = Tensor([2.0, 4.0], device=dev)                                                  # reverse operations
    for got, want in (((10.0 + c), [12.0, 14.0]), ((10.0 - c), [8.0, 6.0]), ((10.0 * c), [20.0, 40.0]), ((10.0 / c), [5.0, 2.5])):
        np.testing.assert_allclose(got.numpy(), want)
    m = Tensor([[1.0, 2.0], [3.0, 4.0]], device=dev) @ Tensor([[2.0, 0.0], [0.0, 2.0]], device=dev)   # matmul
    assert m.shape == (2, 2)
    np.testing.assert_allclose(m.numpy(), [[2.0, 4.0], [6.0, 8.0]])
    with pytest.raises(TypeError):                                                        # matmul type enforcement
        _ = Tensor([[1.0, 2.0]], device=dev) @ 2.0
    v = Tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]], device=dev)                           # view operations
    r = v.reshape((3, 2))
    assert r.shape == (3, 2)
    np.testing.assert_allclose(r.numpy(), [[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]])
    tr = v.transpose()
    assert tr.shape == (3, 2)
    np.testing.assert_allclose(tr.numpy(), [[1.0, 4.0], [2.0, 5.0], [3.0, 6.0]])
    p = Tensor([2.0, 3.0], device=dev, requires_grad=True)                               # autograd graph: z = p q + p
    q = Tensor([4.0, 5.0], device=dev, requires_grad=True)
    (p * q + p).backward()
    np.testing.assert_allclose(p.grad.numpy(), [5.0, 6.0])
    np.testing.assert_allclose(q.grad.numpy(), [2.0, 3.0])
    z = Tensor([1.0], device=dev, requires_grad=True)                                    # zero_grad
    (z * 2.0).backward()
    assert z.grad is not None
    z.zero_grad()
    assert z.grad is None


@pytest.mark.parametrize("dev", DEVICES)
def test_additive_log_and_pow_function_bindings(dev):
    """ormi-core's binding file leaves log and pow out (csrc/bindings/bind_pointwise.cpp:16-25) although the ops exist;
    the additive module binds them as functions next to add, sub, ... of the stock module."""
    from ormi_b200 import tensor as T
    if T.extra is None:
        pytest.skip("ormi_backend_extra not built")
    x = Tensor([1.0, 2.0, 4.0], device=dev)
    e = Tensor([0.5, 2.0, 3.0], device=dev)
    np.testing.assert_allclose(x._wrap(T.extra.log(x._node)).numpy(), np.log([1.0, 2.0, 4.0]), rtol=1e-6)
    np.testing.assert_allclose(x._wrap(T.extra.pow(x._node, e._node)).numpy(), [1.0, 4.0, 64.0], rtol=1e-6)
    np.testing.assert_allclose(x.log().numpy(), np.log([1.0, 2.0, 4.0]), rtol=1e-6)


@pytest.mark.gpu
def test_tensors_follow_the_active_device():
    """One backend context per GPU behind the module: after set_device(1) new CUDA tensors live on GPU 1 and their graphs
    run there; tensors of two devices do not mix."""
    import torch
    from ormi_b200 import tensor as T
    if torch.cuda.device_count() < 2 or T.extra is None:
        pytest.skip("needs two GPUs and the additive module")
    a0 = Tensor(np.arange(8, dtype=np.float32), device="cuda")
    try:
        T.set_device(1)
        assert T.extra.active_device() == 1
        before = T.extra.counter("launches")
        a1 = Tensor(np.arange(8, dtype=np.float32), device="cuda")
        np.testing.assert_allclose((a1 * a1 + 1.0).numpy(), np.arange(8.0) ** 2 + 1.0)
        assert T.extra.counter("launches") > before            # the counter of GPU 1's context moved
        with pytest.raises(RuntimeError, match="cuda:0 and cuda:1|cuda:1 and cuda:0"):
            (a0 + a1).numpy()
        with pytest.raises(RuntimeError):
            T.set_device(64)
    finally:
        T.set_device(0)
    np.testing.assert_allclose((a0 + a0).numpy(), 2 * np.arange(8.0))
