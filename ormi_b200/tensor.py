"""Python ``Tensor`` over ormi-core's own pybind11 module, with the B200 backend underneath.

The extension module ``ormi_backend`` is built from the reference's binding sources, unchanged
(ormi-core/csrc/bindings/*.cpp), on top of ormi-core linked with this repository's backend
(``make -C ormi_b200/csrc/seams``).  This file is the thin Python layer above it and keeps the surface of
ormi-core's ``Tensor`` (ormi-core/src/ormi_core/tensor.py:10-190): constructor arguments, ``shape`` / ``op`` /
``requires_grad`` / ``grad`` / ``device``, the arithmetic operators with scalar promotion, ``@``, ``reshape``,
``transpose``, ``realize``, ``numpy``, ``backward``, ``zero_grad``, ``zero_grad_graph`` and the errors they raise.
Additions (``sum``, ``exp``, ``log``, ``sin``, ``cos``, ``expand``) only call what the module already exports.

A graph built on ``device="cuda"`` is handed whole to the fusion scheduler by ``execute_graph``; nothing in
this file knows about kernels.
"""
from __future__ import annotations

import glob
import importlib.util
import os
from typing import Sequence

import numpy as np

_BUILD_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "seams", "_build")


def _load_backend():
    hits = sorted(h for h in glob.glob(os.path.join(_BUILD_DIR, "ormi_backend*.so")) if "ormi_backend_extra" not in h)
    if not hits:
        raise ImportError("ormi_backend is not built: run `make -C ormi_b200/csrc/seams REF=<ormi checkout>` "
                          "(needs the ormi-core sources and pybind11)")
    # the CPU device's matmul is OpenBLAS' cblas_sgemm, looked up at first use: point the shim at the interpreter's own copy
    if not os.environ.get("ORMI_ORACLE_OPENBLAS"):
        import sysconfig
        site = sysconfig.get_paths()["purelib"]
        for pattern in ("scipy.libs/libscipy_openblas*.so", "opencv_python_headless.libs/libopenblas*.so"):
            found = sorted(glob.glob(os.path.join(site, pattern)))
            if found:
                os.environ["ORMI_ORACLE_OPENBLAS"] = found[0]
                break
    spec = importlib.util.spec_from_file_location("ormi_backend", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


backend = _load_backend()


def _load_extra():
    """The additive bindings (ormi_b200/csrc/seams/b200_bindings_extra.cpp): log / pow as functions, device selection."""
    hits = sorted(glob.glob(os.path.join(_BUILD_DIR, "ormi_backend_extra*.so")))
    if not hits:
        return None
    spec = importlib.util.spec_from_file_location("ormi_backend_extra", hits[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


extra = _load_extra()


def set_device(index: int) -> None:
    """The GPU that later ``device="cuda"`` tensors are placed on (and their graphs run on).  One process per GPU calls
    it once with its local rank; ormi-core itself always uses device 0.  Raises when there is no such device."""
    if extra is None:
        raise RuntimeError("ormi_backend_extra is not built")
    extra.set_device(int(index))


def _engine():
    import ctypes
    lib = ctypes.CDLL(os.path.join(_BUILD_DIR, "libormi_engine_b200.so"))
    lib.ormi_engine_b200_set_option.argtypes = [ctypes.c_char_p, ctypes.c_char_p]
    lib.ormi_engine_b200_counter.argtypes = [ctypes.c_char_p]
    lib.ormi_engine_b200_counter.restype = ctypes.c_longlong
    return lib


def set_option(key: str, value: str) -> None:
    """Backend knobs of the CUDA device ("matmul": fp32 | bf16 | tf32 | 3xtf32, "fusion": on | off); additive, ormi-core
    itself has none.  Raises without a GPU or for an unknown option."""
    if _engine().ormi_engine_b200_set_option(key.encode(), value.encode()) != 0:
        raise RuntimeError(f"cannot set backend option {key}={value} (no GPU, or unknown option)")


def counter(name: str) -> int:
    """A counter of the CUDA device's context (launches, gemm_launches, kernels_compiled, plan_cache_hits, ...)."""
    return int(_engine().ormi_engine_b200_counter(name.encode()))


OpEnum, DeviceEnum, Device, Node = backend.OpEnum, backend.DeviceEnum, backend.Device, backend.Node


class OrmiError(Exception):
    pass


class DeviceMismatchError(OrmiError):
    """Unknown device, or operands that live on different devices (ormi-core/src/ormi_core/exceptions.py:8-15)."""


_DEVICE_NAMES = {"cpu": DeviceEnum.CPU, "cuda": DeviceEnum.CUDA}


def _as_device(device) -> Device:
    if device is None:
        return Device(DeviceEnum.CPU, 0)
    if isinstance(device, Device):
        return device
    if isinstance(device, DeviceEnum):
        return Device(device, 0)
    if isinstance(device, str):
        kind = _DEVICE_NAMES.get(device.lower())
        if kind is None:
            raise DeviceMismatchError(f'Unsupported string backend | Got: "{device}"')
        return Device(kind, 0)
    raise DeviceMismatchError(f'Device argument is of invalid type. | Got: "{type(device)}"')


class Tensor:
    """A lazy node of the graph; nothing runs before ``realize`` / ``numpy``."""

    def __init__(self, data=None, device=None, requires_grad: bool = False, _node: Node | None = None):
        self.device = _as_device(device)
        if _node is not None:
            self._node = _node
        elif data is not None:
            host = data if isinstance(data, np.ndarray) else np.array(data, dtype=np.float32)
            self._node = Node(backend.numpy_to_buffer(host, self.device.type), requires_grad, self.device)
        else:
            self._node = None

    # ------------------------------------------------------------------ attributes
    @property
    def op(self):
        return self._node.op if self._node else OpEnum.LEAF

    @property
    def requires_grad(self) -> bool:
        return bool(self._node.requires_grad) if self._node else False

    @property
    def shape(self):
        return tuple(self._node.shape) if self._node else None

    @property
    def grad(self):
        g = self._node.grad if self._node else None
        return Tensor(_node=g, device=self.device) if g else None

    # ------------------------------------------------------------------ graph building
    def _wrap(self, node: Node) -> "Tensor":
        return Tensor(_node=node, device=self.device)

    def _coerce(self, other) -> "Tensor":
        """Scalars and arrays become leaves on this tensor's device; tensors must already be there."""
        if not isinstance(other, Tensor):
            return Tensor(other, device=self.device)
        if other.device.type != self.device.type:
            raise DeviceMismatchError('Cannot mix devices in operation. | Got: "' + other.device.type.name + '"')
        return other

    def _binary(self, op, other, swapped: bool = False) -> "Tensor":
        other = self._coerce(other)
        pair = [other._node, self._node] if swapped else [self._node, other._node]
        return self._wrap(Node(op, pair, self.device))

    def _unary(self, op) -> "Tensor":
        return self._wrap(Node(op, [self._node], self.device))

    def __add__(self, other): return self._binary(OpEnum.ADD, other)
    def __radd__(self, other): return self._binary(OpEnum.ADD, other)
    def __sub__(self, other): return self._binary(OpEnum.SUB, other)
    def __rsub__(self, other): return self._binary(OpEnum.SUB, other, swapped=True)
    def __mul__(self, other): return self._binary(OpEnum.MUL, other)
    def __rmul__(self, other): return self._binary(OpEnum.MUL, other)
    def __truediv__(self, other): return self._binary(OpEnum.DIV, other)
    def __rtruediv__(self, other): return self._binary(OpEnum.DIV, other, swapped=True)
    def __pow__(self, exponent): return self._binary(OpEnum.POW, exponent)
    def __neg__(self): return self._unary(OpEnum.NEG)

    def __matmul__(self, other):
        if not isinstance(other, Tensor):
            raise TypeError("Matmul requires both operands to be Tensors.")
        if other.device.type != self.device.type:
            raise DeviceMismatchError("Cannot perform MATMUL across different devices")
        return self._wrap(Node(OpEnum.MATMUL, [self._node, other._node], self.device))

    def exp(self): return self._wrap(backend.exp(self._node))
    def sin(self): return self._wrap(backend.sin(self._node))
    def cos(self): return self._wrap(backend.cos(self._node))
    def log(self): return self._wrap(extra.log(self._node)) if extra is not None else self._unary(OpEnum.LOG)

    def sum(self, axes: Sequence[int] = (), keepdims: bool = False) -> "Tensor":
        """Sum over ``axes`` (all axes when empty), as ``ormi::ops::sum``."""
        return self._wrap(backend.sum(self._node, list(axes), keepdims))

    # ------------------------------------------------------------------ views
    def reshape(self, shape: Sequence[int]) -> "Tensor":
        return self._wrap(backend.reshape(self._node, list(shape)))

    def transpose(self, axes: Sequence[int] | None = None) -> "Tensor":
        order = list(axes) if axes is not None else list(range(len(self.shape)))[::-1]
        return self._wrap(backend.transpose(self._node, order))

    def expand(self, shape: Sequence[int]) -> "Tensor":
        return self._wrap(backend.expand(self._node, list(shape)))

    # ------------------------------------------------------------------ execution
    def realize(self) -> "Tensor":
        if self._node is not None and not self._node.is_realized:
            backend.execute_graph(self._node)
        return self

    def numpy(self) -> np.ndarray:
        self.realize()
        if self._node is None or not self._node.is_realized:
            raise RuntimeError("Cannot fetch an unrealized tensor.")
        flat = backend.buffer_to_numpy(self._node.data)
        strides = tuple(4 * s for s in self._node.view.strides)      # the view's strides are in elements
        return np.lib.stride_tricks.as_strided(flat, shape=self.shape, strides=strides)

    def backward(self) -> None:
        if not self.requires_grad:
            raise RuntimeError("Cannot call backward() on a tensor that does not require gradients.")
        backend.compute_gradients(self._node)

    def zero_grad(self) -> None:
        if self._node is not None:
            self._node.grad = None

    def zero_grad_graph(self) -> None:
        if self._node is not None:
            backend.zero_grad_graph(self._node)

    def __repr__(self) -> str:
        state = "realized" if self._node is not None and self._node.is_realized else "lazy"
        return f"Tensor(op={self.op.name}, shape={self.shape}, state={state}, device={self.device.type.name})"
