"""Realizing graphs on a B200 through the C ABI: the Python counterpart of ormi_backend.execute_graph,
numpy_to_buffer and buffer_to_numpy (ormi-core/csrc/bindings/main.cpp:33, bind_memory.cpp:10-60)."""
from __future__ import annotations

import ctypes
import json
from typing import Sequence

import numpy as np

from . import graph as G
from ._lib import lib, check


class Device:
    """One GPU: context, stream and buffer pool behind ``ormi_b200_init``."""

    def __init__(self, index: int = 0):
        handle = ctypes.c_void_p()
        check(lib.ormi_b200_init(index, ctypes.byref(handle)))
        self.handle = handle
        self.index = index
        self._options: dict[str, str] = {}

    def close(self):
        if self.handle:
            lib.ormi_b200_shutdown(self.handle)
            self.handle = None

    # ---- memory (IAllocator surface)
    def alloc(self, nbytes: int) -> int:
        p = ctypes.c_void_p()
        check(lib.ormi_b200_alloc(self.handle, nbytes, ctypes.byref(p)))
        return p.value

    def free(self, ptr: int, nbytes: int):
        if self.handle:
            check(lib.ormi_b200_free(self.handle, ctypes.c_void_p(ptr), nbytes))

    def h2d(self, ptr: int, array: np.ndarray):
        check(lib.ormi_b200_memcpy_h2d(self.handle, ctypes.c_void_p(ptr), array.ctypes.data_as(ctypes.c_void_p), array.nbytes))

    def d2h(self, array: np.ndarray, ptr: int):
        check(lib.ormi_b200_memcpy_d2h(self.handle, array.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(ptr), array.nbytes))

    def h2d_async(self, ptr: int, array: np.ndarray, after_compute: bool = True):
        """Upload from pinned host memory on the upload stream; pair with ``copy_wait(0)`` before the kernels that read it."""
        check(lib.ormi_b200_memcpy_h2d_async(self.handle, ctypes.c_void_p(ptr), array.ctypes.data_as(ctypes.c_void_p), array.nbytes,
                                             1 if after_compute else 0))

    def d2h_async(self, array: np.ndarray, ptr: int):
        """Download into pinned host memory on the download stream, behind the kernels queued so far; ``copy_wait(1)`` waits."""
        check(lib.ormi_b200_memcpy_d2h_async(self.handle, array.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(ptr), array.nbytes))

    def copy_wait(self, direction: int):
        check(lib.ormi_b200_copy_wait(self.handle, direction))

    def upload_mark(self, slot: int):
        """Remembers the upload stream's tail (the uploads queued so far) in one of 32 slots."""
        check(lib.ormi_b200_upload_mark(self.handle, slot))

    def upload_wait(self, slot: int):
        """The compute stream waits for the uploads that were queued when ``upload_mark(slot)`` was called, no later ones."""
        check(lib.ormi_b200_upload_wait(self.handle, slot))

    def sync(self):
        check(lib.ormi_b200_sync(self.handle))

    def set_option(self, key: str, value: str):
        check(lib.ormi_b200_set_option(self.handle, key.encode(), value.encode()))
        self._options[key] = value

    def get_option(self, key: str) -> str:
        """The value last set through this object (the defaults: "matmul" "fp32", "fusion" "on", "tc_pair" "on", "intermediates" "keep")."""
        return self._options.get(key, {"matmul": "fp32", "fusion": "on", "tc_pair": "on", "intermediates": "keep"}.get(key, ""))

    def capture(self):
        """``with dev.capture() as step: ...`` records what the block queues on the compute stream (realize calls, raw
        matmuls) instead of running it; afterwards ``step.launch()`` replays it with one call and ``step.destroy()`` gives
        its buffers back.  Run the block once before capturing it.  Results obtained inside the block stay valid (and are
        rewritten by every replay) until the step is destroyed."""
        return CapturedStep(self)

    def counter(self, name: str) -> int:
        v = ctypes.c_int64()
        check(lib.ormi_b200_get_counter(self.handle, name.encode(), ctypes.byref(v)))
        return v.value

    @property
    def stream(self) -> int:
        return lib.ormi_b200_stream(self.handle) or 0

    # ---- buffers
    def buffer(self, shape) -> G.Buffer:
        buf = G.Buffer(shape)
        buf.dev_ptr = self.alloc(max(4, buf.nbytes))
        buf._release = self.free
        return buf

    def upload(self, array) -> G.Buffer:
        """numpy_to_buffer: a device buffer holding ``array`` (fp32, C order)."""
        arr = np.asarray(array, dtype=np.float32)
        arr = np.ascontiguousarray(arr).reshape(arr.shape)
        buf = self.buffer(arr.shape)
        if arr.nbytes:
            self.h2d(buf.dev_ptr, arr)
        return buf

    def leaf(self, array, requires_grad=False) -> G.Node:
        return G.Node(G.OpEnum.LEAF, data=self.upload(array), requires_grad=requires_grad)

    def const(self, value: float) -> G.Node:
        return self.leaf(np.float32(value))

    def download(self, buf: G.Buffer) -> np.ndarray:
        """buffer_to_numpy: the raw buffer in its own (contiguous) shape."""
        out = np.empty(buf.shape, dtype=np.float32)
        if out.nbytes:
            self.d2h(out, buf.dev_ptr)
        return out

    def ensure_on_device(self, nodes: Sequence[G.Node]):
        for n in nodes:
            if n.is_realized and n.data.dev_ptr is None:
                if n.data.host is None:
                    raise RuntimeError("realized node without data")
                up = self.upload(n.data.host)
                n.data.dev_ptr, n.data._release = up.dev_ptr, up._release
                up._release = None

    # ---- realize
    def realize(self, roots: Sequence[G.Node]):
        """execute_graph for several roots at once.  Every root (and every node the scheduler chose to
        write to memory) ends up realized, with a device buffer attached."""
        roots = [r for r in roots]
        pending = [r for r in roots if not r.is_realized]
        if not pending:
            return
        order = G.topo_order(pending, stop_at_realized=True)
        self.ensure_on_device(order)
        arr, order, root_idx = G.flatten(pending, host_pointers=False, stop_at_realized=True)
        ridx = (ctypes.c_int * len(root_idx))(*root_idx)
        check(lib.ormi_b200_realize(self.handle, arr, len(order), ridx, len(root_idx)))
        base_of = {}
        for i, n in enumerate(order):
            c = arr[i]
            if n.is_realized or not c.data:
                continue
            if c.flags & G.NODE_OWNED:
                buf = G.Buffer(n.shape if c.data_bytes == 4 * max(1, n.numel()) or c.flags & G.NODE_BF16 else [c.data_bytes // 4])
                buf.dev_ptr, buf._release = c.data, self.free
                buf.nbytes = c.data_bytes
                n.bf16 = bool(c.flags & G.NODE_BF16)       # came back as a bf16 matrix: from now on a matmul operand only
                n.data = buf
                base_of[c.data] = buf
        for i, n in enumerate(order):
            c = arr[i]
            if not n.is_realized and c.data and (c.flags & G.NODE_ALIAS):
                n.data = base_of.get(c.data) or _find_buffer(order, c.data)

    def numpy(self, node: G.Node) -> np.ndarray:
        """Tensor.numpy(): realize, copy the buffer to the host and apply the node's view strides
        (ormi-core/src/ormi_core/tensor.py:165-174)."""
        self.realize([node])
        if node.bf16:                                  # a bf16 tensor: widen on the host (exact)
            half = np.empty(node.data.nbytes // 2, dtype=np.uint16)
            self.d2h(half, node.data.dev_ptr)
            return (half.astype(np.uint32) << 16).view(np.float32).reshape(node.shape)
        raw = np.empty(node.data.nbytes // 4, dtype=np.float32)
        self.d2h(raw, node.data.dev_ptr)
        if not node.shape:
            return raw[:1].reshape(()).copy()
        return np.lib.stride_tricks.as_strided(raw, shape=node.shape, strides=[4 * s for s in node.strides]).copy()


def _find_buffer(order, ptr):
    for n in order:
        if n.data is not None and n.data.dev_ptr == ptr:
            return n.data
    raise RuntimeError("alias of an unknown buffer")


class CapturedStep:
    """A step recorded by ``Device.capture()`` (ormi_b200_capture_begin / _end / ormi_b200_graph_launch)."""

    def __init__(self, dev: "Device"):
        self.dev, self.handle = dev, None

    def __enter__(self):
        check(lib.ormi_b200_capture_begin(self.dev.handle))
        return self

    def __exit__(self, exc_type, exc, tb):
        g = ctypes.c_void_p()
        rc = lib.ormi_b200_capture_end(self.dev.handle, ctypes.byref(g))
        if exc_type is None:
            check(rc)
            self.handle = g
        elif rc == 0:
            lib.ormi_b200_graph_destroy(self.dev.handle, g)
        return False

    def launch(self):
        check(lib.ormi_b200_graph_launch(self.dev.handle, self.handle))

    def destroy(self):
        if self.handle is not None and self.dev.handle:
            check(lib.ormi_b200_graph_destroy(self.dev.handle, self.handle))
        self.handle = None


def plan(roots: Sequence[G.Node], host_pointers=True, options: str = "") -> dict:
    """The schedule the backend would run for ``roots`` (needs no GPU).  ``options``: "matmul=bf16,fusion=on,..."."""
    arr, order, root_idx = G.flatten(list(roots), host_pointers=host_pointers, stop_at_realized=True)
    ridx = (ctypes.c_int * len(root_idx))(*root_idx)
    n = ctypes.c_size_t()
    opts = options.encode()
    check(lib.ormi_b200_plan_json_opts(arr, len(order), ridx, len(root_idx), opts, None, 0, ctypes.byref(n)))
    buf = ctypes.create_string_buffer(n.value + 1)
    check(lib.ormi_b200_plan_json_opts(arr, len(order), ridx, len(root_idx), opts, buf, n.value + 1, ctypes.byref(n)))
    out = json.loads(buf.value.decode())
    out["order"] = order
    out["roots"] = root_idx
    return out


def compile_cubin(source: str) -> int:
    """NVRTC-compiles ``source`` for sm_100a; returns the cubin size.  Needs no GPU."""
    n = ctypes.c_size_t()
    check(lib.ormi_b200_compile_cubin(source.encode(), None, 0, ctypes.byref(n)))
    return n.value
