"""TEST INFRASTRUCTURE — Python access to the two CPU checkers.

* ``ref_*``   the unmodified reference engine compiled into ``oracle/_ref/libormi_ref.so``
              (see ``oracle/Makefile`` and ``oracle/ref_driver.cpp``);
* ``port_*``  the C restatement ``oracle/ormi_oracle.c`` (``oracle/libormi_oracle.so``).

Only ``tests/``, the smoke test and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Sequence

import numpy as np

from ormi_b200 import graph as G

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_LIB = os.path.join(_HERE, "_ref", "libormi_ref.so")
PORT_LIB = os.path.join(_HERE, "libormi_oracle.so")
_ref = None
_port = None


def build(verbose=False):
    """Runs the Makefile: always builds the restatement, and the reference library when the reference
    checkout is present on this machine."""
    cmd = ["make", "-C", _HERE]
    if os.environ.get("ORMI_REFERENCE"):
        cmd.append("REF=" + os.environ["ORMI_REFERENCE"])
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if verbose:
        print(out.stdout)


def ref_available() -> bool:
    return os.path.exists(REF_LIB)


def locate_openblas() -> None:
    """Points the cblas shim (ORMI_ORACLE_OPENBLAS) at an OpenBLAS inside the running interpreter's wheels — scipy's or
    opencv's — unless the caller already chose one.  The reference's own dependency is an un-pinned system OpenBLAS."""
    if os.environ.get("ORMI_ORACLE_OPENBLAS"):
        return
    import glob
    import sysconfig
    site = sysconfig.get_paths()["purelib"]
    for pattern in ("scipy.libs/libscipy_openblas*.so", "opencv_python_headless.libs/libopenblas*.so", "numpy.libs/libscipy_openblas*.so"):
        hits = sorted(glob.glob(os.path.join(site, pattern)))
        if hits:
            os.environ["ORMI_ORACLE_OPENBLAS"] = hits[0]
            return


def _load_ref():
    global _ref
    if _ref is None:
        if not ref_available():
            raise RuntimeError(f"{REF_LIB} is missing: run `make -C oracle` on a machine with the reference checkout")
        locate_openblas()
        _ref = ctypes.CDLL(REF_LIB, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        _ref.oracle_ref_last_error.restype = ctypes.c_char_p
        _ref.oracle_ref_blas.restype = ctypes.c_char_p
    return _ref


def _load_port():
    global _port
    if _port is None:
        if not os.path.exists(PORT_LIB):
            build()
        _port = ctypes.CDLL(PORT_LIB, mode=os.RTLD_LOCAL | os.RTLD_NOW)
        _port.oracle_port_last_error.restype = ctypes.c_char_p
    return _port


def ref_blas() -> tuple[str, int]:
    lib = _load_ref()
    return lib.oracle_ref_blas().decode(), int(lib.oracle_ref_blas_threads())


def _i32(values):
    return (ctypes.c_int32 * max(1, len(values)))(*values)


def _prepare_ref(seeds, backward_root, outputs):
    roots = [n for n, _ in outputs] + [n for n, _ in seeds] + [l for _, l in seeds]
    if backward_root is not None:
        roots.append(backward_root)
    arr, order, _ = G.flatten(roots, host_pointers=True, stop_at_realized=False)
    index = {id(n): i for i, n in enumerate(order)}
    seed_nodes = _i32([index[id(n)] for n, _ in seeds])
    seed_leaves = _i32([index[id(l)] for _, l in seeds])
    out_nodes = _i32([index[id(n)] for n, _ in outputs])
    out_kinds = _i32([1 if k == "grad" else 0 for _, k in outputs])
    broot = index[id(backward_root)] if backward_root is not None else -1
    return arr, order, seed_nodes, seed_leaves, out_nodes, out_kinds, broot


def _collect(n_out, caps, run):
    bufs = [np.empty(c, dtype=np.float32) for c in caps]
    ptrs = (ctypes.POINTER(ctypes.c_float) * n_out)(*[b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) for b in bufs])
    cap_arr = (ctypes.c_int64 * n_out)(*caps)
    ndim = (ctypes.c_int32 * n_out)()
    shape = (ctypes.c_int32 * (n_out * G.MAX_DIMS))()
    secs = ctypes.c_double(0.0)
    run(ptrs, cap_arr, ndim, shape, ctypes.byref(secs))
    outs = []
    for i in range(n_out):
        shp = [shape[i * G.MAX_DIMS + d] for d in range(ndim[i])]
        outs.append(bufs[i][: G.numel(shp)].reshape(shp).copy())
    return outs, secs.value


def ref_run(outputs: Sequence[tuple[G.Node, str]], seeds: Sequence[tuple[G.Node, G.Node]] = (),
            backward_root: G.Node | None = None, caps: Sequence[int] | None = None):
    """Runs a FORWARD graph (host-data leaves, nodes built with ormi_b200.graph) on the reference CPU backend.

    ``outputs``: (node, "value" | "grad"); ``seeds``: (node, leaf) pairs meaning ``node.grad = leaf`` before
    ``compute_gradients(backward_root)``.  The Python-side ``grad`` fields are ignored: the reference's own
    autograd builds the backward graph.  Returns (list of arrays, seconds spent in autograd + realize).
    """
    lib = _load_ref()
    arr, order, sn, sl, on, ok, broot = _prepare_ref(seeds, backward_root, outputs)
    if caps is None:
        caps = [max(n.numel() for n in order)] * len(outputs)

    def run(ptrs, cap_arr, ndim, shape, secs):
        rc = lib.oracle_ref_run(arr, len(order), sn, sl, len(seeds), broot, on, ok, len(outputs),
                                ptrs, cap_arr, ndim, shape, secs)
        if rc != 0:
            raise RuntimeError("reference: " + lib.oracle_ref_last_error().decode())

    return _collect(len(outputs), list(caps), run)


def ref_export(outputs, seeds=(), backward_root=None, cap=4096):
    """The graph the reference's autograd builds for the same request, flattened.
    Returns (CNode array, n, origin list, created-leaf fill values, output indices, forward order)."""
    lib = _load_ref()
    arr, order, sn, sl, on, ok, broot = _prepare_ref(seeds, backward_root, outputs)
    exp = (G.CNode * cap)()
    n_exp = ctypes.c_int32(0)
    origin = (ctypes.c_int32 * cap)()
    leaf_val = (ctypes.c_float * cap)()
    out_index = (ctypes.c_int32 * max(1, len(outputs)))()
    rc = lib.oracle_ref_export(arr, len(order), sn, sl, len(seeds), broot, on, ok, len(outputs),
                               exp, cap, ctypes.byref(n_exp), origin, leaf_val, out_index)
    if rc != 0:
        raise RuntimeError("reference: " + lib.oracle_ref_last_error().decode())
    n = n_exp.value
    return exp, n, list(origin[:n]), list(leaf_val[:n]), list(out_index[: len(outputs)]), order


def port_run(outputs: Sequence[G.Node]):
    """Realizes ``outputs`` (already-expanded graph: forward and, if wanted, autograd nodes built by
    ormi_b200.graph) with the C restatement.  Returns (list of arrays, seconds)."""
    lib = _load_port()
    arr, order, roots = G.flatten(list(outputs), host_pointers=True, stop_at_realized=True)
    on = _i32(roots)
    caps = [max(1, n.numel()) for n in outputs]

    def run(ptrs, cap_arr, ndim, shape, secs):
        rc = lib.oracle_port_run(arr, len(order), on, len(outputs), ptrs, cap_arr, ndim, shape, secs)
        if rc != 0:
            raise RuntimeError("oracle port: " + lib.oracle_port_last_error().decode())

    return _collect(len(outputs), caps, run)
