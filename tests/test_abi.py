"""The C-ABI library: loads, exports every symbol the public header declares, and behaves without a GPU."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from ormi_b200 import _lib
from ormi_b200 import graph as G
from ormi_b200 import runtime as RT

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    names = _lib.declared_symbols()
    assert len(names) >= 20
    out = subprocess.run(["nm", "-D", "--defined-only", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if line.strip()}
    missing = [n for n in names if n not in exported]
    assert not missing, missing
    assert set(names) <= set(_lib._SIGNATURES) | set(), sorted(set(names) - set(_lib._SIGNATURES))


def test_library_has_no_link_time_dependency_on_the_oracle_or_the_driver():
    out = subprocess.run(["readelf", "-d", _lib.LIB_PATH], capture_output=True, text=True, check=True).stdout
    needed = [l for l in out.splitlines() if "NEEDED" in l]
    assert not any("oracle" in l or "ormi_ref" in l for l in needed)
    assert not any("libcuda.so" in l for l in needed)      # the driver is reached through the runtime at init


def test_compile_source_matches_the_reference_compiler_contract():
    """ormi-core/csrc/tests/backend/cuda/test_compiler.cpp:43-86 greps the generated source for these."""
    a = G.leaf(np.zeros((2, 2), np.float32))
    b = G.leaf(np.zeros((2, 2), np.float32))

    def compile_(root):
        arr, order, roots = G.flatten([root], host_pointers=True)
        n = ctypes.c_size_t()
        buf = ctypes.create_string_buffer(1 << 16)
        leaves = (ctypes.c_int * 16)()
        nl = ctypes.c_int()
        rc = _lib.lib.ormi_b200_compile_source(arr, len(order), roots[0], buf, len(buf), ctypes.byref(n), leaves, 16, ctypes.byref(nl))
        return rc, buf.value.decode(), nl.value

    rc, src, nl = compile_(G.add(a, b))
    assert rc == 0 and nl == 2
    assert 'extern "C" __global__' in src and "void fused_kernel(float* OUT_Z" in src and "if (idx >= 4) return;" in src
    rc, src, nl = compile_(G.add(a, a))
    assert rc == 0 and nl == 1 and "val_LEAF_0 + val_LEAF_0" in src
    rc, src, _ = compile_(G.sin(a))
    assert rc == 0 and "sinf(" in src
    assert RT.compile_cubin(src) > 0
    rc, _, _ = compile_(G.matmul(a, b))
    assert rc != 0 and b"MATMUL" in _lib.lib.ormi_b200_last_error()


def test_nvrtc_errors_are_reported():
    n = ctypes.c_size_t()
    rc = _lib.lib.ormi_b200_compile_cubin(b"this is not CUDA", None, 0, ctypes.byref(n))
    assert rc != 0 and b"NVRTC" in _lib.lib.ormi_b200_last_error()


def test_scheduling_errors_are_reported():
    bad = (G.CNode * 2)()
    bad[0].op = int(G.OpEnum.LEAF)      # leaf without data
    bad[1].op = int(G.OpEnum.NEG); bad[1].n_parents = 1; bad[1].parents[0] = 0
    roots = (ctypes.c_int * 1)(1)
    n = ctypes.c_size_t()
    buf = ctypes.create_string_buffer(4096)
    assert _lib.lib.ormi_b200_plan_json(bad, 2, roots, 1, buf, 4096, ctypes.byref(n)) == 0
    assert b"leaf without data" in buf.value


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_init_fails_loudly_without_a_gpu():
    """No CPU fallback: without a device the context cannot be created (the reference's tests detect CUDA
    through the same failure, ormi-core/csrc/tests/test_utils.h:17-21)."""
    handle = ctypes.c_void_p()
    assert _lib.lib.ormi_b200_init(0, ctypes.byref(handle)) != 0
    assert b"CUDA Error" in _lib.lib.ormi_b200_last_error()
    with pytest.raises(_lib.BackendError):
        RT.Device(0)
