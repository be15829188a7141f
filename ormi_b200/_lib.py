"""ctypes binding of the C ABI declared in include/ormi_b200.h.

The library is the product: when it is missing, or does not export an entry point the header
declares, importing this module raises — there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
import re

from .graph import CNode

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libormi_b200.so")
HEADER = os.path.join(os.path.dirname(_HERE), "include", "ormi_b200.h")

c_int, c_size_t, c_void_p, c_char_p = ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_char_p
P = ctypes.POINTER

_SIGNATURES = {
    "ormi_b200_init": (c_int, [c_int, P(c_void_p)]),
    "ormi_b200_shutdown": (c_int, [c_void_p]),
    "ormi_b200_last_error": (c_char_p, []),
    "ormi_b200_alloc": (c_int, [c_void_p, c_size_t, P(c_void_p)]),
    "ormi_b200_free": (c_int, [c_void_p, c_void_p, c_size_t]),
    "ormi_b200_trim": (c_int, [c_void_p]),
    "ormi_b200_memset": (c_int, [c_void_p, c_void_p, c_int, c_size_t]),
    "ormi_b200_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ormi_b200_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ormi_b200_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ormi_b200_memcpy_h2d_async": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_int]),
    "ormi_b200_memcpy_d2h_async": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t]),
    "ormi_b200_copy_wait": (c_int, [c_void_p, c_int]),
    "ormi_b200_upload_mark": (c_int, [c_void_p, c_int]),
    "ormi_b200_upload_wait": (c_int, [c_void_p, c_int]),
    "ormi_b200_fill_u32": (c_int, [c_void_p, c_void_p, ctypes.c_uint32, c_size_t]),
    "ormi_b200_fill_u8": (c_int, [c_void_p, c_void_p, ctypes.c_uint8, c_size_t]),
    "ormi_b200_sync": (c_int, [c_void_p]),
    "ormi_b200_stream": (c_void_p, [c_void_p]),
    "ormi_b200_realize": (c_int, [c_void_p, P(CNode), c_int, P(ctypes.c_int), c_int]),
    "ormi_b200_plan_json": (c_int, [P(CNode), c_int, P(ctypes.c_int), c_int, c_char_p, c_size_t, P(c_size_t)]),
    "ormi_b200_plan_json_opts": (c_int, [P(CNode), c_int, P(ctypes.c_int), c_int, c_char_p, c_char_p, c_size_t, P(c_size_t)]),
    "ormi_b200_compile_source": (c_int, [P(CNode), c_int, c_int, c_char_p, c_size_t, P(c_size_t), P(ctypes.c_int), c_int, P(ctypes.c_int)]),
    "ormi_b200_set_lowering": (c_int, [c_int, c_char_p]),
    "ormi_b200_compile_cubin": (c_int, [c_char_p, c_char_p, c_size_t, P(c_size_t)]),
    "ormi_b200_sum": (c_int, [c_void_p, c_void_p, c_int, P(ctypes.c_int32), P(ctypes.c_int32), P(ctypes.c_int32), c_int, c_void_p]),
    "ormi_b200_matmul": (c_int, [c_void_p, c_void_p, c_int, P(ctypes.c_int32), P(ctypes.c_int32),
                                 c_void_p, c_int, P(ctypes.c_int32), P(ctypes.c_int32), c_void_p, c_int, P(ctypes.c_int32)]),
    "ormi_b200_colsum_static": (c_int, [c_void_p, ctypes.c_int64, ctypes.c_int64, c_void_p, c_void_p]),
    "ormi_b200_cvt_bf16_kmajor": (c_int, [c_void_p, c_void_p, ctypes.c_int64, ctypes.c_int64, c_int, c_int, c_void_p]),
    "ormi_b200_gemm_bf16_kmajor": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int]),
    "ormi_b200_cvt_bf16": (c_int, [c_void_p, c_void_p, ctypes.c_int64, c_int, c_int, c_void_p]),
    "ormi_b200_gemm_bf16": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int]),
    "ormi_b200_comm_unique_id": (c_int, [c_char_p]),
    "ormi_b200_comm_init": (c_int, [c_void_p, c_char_p, c_int, c_int]),
    "ormi_b200_allreduce_sum_f32": (c_int, [c_void_p, P(c_void_p), P(c_size_t), c_int, c_int]),
    "ormi_b200_comm_join": (c_int, [c_void_p]),
    "ormi_b200_comm_mark": (c_int, [c_void_p, c_int]),
    "ormi_b200_comm_wait": (c_int, [c_void_p, c_int]),
    "ormi_b200_comm_destroy": (c_int, [c_void_p]),
    "ormi_b200_selftest_wait_timeout": (c_int, [c_void_p, c_int]),
    "ormi_b200_set_option": (c_int, [c_void_p, c_char_p, c_char_p]),
    "ormi_b200_get_counter": (c_int, [c_void_p, c_char_p, P(ctypes.c_int64)]),
    "ormi_b200_capture_begin": (c_int, [c_void_p]),
    "ormi_b200_capture_end": (c_int, [c_void_p, P(c_void_p)]),
    "ormi_b200_graph_launch": (c_int, [c_void_p, c_void_p]),
    "ormi_b200_graph_destroy": (c_int, [c_void_p, c_void_p]),
}


def declared_symbols() -> list[str]:
    """Entry points the public header declares."""
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ormi_b200_[a-z0-9_]+)\s*\(", text)))


def load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m ormi_b200.build` (needs nvcc); "
                          "there is no fallback implementation")
    lib = ctypes.CDLL(LIB_PATH, mode=os.RTLD_LOCAL | os.RTLD_NOW)
    for name in declared_symbols():
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}, which include/ormi_b200.h declares")
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


lib = load()


class BackendError(RuntimeError):
    """A non-zero return of the C ABI (the C++ seams raise std::runtime_error for the same)."""


def check(rc: int):
    if rc != 0:
        raise BackendError(lib.ormi_b200_last_error().decode(errors="replace"))
