"""The allocation-free column sum (ormi_b200_colsum_static), checked against the pooled ormi_b200_sum.

This file is collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It builds its own context, so it passes alone in a fresh process as well as after the others.
"""
import ctypes

import numpy as np
import pytest

from ormi_b200 import workloads as W

pytestmark = pytest.mark.gpu

TOL = 1e-5      # same bound as the other fp32 reduction tests: max|a - b| <= TOL * max|b|


def _pooled_colsum(dev, lib, check, src_ptr, rows, cols):
    out = dev.buffer([cols])
    shape = (ctypes.c_int32 * 2)(rows, cols)
    strides = (ctypes.c_int32 * 2)(cols, 1)
    axes = (ctypes.c_int32 * 1)(0)
    check(lib.ormi_b200_sum(dev.handle, ctypes.c_void_p(src_ptr), 2, shape, strides, axes, 1, ctypes.c_void_p(out.dev_ptr)))
    return dev.download(out)


def test_static_scratch_colsum_matches_pooled_sum_twice_in_a_row():
    from ormi_b200._lib import lib, check
    from ormi_b200.runtime import Device
    dev = Device(0)
    try:
        # two calls in a row that use the shared scratch differently: the second is smaller, so stale partial rows
        # of the first call are still lying in the array when it runs
        for seed, (rows, cols) in enumerate([(3000, 4096), (517, 1000)]):
            host = W.normal(seed, (rows, cols))
            src = dev.upload(host)
            dst = dev.buffer([cols])
            check(lib.ormi_b200_colsum_static(ctypes.c_void_p(src.dev_ptr), rows, cols, ctypes.c_void_p(dst.dev_ptr),
                                              ctypes.c_void_p(dev.stream)))
            got = dev.download(dst)
            want = _pooled_colsum(dev, lib, check, src.dev_ptr, rows, cols)
            scale = np.abs(want).max()
            assert np.abs(got - want).max() <= TOL * scale
            assert np.abs(got - host.sum(axis=0, dtype=np.float64)).max() <= TOL * scale
        # beyond the fixed scratch: refused with a clear message, nothing launched
        big = dev.buffer([4])
        rc = lib.ormi_b200_colsum_static(ctypes.c_void_p(big.dev_ptr), 1, 65537, ctypes.c_void_p(big.dev_ptr), None)
        assert rc != 0 and b"exceed the fixed scratch" in lib.ormi_b200_last_error()
    finally:
        dev.close()
