"""The run-time compiled tensor-core GEMM on bf16 operands in their own row-major layouts, through the C ABI
(ormi_b200_cvt_bf16 / ormi_b200_gemm_bf16): every operand layout, one SM and a pair of SMs per MMA, ragged shapes.

Two checks per case: operands that are exactly representable in bf16 (small integers) must give the fp32 product bit
for bit — a wrong descriptor, swizzle or tile coordinate cannot hide behind a tolerance — and N(0, 1/sqrt(K))
operands are compared with the CPU oracle's fp32 matmul within the bf16 tolerance of 2e-2.
"""
import ctypes
import math

import numpy as np
import pytest

from ormi_b200 import graph as G
from ormi_b200 import workloads as W
from oracle import oracle as O

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2


def rel(a, b):
    return float(np.abs(a - b).max() / max(1e-30, np.abs(b).max()))


def run_gemm(dev, a, b, ta, tb):
    """a [M,K], b [K,N] fp32 on the host; the device gets them stored plain (0) or transposed (1)."""
    from ormi_b200._lib import lib, check
    M, K = a.shape
    N = b.shape[1]
    sa = np.ascontiguousarray(a.T) if ta else a
    sb = np.ascontiguousarray(b.T) if tb else b
    da, db = dev.upload(sa), dev.upload(sb)
    a16, b16, c = dev.alloc(sa.size * 2), dev.alloc(sb.size * 2), dev.buffer([M, N])
    try:
        check(lib.ormi_b200_cvt_bf16(dev.handle, ctypes.c_void_p(da.dev_ptr), sa.shape[1], sa.shape[0], sa.shape[1], ctypes.c_void_p(a16)))
        check(lib.ormi_b200_cvt_bf16(dev.handle, ctypes.c_void_p(db.dev_ptr), sb.shape[1], sb.shape[0], sb.shape[1], ctypes.c_void_p(b16)))
        check(lib.ormi_b200_gemm_bf16(dev.handle, ctypes.c_void_p(a16), ta, ctypes.c_void_p(b16), tb, ctypes.c_void_p(c.dev_ptr), M, N, K))
        return dev.download(c)
    finally:
        dev.free(a16, sa.size * 2)
        dev.free(b16, sb.size * 2)


@pytest.mark.parametrize("pair", ["off", "on"])
@pytest.mark.parametrize("mnk", [(128, 256, 64), (256, 256, 128), (512, 768, 320), (1024, 1024, 1024), (264, 520, 200),
                                 (8, 4096, 64), (2048, 64, 1504), (1000, 1256, 72)])
def test_every_operand_layout_is_exact_on_integers(pair, mnk):
    from ormi_b200.runtime import Device
    M, N, K = mnk
    dev = Device(0)
    try:
        dev.set_option("tc_pair", pair)
        ai = np.random.default_rng(0).integers(-4, 5, size=(M, K)).astype(np.float32)
        bi = np.random.default_rng(1).integers(-4, 5, size=(K, N)).astype(np.float32)
        want = ai @ bi
        for ta in (0, 1):
            for tb in (0, 1):
                if (ta and M % 8) or (not ta and K % 8) or (tb and K % 8) or (not tb and N % 8):
                    continue                     # the contiguous dimension of a bf16 operand must be a multiple of 8
                got = run_gemm(dev, ai, bi, ta, tb)
                assert np.array_equal(got, want), (ta, tb, float(np.abs(got - want).max()))
        dev.sync()
    finally:
        dev.close()


@pytest.mark.parametrize("mnk", [(2048, 2048, 2048), (4096, 1024, 4096), (8192, 8192, 8192)])
def test_against_the_oracle_matmul(device, mnk):
    """configs[2] shapes: the oracle's fp32 matmul (cblas_sgemm of the reference CPU backend) on the same operands.
    At 8192^3 the oracle computes a slice of 256 rows of C, so that its loop fallback stays usable."""
    M, N, K = mnk
    a = W.normal(0, (M, K), 1 / math.sqrt(K))
    b = W.normal(1, (K, N), 1 / math.sqrt(K))
    got = run_gemm(device, a, b, 0, 0)
    rows = slice(0, M) if M * N * K <= 2 ** 35 else slice(M // 2 - 128, M // 2 + 128)
    root = G.matmul(G.leaf(a[rows]), G.leaf(b))
    (want,), _ = O.ref_run([(root, "value")]) if O.ref_available() else O.port_run([root])
    assert rel(got[rows], want) <= BF16_TOL
    # and tighter than the tolerance asks: bf16 rounding of the operands alone gives about 3e-3
    assert rel(got[rows], want) <= 6e-3
