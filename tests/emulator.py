"""TEST INFRASTRUCTURE: executes a schedule (ormi_b200.runtime.plan) on the CPU.

Every generated kernel is compiled unchanged with g++ against tests/cuda_emul.h and launched with its
real grid/block geometry; GEMM steps are computed with numpy — for a step of the tensor-core kernel, on operands
rounded to bf16 (taken from the bf16 twin an earlier step wrote, when the plan says so), followed by the step's
generated epilogue, compiled from the same text the kernel template receives.  This checks the scheduler and the
code generator against the oracle without a GPU.  It is not a fallback: nothing in the package imports it.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE = os.path.join(tempfile.gettempdir(), "ormi_b200_emul")


def _compile(sources: list[tuple[str, str]]):
    os.makedirs(_CACHE, exist_ok=True)
    text = '#define ORMI_EMULATE 1\n#include "cuda_emul.h"\n' + "\n".join(src for _, src in sources)
    tag = hashlib.sha1(text.encode()).hexdigest()[:16]
    so = os.path.join(_CACHE, f"k_{tag}.so")
    if not os.path.exists(so):
        cpp = os.path.join(_CACHE, f"k_{tag}.cpp")
        with open(cpp, "w") as f:
            f.write(text)
        cmd = ["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread", "-I", _HERE, cpp, "-o", so]
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            raise RuntimeError("emulator compile failed:\n" + out.stderr[:4000])
    return ctypes.CDLL(so)


def run_plan(plan: dict) -> dict:
    """Runs the plan; returns {node index: np.ndarray (raw contiguous buffer)} for plan["results"]."""
    if plan["error"]:
        raise RuntimeError(plan["error"])
    order = plan["order"]
    bufs = []
    for b in plan["buffers"]:
        if b["kind"] == "error":
            bufs.append(np.zeros(64, dtype=np.float32))    # the device word buffer: error word, counters (ints; all-zero bits)
        elif b["kind"] == "external":
            host = order[b["node"]].data.host
            if order[b["node"]].bf16:            # a bf16 tensor the caller holds: raw 16-bit words
                bufs.append(np.ascontiguousarray(host, dtype=np.uint16).reshape(-1))
            else:
                bufs.append(np.ascontiguousarray(host, dtype=np.float32).reshape(-1))
        elif b["kind"] == "twin16":
            bufs.append(np.full(max(1, b["bytes"] // 2), 0x7fc0, dtype=np.uint16))      # bf16 NaN until written
        else:
            bufs.append(np.full(max(1, b["bytes"] // 4), np.nan, dtype=np.float32))
    kernels = [(s["name"], s["source"]) for s in plan["steps"] if s["type"] == "kernel"]
    kernels += [(f"epi_{i}", _epilogue_source(f"epi_{i}", s)) for i, s in enumerate(plan["steps"]) if s["type"] == "gemm" and s.get("epilogue")]
    lib = _compile(kernels) if kernels else None
    for s in plan["steps"]:
        if s["type"] == "kernel":
            fn = ctypes.cast(getattr(lib, s["name"]), ctypes.c_void_p)
            args = (ctypes.c_void_p * len(s["args"]))(*[bufs[a].ctypes.data for a in s["args"]])
            rc = lib.emul_launch(fn, s["grid"], s["block"], args, len(s["args"]))
            assert rc == 0
        elif s.get("tc"):
            _gemm_tc(s, bufs, lib, f"epi_{plan['steps'].index(s)}")
        else:
            _gemm(s, bufs)
    return {r["node"]: bufs[r["buffer"]] for r in plan["results"]}


def _epilogue_source(name, s):
    """The generated epilogue text of a tensor-core GEMM step as plain loops.  The 32 lanes of a warp (8 column groups
    `cq` x 4 row groups `rsub`) are walked one after the other over a 32-row block x 32-column chunk; column sums are
    carried from one row group to the next of the same column group, global sums from every lane to the next (the
    emulator's ormi_epi_rows / ormi_epi_all are the identity), and the lane that is walked last plays lane 0."""
    import re
    csums = sorted(set(re.findall(r"float cs(\d+)\[4\]", s["epi_cols"])))
    gsums = sorted(set(re.findall(r"float gs(\d+) =", s["epi_cols"])))
    carry_in = " ".join(f"if (have_c) for (int j = 0; j < 4; ++j) cs{o}[j] = ccarry[{k}][j];" for k, o in enumerate(csums))
    carry_in += " " + " ".join(f"if (have_g) gs{o} = gcarry[{k}];" for k, o in enumerate(gsums))
    carry_out = " ".join(f"for (int j = 0; j < 4; ++j) ccarry[{k}][j] = cs{o}[j];" for k, o in enumerate(csums)) + " have_c = true; "
    carry_out += " ".join(f"gcarry[{k}] = gs{o};" for k, o in enumerate(gsums)) + " have_g = true;"
    return (s["epi_prelude"] + f'\nextern "C" void {name}(float* C, const float* P, int M, int N{s["epi_params"]}) {{\n'
            f'    {s["epi_init"]}\n'
            f'    for (int row0 = 0; row0 < M; row0 += 32) for (int col0 = 0; col0 < N; col0 += 32) {{\n'
            f'        float gcarry[8]; bool have_g = false;\n'
            f'        for (int cq = 0; cq < 8; ++cq) {{\n            const int gcol = col0 + 4 * cq;\n'
            f'            float ccarry[8][4]; bool have_c = false;\n'
            f'            for (int rsub_i = 0; rsub_i < 4; ++rsub_i) {{\n                const int rsub = rsub_i == 3 ? 0 : rsub_i + 1;\n'
            f'                const int lane = (cq == 7 && rsub == 0) ? 0 : 1 + 8 * rsub + cq;\n'
            f'                {s["epi_cols"]}\n                {carry_in}\n'
            f'                for (int p = 0; p < 8; ++p) {{\n                    const int grow = row0 + 4 * p + rsub;\n'
            f'                    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);\n'
            f'                    if (grow < M && gcol < N) acc = make_float4(P[(long long)grow * N + gcol], P[(long long)grow * N + gcol + 1], '
            f'P[(long long)grow * N + gcol + 2], P[(long long)grow * N + gcol + 3]);\n'
            f'                    {s["epi_pre"]}\n                    if (grow < M && gcol < N) {{ {s["epi_body"]} }}\n                }}\n'
            f'                {carry_out}\n                if (rsub == 0) {{ {s["epi_end"]} }}\n            }}\n        }}\n    }}\n}}\n')


def _to_bf16(x):
    """fp32 -> bf16 (round to nearest even) -> fp32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return (r.astype(np.uint32) << 16).view(np.float32)


def _gemm_tc(s, bufs, lib, epi_name):
    M, N, K = s["M"], s["N"], s["K"]

    def operand(buf, twin, rows, cols, trans, ld):
        srows, scols = (cols, rows) if trans else (rows, cols)          # the stored matrix
        if twin >= 0:      # a bf16 twin written earlier in the plan, or a bf16 tensor of the caller (then twin == buf)
            mat = (bufs[twin][: srows * scols].astype(np.uint32) << 16).view(np.float32).reshape(srows, scols)
        else:
            mat = _to_bf16(np.lib.stride_tricks.as_strided(bufs[buf], shape=(srows, scols), strides=(4 * ld, 4)))
        return mat.T if trans else mat

    A = operand(s["a"], s["a16"], M, K, s["trans_a"], s["lda"])
    B = operand(s["b"], s["b16"], K, N, s["trans_b"], s["ldb"])
    prod = np.ascontiguousarray((A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32))
    if not s["epilogue"]:
        bufs[s["c"]][: M * N] = prod.reshape(-1)
        return
    fn = getattr(lib, epi_name)
    args = [ctypes.c_void_p(bufs[s["c"]].ctypes.data if s["store_c"] else None), ctypes.c_void_p(prod.ctypes.data), ctypes.c_int(M), ctypes.c_int(N)]
    args += [ctypes.c_void_p(bufs[a].ctypes.data) for a in s["epi_args"]]
    fn.restype = None
    fn(*args)


def _gemm(s, bufs):
    M, N, K = s["M"], s["N"], s["K"]
    a, b, c = bufs[s["a"]], bufs[s["b"]], bufs[s["c"]]
    bshape = s["bshape"]
    for bi in range(s["batch"]):
        rem, oa, ob = bi, 0, 0
        for d in range(len(bshape) - 1, -1, -1):
            coord = rem % bshape[d]
            rem //= bshape[d]
            oa += coord * s["astride"][d]
            ob += coord * s["bstride"][d]
        sa = (1, s["lda"]) if s["trans_a"] else (s["lda"], 1)
        sb = (1, s["ldb"]) if s["trans_b"] else (s["ldb"], 1)
        A = np.lib.stride_tricks.as_strided(a[oa:], shape=(M, K), strides=(4 * sa[0], 4 * sa[1]))
        B = np.lib.stride_tricks.as_strided(b[ob:], shape=(K, N), strides=(4 * sb[0], 4 * sb[1]))
        c[bi * M * N:(bi + 1) * M * N] = (A.astype(np.float32) @ B.astype(np.float32)).reshape(-1)


def realize(roots, options=""):
    """Plan + run; returns the logical value (view strides applied) of each root."""
    from ormi_b200 import runtime as RT
    plan = RT.plan(list(roots), host_pointers=True, options=options)
    res = run_plan(plan)
    order = plan["order"]
    outs = []
    for r, root in zip(plan["roots"], roots):
        if root.is_realized:
            raw = np.ascontiguousarray(root.data.host).reshape(-1)
        else:
            raw = res[r]
        if raw.dtype == np.uint16:       # a root materialized as bf16 only: widen (exact)
            raw = (raw.astype(np.uint32) << 16).view(np.float32)
        if not root.shape:
            outs.append(raw[:1].reshape(()).copy())
        else:
            outs.append(np.lib.stride_tricks.as_strided(raw, shape=root.shape, strides=[4 * st for st in root.strides]).copy())
    return outs, plan
