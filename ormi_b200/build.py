"""Builds the C-ABI shared library ``ormi_b200/libormi_b200.so`` for sm_100a with nvcc (in-tree)."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
ROOT = os.path.dirname(HERE)
LIB = os.path.join(HERE, "libormi_b200.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

SOURCES = ["abi.cu", "runtime.cu", "fusion.cpp", "codegen.cpp", "gemm_ffma.cu", "gemm_tcgen05.cu", "gemm_tc.cu", "colsum_static.cu", "comm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-cudart", "static",
]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(ROOT, "include", "ormi_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = os.path.join(CUDA_HOME, "bin", "nvcc")
    objs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(HERE, "build", src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-I", CSRC, "-I", os.path.join(ROOT, "include"), "-c",
               os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out.strip():
            print(f"== {src}\n{out}")
    link = [nvcc, "-shared", "-cudart", "static", "-o", LIB, *objs, "-L", os.path.join(CUDA_HOME, "lib64"), "-lnvrtc",
            "-Xlinker", f"-rpath={os.path.join(CUDA_HOME, 'lib64')}"]
    out = subprocess.run(link, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("link failed:\n" + out.stdout + out.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
