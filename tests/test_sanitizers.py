"""The fusion scheduler and the code generator (plain C++, no CUDA) built with AddressSanitizer and
UndefinedBehaviorSanitizer and driven over a spread of graphs: softmax / layernorm forward + backward on ragged and wide
rows, the MLP training step in every arithmetic, sums of every kind, views, matmul layouts, the extension ops — with the
option strings the product takes.  A heap overrun, a use after free or undefined arithmetic in the host code ends the
child process with a report."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(ROOT, "ormi_b200", "csrc")


def _runtime(name):
    out = subprocess.run(["g++", "-print-file-name=" + name], capture_output=True, text=True).stdout.strip()
    return out if os.path.isabs(out) and os.path.exists(out) else None


def test_scheduler_and_codegen_under_asan_ubsan(tmp_path):
    asan = _runtime("libasan.so")
    if asan is None:
        pytest.skip("no AddressSanitizer runtime beside g++")
    lib = str(tmp_path / "libsched_san.so")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fPIC", "-shared", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
           "-I", os.path.join(ROOT, "include"), "-I", CSRC, os.path.join(CSRC, "fusion.cpp"), os.path.join(CSRC, "codegen.cpp"),
           os.path.join(HERE, "sanitize", "sched_harness.cpp"), "-o", lib]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-3000:]
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([sys.executable, os.path.join(HERE, "sanitize", "drive.py"), lib], capture_output=True, text=True, env=env, timeout=900)
    report = run.stdout[-2000:] + run.stderr[-4000:]
    assert run.returncode == 0, report
    assert "AddressSanitizer" not in report and "runtime error:" not in report, report
    assert "planned" in run.stdout and ", 0 refused" in run.stdout, report
