"""Run under LD_PRELOAD=libasan: plans a spread of graphs through the sanitized scheduler + code generator.

usage: drive.py <libsched_san.so>.  Prints "planned N graphs" on success; a sanitizer report ends the process."""
import ctypes
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from ormi_b200 import graph as G            # noqa: E402
from ormi_b200 import workloads as W        # noqa: E402

san = ctypes.CDLL(sys.argv[1])
san.sched_plan_json.restype = ctypes.c_int
san.sched_compile_simple.restype = ctypes.c_int


def plan(roots, options=""):
    arr, order, root_idx = G.flatten(list(roots), host_pointers=True, stop_at_realized=True)
    ridx = (ctypes.c_int * len(root_idx))(*root_idx)
    n = ctypes.c_size_t()
    buf = ctypes.create_string_buffer(1 << 22)
    rc = san.sched_plan_json(arr, len(order), ridx, len(root_idx), options.encode(), buf, len(buf), ctypes.byref(n))
    if rc != 0:
        return {"error": buf.value.decode(), "steps": []}
    out = json.loads(buf.value.decode())
    for r in root_idx:
        san.sched_compile_simple(arr, len(order), r, ctypes.byref(n))
    return out


def leaf(shape, seed, grad=False):
    return G.leaf(W.normal(seed, shape), grad)


count = 0
errors = []


def go(roots, options=("", "fusion=off", "matmul=bf16", "matmul=bf16,intermediates=free", "aligned=0", "tune.rows_vpt=8,tune.rows_stage=2")):
    global count
    for o in options:
        out = plan(roots, o)
        count += 1
        if out["error"] or not out["steps"]:
            errors.append((o, out["error"]))


# softmax / layernorm forward + backward, ragged and wide rows
for shape in ((8, 16), (5, 33), (64, 4096), (3, 20000), (1, 7), (130, 1000)):
    x = leaf(shape, 1, True)
    y = W.softmax(x)
    y.grad = leaf(shape, 2)
    G.compute_gradients(y)
    go([y, x.grad])
    x = leaf(shape, 3, True)
    g, b = leaf(shape[-1:], 4, True), leaf(shape[-1:], 5, True)
    z = W.layernorm(x, g, b)
    z.grad = leaf(shape, 6)
    G.compute_gradients(z)
    go([z, x.grad, g.grad, b.grad])
# the MLP training step, aligned and ragged widths
for B, D, H in ((256, 128, 512), (128, 136, 264), (33, 20, 50), (8192, 2048, 8192)):
    x, t = leaf((B, D), 0), leaf((B, D), 1)
    w1, b1 = leaf((D, H), 2, True), leaf((H,), 4, True)
    w2, b2 = leaf((H, D), 3, True), leaf((D,), 5, True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    G.compute_gradients(loss)
    go([loss] + [W.sgd_update(p, 0.1) for p in (w1, b1, w2, b2)])
    go([loss] + [p.grad for p in (w1, b1, w2, b2)])
# sums of every kind, views, matmul layouts, extension ops
a = leaf((6, 5, 4), 7)
for axes in ([], [0], [1], [2], [0, 1], [1, 2], [0, 2], [0, 1, 2]):
    for keep in (False, True):
        go([G.sum_(G.mul(a, a), axes, keep)], ("", "fusion=off"))
m1, m2 = leaf((12, 20), 8), leaf((20, 28), 9)
go([G.matmul(m1, m2), G.matmul(G.transpose(m2, [1, 0]), G.transpose(m1, [1, 0])), G.sum_(G.transpose(m1, [1, 0]), [0], False)])
go([G.exp(G.expand(G.reshape(leaf((4,), 10), [1, 4]), [3, 4]))])
go([W.fused_rowsum(leaf((40, 48), 11), leaf((40, 48), 12), leaf((40, 48), 13))])
xs = leaf((9, 31), 14, True)
ys = W.softmax_stable(xs)
ys.grad = leaf((9, 31), 15)
G.compute_gradients(ys)
go([ys, xs.grad])
print("planned", count, "graphs,", len(errors), "refused", errors[:3])
