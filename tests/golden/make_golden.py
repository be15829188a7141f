"""Generates the golden vectors under tests/golden/ by running the UNMODIFIED reference CPU backend
(oracle/_ref, built from the reference checkout by oracle/Makefile) on seeded inputs.

    python tests/golden/make_golden.py

Each case is a function returning (roots, ref_request): ``roots`` are nodes of the expanded graph
(autograd done by ormi_b200.graph) that the tests evaluate with their own checker or on the GPU;
``ref_request`` is the same request phrased for the reference (its own autograd builds the backward).
Inputs are regenerated from the seeds, only the reference's outputs are stored.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from ormi_b200 import graph as G          # noqa: E402
from ormi_b200 import workloads as W      # noqa: E402


def fused_rowsum():
    a, b, c = (G.leaf(W.normal(i, (64, 256))) for i in range(3))
    y = W.fused_rowsum(a, b, c)
    return [y], dict(outputs=[(y, "value")])


def softmax():
    x = G.leaf(W.normal(0, (64, 256), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(1, (64, 256)))
    y = W.softmax(x)
    req = dict(outputs=[(y, "value"), (x, "grad")], seeds=[(y, gy)], backward_root=y)
    y.grad = gy
    G.compute_gradients(y)
    return [y, x.grad], req


def layernorm():
    x = G.leaf(W.normal(0, (64, 256), math.sqrt(2.0)), True)
    g = G.leaf(W.uniform(2, (256,), 0.5, 1.5), True)
    b = G.leaf(W.normal(3, (256,), 0.1), True)
    gy = G.leaf(W.normal(1, (64, 256)))
    y = W.layernorm(x, g, b)
    req = dict(outputs=[(y, "value"), (x, "grad"), (g, "grad"), (b, "grad")], seeds=[(y, gy)], backward_root=y)
    y.grad = gy
    G.compute_gradients(y)
    return [y, x.grad, g.grad, b.grad], req


def mlp_step():
    B, D, H = 64, 32, 128
    x, t = G.leaf(W.normal(0, (B, D))), G.leaf(W.normal(1, (B, D)))
    w1, b1 = G.leaf(W.kaiming_uniform(2, D, (D, H)), True), G.leaf(np.zeros(H, np.float32), True)
    w2, b2 = G.leaf(W.kaiming_uniform(3, H, (H, D)), True), G.leaf(np.zeros(D, np.float32), True)
    loss = W.mlp_loss(x, w1, b1, w2, b2, t)
    req = dict(outputs=[(loss, "value")] + [(p, "grad") for p in (w1, b1, w2, b2)], backward_root=loss)
    G.compute_gradients(loss)
    return [loss, w1.grad, b1.grad, w2.grad, b2.grad], req


def broadcast_views_forward():
    """Strided views, row / column / scalar broadcasts and every pointwise op in one graph.

    Two shapes are avoided on purpose because the reference itself mis-computes them: a SUM whose operand
    is a view (cpu/kernels/reduce/sum.cpp:27-29 divides the flat buffer index by the view strides), and a
    broadcast over a middle dimension (core/adjoint.cpp:22-31 builds a keepdims=false SUM but gives it a
    kept-dims view, which sum.cpp:40-45 then indexes out of bounds)."""
    a = G.leaf(W.uniform(0, (8, 3), 0.5, 2.0), True)
    b = G.leaf(W.uniform(1, (3, 8), 0.5, 2.0), True)
    c = G.leaf(W.uniform(3, (3, 1), 0.5, 1.5), True)
    e = G.leaf(W.uniform(2, (8,), 1.0, 2.0), True)
    at = G.transpose(a, [1, 0])
    t = G.div(G.log(G.mul(at, b)), G.cos(G.sin(b)))
    t = G.sub(G.pow_(G.add(G.mul(t, t), G.const(0.5)), e), G.neg(G.exp(G.mul(at, c))))
    root = G.sum_(t, [0], True)
    return root, [a, b, c, e]


def broadcast_views():
    root, params = broadcast_views_forward()
    req = dict(outputs=[(root, "value")] + [(p, "grad") for p in params], backward_root=root)
    G.compute_gradients(root)
    return [root] + [p.grad for p in params], req


CASES = {"fused_rowsum": fused_rowsum, "softmax": softmax, "layernorm": layernorm, "mlp_step": mlp_step,
         "broadcast_views": broadcast_views}


def main():
    from oracle import oracle as O
    if not O.ref_available():
        O.build()
    for name, build in CASES.items():
        _, req = build()
        outs, _ = O.ref_run(**req)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **{f"out{i}": o for i, o in enumerate(outs)})
        print(name, [o.shape for o in outs])


if __name__ == "__main__":
    main()
