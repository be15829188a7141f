"""The benchmark workloads, written with the reference's existing op set.

Ormi has no relu / abs / sqrt / mean / gelu / max ops (ormi-core/csrc/core/ops.h:4-10), so each workload
is composed from NEG EXP ADD SUB MUL DIV POW SUM MATMUL and rank-0 constant leaves.  The same builders
drive the reference CPU backend (the checker) and the B200 backend, so both evaluate the same graph.
"""
from __future__ import annotations

import numpy as np

from . import graph as G

C = G.const


def abs_(z):
    """|z| = (z*z) ** 0.5"""
    return G.pow_(G.mul(z, z), C(0.5))


def relu(z):
    """relu(z) = (z + |z|) * 0.5"""
    return G.mul(G.add(z, abs_(z)), C(0.5))


def fused_rowsum(a, b, c):
    """y = sum(relu(a*b + c) * exp(-|a|), axis=1)   — 11 pointwise nodes and one SUM."""
    return G.sum_(G.mul(relu(G.add(G.mul(a, b), c)), G.exp(G.neg(abs_(a)))), [1], False)


def softmax(x):
    """Row softmax, unstabilised (there is no MAX op): e / sum(e, axis=1, keepdims)."""
    e = G.exp(x)
    return G.div(e, G.sum_(e, [1], True))


def softmax_stable(x):
    """Row softmax with the row maximum subtracted first (extension op MAX): e = exp(x - max); e / sum(e)."""
    e = G.exp(G.sub(x, G.max_(x, [1], True)))
    return G.div(e, G.sum_(e, [1], True))


def relu_max(z):
    """relu(z) = maximum(z, 0) (extension op MAXIMUM)."""
    return G.maximum(z, C(0.0))


def layernorm(x, g, b, eps=1e-5):
    n = x.shape[-1]
    inv_n = C(1.0 / n)
    mean = G.mul(G.sum_(x, [1], True), inv_n)
    xc = G.sub(x, mean)
    var = G.mul(G.sum_(G.mul(xc, xc), [1], True), inv_n)
    xhat = G.div(xc, G.pow_(G.add(var, C(eps)), C(0.5)))
    return G.add(G.mul(xhat, g), b)


def gelu_tanh(u):
    """tanh-form GELU with tanh(z) = 1 - 2 / (exp(2z) + 1)."""
    z = G.mul(C(0.79788456), G.add(u, G.mul(C(0.044715), G.pow_(u, C(3.0)))))
    th = G.sub(C(1.0), G.div(C(2.0), G.add(G.exp(G.mul(C(2.0), z)), C(1.0))))
    return G.mul(G.mul(C(0.5), u), G.add(C(1.0), th))


def mlp_loss(x, w1, b1, w2, b2, t, scale=None, taps=None):
    """loss = mean((gelu(x@W1 + b1) @ W2 + b2 - t)^2); ``scale`` overrides 1/(B*D) (batch-sharded runs
    divide by the global batch).  ``taps``, a dict, receives the hidden activation node under "h", the first matmul
    under "xw1" and the output under "out" (a host loop that realizes the step in several calls holds on to these)."""
    xw1 = G.matmul(x, w1)
    u = G.add(xw1, b1)
    h = gelu_tanh(u)
    out = G.add(G.matmul(h, w2), b2)
    if taps is not None:
        taps["h"], taps["xw1"], taps["out"] = h, xw1, out
    d = G.sub(out, t)
    if scale is None:
        scale = 1.0 / (out.shape[0] * out.shape[1])
    return G.mul(G.sum_(G.mul(d, d), [], False), C(scale))


def sgd_update(param, lr):
    """p_new = p - lr * p.grad"""
    return G.sub(param, G.mul(C(lr), param.grad))


# ---------------------------------------------------------------------------- seeded inputs

def normal(seed, shape, std=1.0, mean=0.0):
    return (np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(std)
            + np.float32(mean)).astype(np.float32)


def uniform(seed, shape, lo, hi):
    return np.random.default_rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


def kaiming_uniform(seed, fan_in, shape):
    bound = float(np.sqrt(6.0 / fan_in))
    return uniform(seed, shape, -bound, bound)
