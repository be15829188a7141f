"""Host-side mirror of ormi-core's lazy graph: Node, shape/stride rules, op constructors, autograd.

This is the Python face of the interface the B200 backend plugs in behind.  It restates, in Python,
the parts of ormi-core that *generate* the graphs the realize path sees — nothing here computes
tensor values:

* ``Node``                      ormi-core/csrc/core/node.h:12-37, node.cpp:8-32
* shape / broadcast rules       ormi-core/csrc/core/shape.cpp:19-63
* op constructors + adjoints    ormi-core/csrc/core/ops/pointwise/*.cpp, reduce/sum.cpp, blas/matmul.cpp,
                                view/{transpose,reshape,expand}.cpp
* ``unbroadcast``               ormi-core/csrc/core/adjoint.cpp:5-34
* ``compute_gradients``         ormi-core/csrc/core/autograd.cpp:12-58
* ``flatten``                   turns a graph into the ``ormi_b200_node`` array of include/ormi_b200.h

The tests compare the graphs produced here, node for node, with the graphs the reference's own
autograd produces.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Iterable, Sequence

import numpy as np

MAX_DIMS = 8


class OpEnum(enum.IntEnum):
    """Same names and values as ormi::ops::OpEnum (ormi-core/csrc/core/ops.h:4-10)."""
    LEAF = 0
    CONST = 1
    NEG = 2
    EXP = 3
    LOG = 4
    SIN = 5
    COS = 6
    ADD = 7
    SUB = 8
    MUL = 9
    DIV = 10
    POW = 11
    MATMUL = 12
    SUM = 13
    TRANSPOSE = 14
    RESHAPE = 15
    EXPAND = 16
    FRAC_DERIV = 17
    # Extension ops (no counterpart in ormi::ops::OpEnum; values kept clear of the reference's range).  They exist in
    # this module, in the C ABI, in the backend and in the extended part of the CPU oracle port only.
    MAXIMUM = 100      # pointwise max(a, b), broadcasting like ADD
    GE = 101           # pointwise a >= b ? 1 : 0 (no gradient)
    MAX = 102          # reduction over axes, same axes / keepdims rules as SUM


VIEW_OPS = (OpEnum.TRANSPOSE, OpEnum.RESHAPE, OpEnum.EXPAND)
UNARY_OPS = (OpEnum.NEG, OpEnum.EXP, OpEnum.LOG, OpEnum.SIN, OpEnum.COS)
BINARY_OPS = (OpEnum.ADD, OpEnum.SUB, OpEnum.MUL, OpEnum.DIV, OpEnum.POW)
EXT_BINARY_OPS = (OpEnum.MAXIMUM, OpEnum.GE)
REDUCE_OPS = (OpEnum.SUM, OpEnum.MAX)

NODE_KEEP = 1
NODE_OWNED = 2
NODE_ALIAS = 4
NODE_TWIN16 = 8           # in: also write this root's bf16 copy ("bf16" matmul arithmetic; a later matmul reads it)
NODE_BF16 = 16            # in: materialize this root as bf16 only / this realized node's buffer holds bf16; out: the buffer is bf16
NODE_REQUIRES_GRAD = 0x100  # only read by the oracle driver


class CNode(ctypes.Structure):
    """ctypes twin of ``ormi_b200_node``."""
    _fields_ = [
        ("op", ctypes.c_int32),
        ("n_parents", ctypes.c_int32),
        ("parents", ctypes.c_int32 * 2),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.c_int32 * MAX_DIMS),
        ("strides", ctypes.c_int32 * MAX_DIMS),
        ("n_axes", ctypes.c_int32),
        ("axes", ctypes.c_int32 * MAX_DIMS),
        ("keepdims", ctypes.c_int32),
        ("flags", ctypes.c_uint32),
        ("data", ctypes.c_void_p),
        ("data_bytes", ctypes.c_int64),
    ]


def calc_contiguous_strides(shape: Sequence[int]) -> list[int]:
    """ormi-core/csrc/core/shape.cpp:19-25."""
    strides = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = strides[i + 1] * shape[i + 1]
    return strides


def broadcast_shapes(a: Sequence[int], b: Sequence[int]) -> list[int]:
    """Right-aligned numpy broadcasting (ormi-core/csrc/core/shape.cpp:27-44)."""
    n = max(len(a), len(b))
    out = []
    for i in range(n):
        da = 1 if i < n - len(a) else a[i - (n - len(a))]
        db = 1 if i < n - len(b) else b[i - (n - len(b))]
        if da != db and da != 1 and db != 1:
            raise RuntimeError("Operands could not be broadcast together.")
        out.append(max(da, db))
    return out


def numel(shape: Sequence[int]) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class Buffer:
    """A realized tensor: host array (oracle runs) and/or a device allocation (B200 runs).

    Mirrors ormi::Buffer (ormi-core/csrc/core/memory.h:9-20): pointer, byte size, shape.  ``release`` is
    called when the last owner drops it and hands the device block back to the pool.
    """
    __slots__ = ("host", "dev_ptr", "nbytes", "shape", "_release", "__weakref__")

    def __init__(self, shape, host=None, dev_ptr=None, release=None):
        self.shape = [int(s) for s in shape]
        self.nbytes = 4 * numel(self.shape)
        self.host = host
        self.dev_ptr = dev_ptr
        self._release = release

    def __del__(self):
        rel, self._release = self._release, None
        if rel is not None and self.dev_ptr:
            try:
                rel(self.dev_ptr, self.nbytes)
            except Exception:
                pass


class Node:
    """Mirror of ormi::Node (ormi-core/csrc/core/node.h:12-37)."""
    __slots__ = ("op", "parents", "data", "grad", "requires_grad", "shape", "strides",
                 "axes", "keepdims", "keep", "twin16", "bf16", "name", "__weakref__")

    def __init__(self, op, parents=(), *, data: Buffer | None = None, requires_grad=False,
                 axes: Sequence[int] = (), keepdims=False, shape: Sequence[int] | None = None):
        self.op = OpEnum(op)
        self.parents = list(parents)
        self.data = data
        self.grad: Node | None = None
        self.axes = [int(a) for a in axes]
        self.keepdims = bool(keepdims)
        self.keep = False
        self.twin16 = False
        self.bf16 = False          # a matmul operand kept as bf16 only (ORMI_NODE_BF16)
        self.name = None
        if self.op == OpEnum.LEAF:
            # leaf constructor, node.cpp:8-13
            assert data is not None
            self.requires_grad = bool(requires_grad)
            self.shape = list(data.shape)
            self.strides = calc_contiguous_strides(self.shape)
            return
        # internal constructor, node.cpp:16-32
        self.requires_grad = any(p.requires_grad for p in self.parents)
        self.shape = _infer_shape(self, shape)
        self.strides = _infer_strides(self)
        if len(self.shape) > MAX_DIMS:
            raise RuntimeError(f"more than {MAX_DIMS} dimensions")

    @property
    def is_realized(self) -> bool:
        return self.data is not None

    def numel(self) -> int:
        return numel(self.shape)

    def __repr__(self):
        return f"Node({self.op.name}, shape={self.shape}, strides={self.strides})"


# ---------------------------------------------------------------------------- shape rules

def _infer_shape(node: Node, target: Sequence[int] | None) -> list[int]:
    op, ps = node.op, node.parents
    if op in UNARY_OPS:
        return list(ps[0].shape)                                   # shape.cpp:57-59
    if op in BINARY_OPS or op in EXT_BINARY_OPS:
        return broadcast_shapes(ps[0].shape, ps[1].shape)           # shape.cpp:61-63
    if op == OpEnum.MATMUL:
        return _infer_matmul_shape(ps)
    if op in REDUCE_OPS:
        return _infer_sum_shape(ps[0].shape, node.axes, node.keepdims)
    if op == OpEnum.TRANSPOSE:
        if len(ps[0].shape) != len(node.axes):
            raise RuntimeError("TRANSPOSE axes count must match tensor dimensions.")
        return [ps[0].shape[a] for a in node.axes]                  # transpose.cpp:18-32
    if op in (OpEnum.RESHAPE, OpEnum.EXPAND):
        return [int(s) for s in target]                             # reshape.cpp:18-21, expand.cpp:19-22
    raise RuntimeError("Shape inference rule not registered for this OpEnum.")


def _infer_matmul_shape(ps) -> list[int]:
    """ormi-core/csrc/core/ops/blas/matmul.cpp:27-67."""
    if len(ps) < 2:
        raise RuntimeError("MATMUL requires 2 parents.")
    a, b = ps[0].shape, ps[1].shape
    if len(a) < 2 or len(b) < 2:
        raise RuntimeError("MATMUL requires operands to have at least 2 dimensions.")
    if a[-1] != b[-2]:
        raise RuntimeError("MATMUL inner dimensions must match (K_a != K_b).")
    out = []
    if len(a) > 2 or len(b) > 2:
        try:
            out = broadcast_shapes(a[:-2], b[:-2])
        except RuntimeError:
            raise RuntimeError("MATMUL batch dimensions could not be broadcast together.")
    return out + [a[-2], b[-1]]


def _infer_sum_shape(in_shape, axes, keepdims) -> list[int]:
    """ormi-core/csrc/core/ops/reduce/sum.cpp:25-55."""
    if not axes:
        return [1] * len(in_shape) if keepdims else []
    out = []
    for d, s in enumerate(in_shape):
        if d not in axes:
            out.append(s)
        elif keepdims:
            out.append(1)
    return out


def _infer_strides(node: Node) -> list[int]:
    op = node.op
    if op == OpEnum.TRANSPOSE:                                      # transpose.cpp:55-64
        return [node.parents[0].strides[a] for a in node.axes]
    if op == OpEnum.RESHAPE:
        return _reshape_strides(node.parents[0].shape, node.parents[0].strides, node.shape)
    if op == OpEnum.EXPAND:                                         # expand.cpp:35-57
        p = node.parents[0]
        off = len(node.shape) - len(p.shape)
        out = []
        for i, s in enumerate(node.shape):
            if i < off:
                out.append(0)
            elif p.shape[i - off] == 1 and s > 1:
                out.append(0)
            else:
                out.append(p.strides[i - off])
        return out
    return calc_contiguous_strides(node.shape)


def _reshape_strides(old_shape, old_strides, out_shape) -> list[int]:
    """Zero-copy reshape stride rule (ormi-core/csrc/core/ops/view/reshape.cpp:37-92)."""
    if not old_shape:
        return calc_contiguous_strides(out_shape)
    new = [0] * len(out_shape)
    o = n = 0
    while n < len(out_shape) and o < len(old_shape):
        old_size, new_size = old_shape[o], out_shape[n]
        o_end, n_end = o + 1, n + 1
        while old_size != new_size:
            if old_size < new_size:
                if o_end >= len(old_shape):
                    raise RuntimeError("RESHAPE size mismatch.")
                old_size *= old_shape[o_end]
                o_end += 1
            else:
                if n_end >= len(out_shape):
                    raise RuntimeError("RESHAPE size mismatch.")
                new_size *= out_shape[n_end]
                n_end += 1
        for i in range(o, o_end - 1):
            if old_shape[i] != 1 and old_shape[i + 1] != 1:
                if old_strides[i] != old_shape[i + 1] * old_strides[i + 1]:
                    raise RuntimeError("RESHAPE cannot be performed as a zero-copy view because the tensor "
                                       "is not contiguous across merged dimensions.")
        cur = old_strides[o_end - 1]
        for i in range(n_end - 1, n - 1, -1):
            new[i] = cur
            cur *= out_shape[i]
        o, n = o_end, n_end
    while o < len(old_shape):
        if old_shape[o] != 1:
            raise RuntimeError("RESHAPE size mismatch trailing dims.")
        o += 1
    while n < len(out_shape):
        if out_shape[n] != 1:
            raise RuntimeError("RESHAPE size mismatch trailing dims.")
        new[n] = 1
        n += 1
    return new


# ---------------------------------------------------------------------------- op constructors

def leaf(array, requires_grad=False) -> Node:
    """A leaf over host data (uploaded by the runtime on first use)."""
    arr = np.asarray(array, dtype=np.float32)
    arr = np.ascontiguousarray(arr).reshape(arr.shape)   # ascontiguousarray would turn rank 0 into rank 1
    return Node(OpEnum.LEAF, data=Buffer(arr.shape, host=arr), requires_grad=requires_grad)


def const(value: float) -> Node:
    """Rank-0 constant leaf, like ``Node(full({}, v))``."""
    return leaf(np.float32(value))


def _un(op):
    def f(a: Node) -> Node:
        return Node(op, [a])
    return f


def _bin(op):
    def f(a: Node, b: Node) -> Node:
        return Node(op, [a, b])
    return f


neg, exp, log, sin, cos = (_un(o) for o in UNARY_OPS)
add, sub, mul, div, pow_ = (_bin(o) for o in BINARY_OPS)


def matmul(a: Node, b: Node) -> Node:
    return Node(OpEnum.MATMUL, [a, b])


def sum_(a: Node, axes: Iterable[int] = (), keepdims=False) -> Node:
    return Node(OpEnum.SUM, [a], axes=list(axes), keepdims=keepdims)


def maximum(a: Node, b: Node) -> Node:
    """Extension: pointwise max(a, b)."""
    return Node(OpEnum.MAXIMUM, [a, b])


def ge(a: Node, b: Node) -> Node:
    """Extension: 1.0 where a >= b, else 0.0; carries no gradient."""
    n = Node(OpEnum.GE, [a, b])
    n.requires_grad = False
    return n


def max_(a: Node, axes: Iterable[int] = (), keepdims=False) -> Node:
    """Extension: maximum over ``axes`` (all axes when empty), shaped like ``sum_``."""
    return Node(OpEnum.MAX, [a], axes=list(axes), keepdims=keepdims)


def mean(a: Node, axes: Iterable[int] = (), keepdims=False) -> Node:
    """Extension (a composition, no new op): SUM over ``axes`` times 1 / (number of reduced elements)."""
    axes = list(axes)
    count = numel(a.shape) if not axes else numel([a.shape[d] for d in axes])
    return Node(OpEnum.MUL, [sum_(a, axes, keepdims), const(1.0 / count)])


def transpose(a: Node, axes: Sequence[int]) -> Node:
    return Node(OpEnum.TRANSPOSE, [a], axes=list(axes))


def reshape(a: Node, shape: Sequence[int]) -> Node:
    return Node(OpEnum.RESHAPE, [a], shape=list(shape))


def expand(a: Node, shape: Sequence[int]) -> Node:
    return Node(OpEnum.EXPAND, [a], shape=list(shape))


# ---------------------------------------------------------------------------- autograd

def unbroadcast(grad: Node, target_shape: Sequence[int]) -> Node:
    """ormi-core/csrc/core/adjoint.cpp:5-34: SUM over the broadcast axes, view overwritten to the target."""
    target_shape = list(target_shape)
    if grad.shape == target_shape:
        return grad
    ng, nt = len(grad.shape), len(target_shape)
    axes = list(range(ng - nt))
    for i in range(ng - nt, ng):
        if target_shape[i - (ng - nt)] == 1 and grad.shape[i] > 1:
            axes.append(i)
    if not axes:
        return grad
    s = Node(OpEnum.SUM, [grad], axes=axes, keepdims=False)
    s.shape = target_shape
    s.strides = calc_contiguous_strides(target_shape)
    return s


def _accumulate(p: Node, local: Node):
    p.grad = local if p.grad is None else Node(OpEnum.ADD, [p.grad, local])


def _adj_add(n):                                                    # add.cpp:14-23
    for p in n.parents[:2]:
        if p.requires_grad:
            _accumulate(p, unbroadcast(n.grad, p.shape))


def _adj_sub(n):                                                    # sub.cpp:14-30
    x, y = n.parents
    if x.requires_grad:
        _accumulate(x, unbroadcast(n.grad, x.shape))
    if y.requires_grad:
        _accumulate(y, unbroadcast(Node(OpEnum.NEG, [n.grad]), y.shape))


def _adj_mul(n):                                                    # mul.cpp:14-31
    x, y = n.parents
    if x.requires_grad:
        _accumulate(x, unbroadcast(Node(OpEnum.MUL, [n.grad, y]), x.shape))
    if y.requires_grad:
        _accumulate(y, unbroadcast(Node(OpEnum.MUL, [n.grad, x]), y.shape))


def _adj_div(n):                                                    # div.cpp:14-36
    x, y = n.parents
    dz = n.grad
    if x.requires_grad:
        _accumulate(x, unbroadcast(Node(OpEnum.DIV, [dz, y]), x.shape))
    if y.requires_grad:
        y_sq = Node(OpEnum.MUL, [y, y])
        x_div = Node(OpEnum.DIV, [x, y_sq])
        dz_mul = Node(OpEnum.MUL, [dz, x_div])
        _accumulate(y, unbroadcast(Node(OpEnum.NEG, [dz_mul]), y.shape))


def _adj_pow(n):                                                    # pow.cpp:14-43
    x, y = n.parents
    dz = n.grad
    if x.requires_grad:
        ones = leaf(np.ones(y.shape, dtype=np.float32))
        y_m1 = Node(OpEnum.SUB, [y, ones])
        x_pow = Node(OpEnum.POW, [x, y_m1])
        y_mul = Node(OpEnum.MUL, [y, x_pow])
        _accumulate(x, unbroadcast(Node(OpEnum.MUL, [dz, y_mul]), x.shape))
    if y.requires_grad:
        log_x = Node(OpEnum.LOG, [x])
        n_log = Node(OpEnum.MUL, [n, log_x])
        _accumulate(y, unbroadcast(Node(OpEnum.MUL, [dz, n_log]), y.shape))


def _adj_neg(n):                                                    # neg.cpp:11-19
    x = n.parents[0]
    if x.requires_grad:
        _accumulate(x, unbroadcast(Node(OpEnum.NEG, [n.grad]), x.shape))


def _adj_exp(n):                                                    # exp.cpp:11-19
    x = n.parents[0]
    if x.requires_grad:
        _accumulate(x, unbroadcast(Node(OpEnum.MUL, [n, n.grad]), x.shape))


def _adj_log(n):                                                    # log.cpp:14-26
    x = n.parents[0]
    if x.requires_grad:
        _accumulate(x, unbroadcast(Node(OpEnum.DIV, [n.grad, x]), x.shape))


def _adj_sin(n):                                                    # sin.cpp:11-20
    x = n.parents[0]
    if x.requires_grad:
        c = Node(OpEnum.COS, [x])
        _accumulate(x, unbroadcast(Node(OpEnum.MUL, [c, n.grad]), x.shape))


def _adj_cos(n):                                                    # cos.cpp: d cos = -sin(x) * dz
    x = n.parents[0]
    if x.requires_grad:
        s = Node(OpEnum.SIN, [x])
        ns = Node(OpEnum.NEG, [s])
        _accumulate(x, unbroadcast(Node(OpEnum.MUL, [ns, n.grad]), x.shape))


def _adj_sum(n):                                                    # reduce/sum.cpp:59-97
    x = n.parents[0]
    if not x.requires_grad:
        return
    dz = n.grad
    if not n.keepdims:
        target = list(x.shape)
        if not n.axes:
            target = [1] * len(target)
        else:
            for a in n.axes:
                target[a] = 1
        dz = Node(OpEnum.RESHAPE, [dz], shape=target)
    _accumulate(x, Node(OpEnum.EXPAND, [dz], shape=list(x.shape)))


def _adj_maximum(n):
    """Extension: the gradient goes to the larger operand; on a tie to the first one."""
    a, b = n.parents
    first = Node(OpEnum.GE, [a, b])
    first.requires_grad = False
    if a.requires_grad:
        _accumulate(a, unbroadcast(Node(OpEnum.MUL, [n.grad, first]), a.shape))
    if b.requires_grad:
        second = Node(OpEnum.SUB, [const(1.0), first])
        _accumulate(b, unbroadcast(Node(OpEnum.MUL, [n.grad, second]), b.shape))


def _adj_max(n):
    """Extension: the gradient flows to every element equal to the maximum of its group (ties share nothing: each tied
    element receives the full gradient, the derivative of max along each of them)."""
    x = n.parents[0]
    if not x.requires_grad:
        return
    dz, m = n.grad, n
    if not n.keepdims:
        target = list(x.shape)
        if not n.axes:
            target = [1] * len(target)
        else:
            for a in n.axes:
                target[a] = 1
        dz = Node(OpEnum.RESHAPE, [dz], shape=target)
        m = Node(OpEnum.RESHAPE, [n], shape=target)
    hit = Node(OpEnum.GE, [x, Node(OpEnum.EXPAND, [m], shape=list(x.shape))])
    hit.requires_grad = False
    _accumulate(x, Node(OpEnum.MUL, [Node(OpEnum.EXPAND, [dz], shape=list(x.shape)), hit]))


def _adj_matmul(n):                                                 # blas/matmul.cpp:71-135
    x, y = n.parents
    dz = n.grad

    def t_axes(nd):
        ax = list(range(nd))
        if nd >= 2:
            ax[-2], ax[-1] = ax[-1], ax[-2]
        return ax

    if x.requires_grad:
        y_t = Node(OpEnum.TRANSPOSE, [y], axes=t_axes(len(y.shape)))
        _accumulate(x, unbroadcast(Node(OpEnum.MATMUL, [dz, y_t]), x.shape))
    if y.requires_grad:
        x_t = Node(OpEnum.TRANSPOSE, [x], axes=t_axes(len(x.shape)))
        _accumulate(y, unbroadcast(Node(OpEnum.MATMUL, [x_t, dz]), y.shape))


def _adj_transpose(n):                                              # view/transpose.cpp:34-53
    x = n.parents[0]
    if not x.requires_grad:
        return
    inv = [0] * len(n.axes)
    for i, a in enumerate(n.axes):
        inv[a] = i
    _accumulate(x, Node(OpEnum.TRANSPOSE, [n.grad], axes=inv))


def _adj_reshape(n):                                                # view/reshape.cpp:23-35
    x = n.parents[0]
    if x.requires_grad:
        _accumulate(x, Node(OpEnum.RESHAPE, [n.grad], shape=list(x.shape)))


def _adj_expand(n):                                                 # view/expand.cpp:24-33
    x = n.parents[0]
    if x.requires_grad:
        _accumulate(x, unbroadcast(n.grad, x.shape))


_ADJOINTS = {
    OpEnum.ADD: _adj_add, OpEnum.SUB: _adj_sub, OpEnum.MUL: _adj_mul, OpEnum.DIV: _adj_div,
    OpEnum.POW: _adj_pow, OpEnum.NEG: _adj_neg, OpEnum.EXP: _adj_exp, OpEnum.LOG: _adj_log,
    OpEnum.SIN: _adj_sin, OpEnum.COS: _adj_cos, OpEnum.SUM: _adj_sum, OpEnum.MATMUL: _adj_matmul,
    OpEnum.TRANSPOSE: _adj_transpose, OpEnum.RESHAPE: _adj_reshape, OpEnum.EXPAND: _adj_expand,
    OpEnum.MAXIMUM: _adj_maximum, OpEnum.MAX: _adj_max, OpEnum.GE: lambda n: None,
}


def topo_order(roots: Sequence[Node], stop_at_realized=False) -> list[Node]:
    """Post-order DFS, parents before children (ormi-core/csrc/core/autograd.cpp:12-22), iterative."""
    seen, order = set(), []
    for root in roots:
        stack = [(root, 0)]
        while stack:
            node, i = stack.pop()
            if id(node) in seen:
                continue
            parents = [] if (stop_at_realized and node.is_realized) else node.parents
            if i < len(parents):
                stack.append((node, i + 1))
                if id(parents[i]) not in seen:
                    stack.append((parents[i], 0))
            else:
                seen.add(id(node))
                order.append(node)
    return order


def compute_gradients(root: Node):
    """ormi-core/csrc/core/autograd.cpp:24-47: seed with ones unless a gradient is already set, then run
    the adjoint rules in reverse topological order.  Only builds graph nodes."""
    topo = topo_order([root])
    if root.grad is None:
        root.grad = leaf(np.ones(root.shape, dtype=np.float32))
    for node in reversed(topo):
        if node.grad is None or node.op == OpEnum.LEAF:
            continue
        rule = _ADJOINTS.get(node.op)
        if rule is None:
            raise RuntimeError("No Adjoint rule registered for operation.")
        rule(node)


def zero_grad_graph(root: Node):
    """ormi-core/csrc/core/autograd.cpp:49-58."""
    for node in topo_order([root]):
        node.grad = None


# ---------------------------------------------------------------------------- flattening

def flatten(roots: Sequence[Node], *, host_pointers=False, stop_at_realized=True):
    """Flattens the graph under ``roots`` into a ctypes array of ``ormi_b200_node`` in topological order.

    Returns ``(array, order, root_indices)``.  ``host_pointers=True`` stores the host array address of
    realized nodes in ``data`` (oracle runs); otherwise the device pointer.
    """
    order = topo_order(roots, stop_at_realized=stop_at_realized)
    index = {id(n): i for i, n in enumerate(order)}
    arr = (CNode * max(1, len(order)))()
    for i, n in enumerate(order):
        c = arr[i]
        c.op = int(n.op)
        c.ndim = len(n.shape)
        for d, (s, st) in enumerate(zip(n.shape, n.strides)):
            c.shape[d] = s
            c.strides[d] = st
        c.n_axes = len(n.axes)
        for d, a in enumerate(n.axes):
            c.axes[d] = a
        c.keepdims = int(n.keepdims)
        c.flags = ((NODE_KEEP if n.keep else 0) | (NODE_TWIN16 if n.twin16 else 0) | (NODE_BF16 if n.bf16 else 0) |
                   (NODE_REQUIRES_GRAD if n.requires_grad else 0))
        if n.is_realized and stop_at_realized or n.op == OpEnum.LEAF:
            c.n_parents = 0
            buf = n.data
            if host_pointers:
                if buf.host is None:
                    raise RuntimeError("node has no host data")
                c.data = buf.host.ctypes.data
            else:
                c.data = buf.dev_ptr
            c.data_bytes = buf.nbytes
        else:
            c.n_parents = len(n.parents)
            for k, p in enumerate(n.parents[:2]):
                c.parents[k] = index[id(p)]
    return arr, order, [index[id(r)] for r in roots]
