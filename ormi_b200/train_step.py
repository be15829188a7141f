"""A repeated training step over the graph API, batch-sharded over ranks.

The step is ordinary Ormi graph code (ormi_b200.workloads.mlp_loss, compute_gradients, sgd_update).  What this
module adds is the host loop a data-parallel job needs around ``ormi_b200_realize``:

* the step is split into *phases* (roots that are realized together).  Between phases the gradients that are
  already complete go out through ``ormi_b200_allreduce_sum_f32`` on the second stream, and the compute stream
  waits for each bucket only where its sums are first read (``ormi_b200_comm_mark`` / ``ormi_b200_comm_wait``);
* each phase is flattened once; every later step patches the device pointers of its inputs into the flattened
  graph and hands it to the backend again (plan and kernels come from the caches), so a step costs a few C calls;
* parameters ping-pong: the update phase returns fresh buffers that become the next step's leaves.

Sharding rule (rows of x and t are split evenly over the ranks, weights are replicated): each rank's loss is
scaled by 1 / (global_batch * D), so the *sum* of the local gradients over ranks is the gradient of the global
mean loss; that sum is the only exchange of a step.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Sequence

import numpy as np

from . import graph as G
from . import workloads as W
from ._lib import lib, check


class _Phase:
    def __init__(self, dev, roots: Sequence[G.Node], produced: dict, externals: dict):
        order = G.topo_order(list(roots), stop_at_realized=True)
        dev.ensure_on_device(order)
        arr, order, ridx = G.flatten(list(roots), host_pointers=False, stop_at_realized=True)
        self.arr, self.order, self.n = arr, order, len(order)
        self.template = bytes(arr)
        self.roots = list(ridx)
        self.ridx = (ctypes.c_int * len(ridx))(*ridx)
        # where each realized input of this phase comes from
        self.bind_external = []      # (index, name)
        self.bind_produced = []      # (index, key) with key = id(node) of a node an earlier phase materialized
        for i, n in enumerate(order):
            if not n.is_realized:
                continue
            if id(n) in externals:
                self.bind_external.append((i, externals[id(n)]))
            elif id(n) in produced:
                self.bind_produced.append((i, id(n)))
        self.node_ids = [id(n) for n in order]


class StepProgram:
    """Phases of one step, re-run every step with patched pointers."""

    def __init__(self, dev):
        self.dev = dev
        self.phases: list[_Phase] = []
        self.produced: dict[int, tuple[int, int]] = {}     # id(node) -> (ptr, bytes) of the current step
        self.externals: dict[int, str] = {}                # id(node) -> name
        self.ext_ptr: dict[str, tuple[int, int]] = {}      # name -> (ptr, bytes)
        self._keepalive = []
        # "free": what a phase materializes without being asked for (no root, not flagged keep) is scratch of that call
        # instead of coming back to be freed here
        self.intermediates = "keep"

    def _realize_options(self):
        """Sets the program's "intermediates" option for one realize call; returns what to restore."""
        before = self.dev.get_option("intermediates") or "keep"
        if before != self.intermediates:
            self.dev.set_option("intermediates", self.intermediates)
        return before

    def external(self, name: str, node: G.Node):
        self.dev.ensure_on_device([node])
        self.externals[id(node)] = name
        self.ext_ptr[name] = (node.data.dev_ptr, node.data.nbytes)
        self._keepalive.append(node)

    def add_phase(self, roots: Sequence[G.Node]) -> _Phase:
        """Flattens the phase, then realizes it once so that later phases see its outputs as inputs."""
        ph = _Phase(self.dev, roots, self.produced, self.externals)
        self.phases.append(ph)
        pending = [n for n in ph.order if not n.is_realized]
        before = self._realize_options()
        try:
            self.dev.realize(list(roots))
        finally:
            if before != self.intermediates:
                self.dev.set_option("intermediates", before)
        for n in pending:               # what this phase wrote to memory: inputs of later phases
            if n.is_realized:
                self.produced.setdefault(id(n), (n.data.dev_ptr, n.data.nbytes))
        self._keepalive.extend(roots)
        return ph

    def run_phase(self, k: int, step_outputs: dict) -> dict:
        """Runs phase k; `step_outputs` maps id(node) -> (ptr, bytes) of what this step has produced so far and is
        extended with this phase's owned outputs.  Returns {root position: (ptr, bytes)}."""
        ph = self.phases[k]
        ctypes.memmove(ph.arr, ph.template, len(ph.template))
        for i, name in ph.bind_external:
            ph.arr[i].data = self.ext_ptr[name][0]
        for i, key in ph.bind_produced:
            ph.arr[i].data = step_outputs[key][0]
        before = self._realize_options()
        try:
            check(lib.ormi_b200_realize(self.dev.handle, ph.arr, ph.n, ph.ridx, len(ph.roots)))
        finally:
            if before != self.intermediates:
                self.dev.set_option("intermediates", before)
        for i in range(ph.n):
            c = ph.arr[i]
            if c.flags & (G.NODE_OWNED | G.NODE_ALIAS) and c.data:
                step_outputs[ph.node_ids[i]] = (c.data, c.data_bytes)
                if c.flags & G.NODE_OWNED:      # only these were allocated by this step (an alias is a view of something else)
                    step_outputs.setdefault("owned", []).append((c.data, c.data_bytes))
        return {pos: step_outputs[ph.node_ids[r]] for pos, r in enumerate(ph.roots) if ph.node_ids[r] in step_outputs}


class MLPTrainer:
    """The 2-layer MLP training step of the benchmark (tanh-GELU, mean squared error, SGD), one rank of `world`.

    x, t: this rank's rows.  w1, b1, w2, b2: replicated parameters (numpy arrays).  The gradient all-reduce runs
    only when ``world > 1`` (the communicator must have been initialised on ``dev``).

    Schedule of one step with ``world > 1`` (plain SGD, only the order of independent work is chosen):

        F   h = gelu(x W1 + b1)                      beside the all-reduce of the previous step's dW2, db2
        U2  W2, b2 -= lr * (dW2, db2 of the previous step)         after that all-reduce
        B1  loss, dW1, db1                           -> all-reduce bucket 1 on the second stream
        B2  dW2, db2                                 beside bucket 1 -> all-reduce bucket 2
        U1  W1, b1 -= lr * (dW1, db1)                after bucket 1

    so bucket 1 hides behind the dW2 GEMM and bucket 2 behind the next step's first GEMM.  `flush` applies the
    update that is still pending after the last step.
    """

    def __init__(self, dev, x, t, w1, b1, w2, b2, lr: float, global_batch: int | None = None, world: int = 1,
                 overlap: bool = True, bf16_matmuls: bool | None = None):
        self.dev, self.world, self.overlap = dev, world, overlap
        if bf16_matmuls is None:
            bf16_matmuls = dev.get_option("matmul") == "bf16"
        B, D = x.shape[0], t.shape[1]
        self.global_batch = global_batch or B * world
        scale = 1.0 / (self.global_batch * D)
        p = self.prog = StepProgram(dev)
        xn, tn = dev.leaf(x), dev.leaf(t)
        params = {k: dev.leaf(v, True) for k, v in (("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2))}
        for k, n in (("x", xn), ("t", tn), *params.items()):
            p.external(k, n)
        taps: dict = {}
        loss = W.mlp_loss(xn, params["w1"], params["b1"], params["w2"], params["b2"], tn, scale=scale, taps=taps)
        G.compute_gradients(loss)
        self.names = ["w1", "b1", "w2", "b2"]
        grads = {k: params[k].grad for k in self.names}

        def weight_update(node, k):
            # the new weight matrices are matmul operands of the next step: in "bf16" arithmetic the update kernel
            # writes their bf16 copies along (the flag is ignored by the other arithmetics)
            node.twin16 = k in ("w1", "w2")
            return node
        if world == 1:
            # one realize call per step whose roots are all that is read afterwards
            p.intermediates = "free"
            ups = [weight_update(W.sgd_update(params[k], lr), k) for k in self.names]
            p.add_phase([loss] + ups)
        else:
            # the updates read the summed gradients as plain inputs; until a step has produced some they are zero
            self._zero = {}
            g_leaf = {}
            for k in self.names:
                g_leaf[k] = dev.leaf(np.zeros(params[k].shape, dtype=np.float32))
                p.external("g" + k, g_leaf[k])
                self._zero[k] = p.ext_ptr["g" + k]
            lr_c = dev.const(lr)
            up = {k: weight_update(G.sub(params[k], G.mul(lr_c, g_leaf[k])), k) for k in self.names}
            # what a later phase reads is held on to explicitly: the first product (the backward pass re-derives the
            # GELU from it) and the gradient of the output (its matmuls are split over phases B1 and B2)
            taps["xw1"].keep = True
            if taps["out"].grad is not None:
                taps["out"].grad.keep = True
            # h is read by two matmuls of later phases and by nothing else: in "bf16" arithmetic it leaves phase F as a
            # bf16 matrix only (the backend hands back what it made; with other arithmetics the flag is not set)
            taps["h"].bf16 = bf16_matmuls
            p.add_phase([taps["h"]])                             # F
            p.add_phase([up["w2"], up["b2"]])                    # U2
            p.add_phase([loss, grads["w1"], grads["b1"]])        # B1
            p.add_phase([grads["w2"], grads["b2"]])              # B2
            p.add_phase([up["w1"], up["b1"]])                    # U1
            self._pending = None          # (dW2, db2) of the last step, still to be applied
        self.loss_ptr = None
        self.steps_done = 0
        self._initial = set(self.names)   # parameters still in the buffers the constructor uploaded
        # the build pass above already ran one step worth of kernels but did not move the parameters
        dev.sync()

    def _allreduce(self, entries, slot):
        n = len(entries)
        bufs = (ctypes.c_void_p * n)(*[e[0] for e in entries])
        counts = (ctypes.c_size_t * n)(*[e[1] // 4 for e in entries])
        check(lib.ormi_b200_allreduce_sum_f32(self.dev.handle, bufs, counts, n, 1 if self.overlap else 0))
        if self.overlap:
            check(lib.ormi_b200_comm_mark(self.dev.handle, slot))

    def _wait(self, slot):
        if self.overlap:
            check(lib.ormi_b200_comm_wait(self.dev.handle, slot))

    def _replace(self, name, new):
        """Parameter `name` now lives in `new`; its old buffer goes back to the pool unless the constructor's
        leaf still owns it."""
        p = self.prog
        if name in self._initial:
            self._initial.discard(name)
        else:
            self.dev.free(*p.ext_ptr[name])
        p.ext_ptr[name] = new

    def _apply_pending(self, outs):
        """U2: the second layer's update with the gradients the previous step left behind."""
        p = self.prog
        self._wait(2)
        res = p.run_phase(1, outs)
        self._replace("w2", res[0])
        self._replace("b2", res[1])
        if self._pending is not None:
            for buf in self._pending:
                self.dev.free(*buf)
            self._pending = None
        p.ext_ptr["gw2"], p.ext_ptr["gb2"] = self._zero["w2"], self._zero["b2"]
        return {res[0][0], res[1][0]}

    def step(self):
        p, dev = self.prog, self.dev
        outs: dict = {}
        if self.world == 1:
            res = p.run_phase(0, outs)
            loss = res[0]
            keep = {loss[0]}
            for i, k in enumerate(self.names):
                self._replace(k, res[1 + i])
                keep.add(res[1 + i][0])
        else:
            p.run_phase(0, outs)                                   # F
            keep = self._apply_pending(outs)                       # U2
            res = p.run_phase(2, outs)                             # B1
            loss, dw1, db1 = res[0], res[1], res[2]
            self._allreduce([dw1, db1, loss], 1)
            res = p.run_phase(3, outs)                             # B2
            dw2, db2 = res[0], res[1]
            self._allreduce([dw2, db2], 2)
            self._wait(1)
            p.ext_ptr["gw1"], p.ext_ptr["gb1"] = dw1, db1
            res = p.run_phase(4, outs)                             # U1
            self._replace("w1", res[0])
            self._replace("b1", res[1])
            self._pending = (dw2, db2)
            p.ext_ptr["gw2"], p.ext_ptr["gb2"] = dw2, db2
            keep |= {res[0][0], res[1][0], dw2[0], db2[0], loss[0]}
        # everything else this step produced goes back to the pool (stream-ordered: kernels already queued finish first)
        for ptr, nbytes in outs.get("owned", []):
            if ptr not in keep:
                dev.free(ptr, nbytes)
        if self.loss_ptr is not None:
            dev.free(*self.loss_ptr)
        self.loss_ptr = loss
        self.steps_done += 1

    def flush(self):
        """Applies the update a multi-rank step leaves pending (W2, b2), so that `parameter` sees step-complete values."""
        if self.world > 1 and self._pending is not None:
            outs: dict = {}
            keep = self._apply_pending(outs)
            for ptr, nbytes in outs.get("owned", []):
                if ptr not in keep:
                    self.dev.free(ptr, nbytes)

    def loss(self) -> float:
        """Global loss of the last step (already summed over ranks when world > 1)."""
        out = np.empty(1, dtype=np.float32)
        self.dev.d2h(out, self.loss_ptr[0])
        return float(out[0])

    def parameter(self, name: str) -> np.ndarray:
        self.flush()
        ptr, nbytes = self.prog.ext_ptr[name]
        out = np.empty(nbytes // 4, dtype=np.float32)
        self.dev.d2h(out, ptr)
        return out


def init_comm(dev, rank: int, world: int, broadcast: Callable[[bytes | None], bytes]):
    """Creates the NCCL communicator of `dev`.  `broadcast(payload_or_None)` must return rank 0's 128-byte id on
    every rank (torch.distributed, MPI, a shared file — whatever the host has)."""
    buf = ctypes.create_string_buffer(128)
    if rank == 0:
        check(lib.ormi_b200_comm_unique_id(buf))
    uid = broadcast(bytes(buf.raw) if rank == 0 else None)
    check(lib.ormi_b200_comm_init(dev.handle, uid, rank, world))
