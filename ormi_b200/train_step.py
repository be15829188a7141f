"""A repeated training step over the graph API, batch-sharded over ranks.

The step is ordinary Ormi graph code (ormi_b200.workloads.mlp_loss, compute_gradients, sgd_update).  What this
module adds is the host loop a data-parallel job needs around ``ormi_b200_realize``:

* the step is split into *phases* (roots that are realized together).  Between phases the gradients that are
  already complete go out through ``ormi_b200_allreduce_sum_f32`` on the second stream, so the all-reduce of the
  last layer's gradients overlaps the GEMMs that produce the first layer's;
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
        self.dev.realize(list(roots))
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
        check(lib.ormi_b200_realize(self.dev.handle, ph.arr, ph.n, ph.ridx, len(ph.roots)))
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
    """

    def __init__(self, dev, x, t, w1, b1, w2, b2, lr: float, global_batch: int | None = None, world: int = 1,
                 overlap: bool = True):
        self.dev, self.world, self.overlap = dev, world, overlap
        B, D = x.shape[0], t.shape[1]
        self.global_batch = global_batch or B * world
        scale = 1.0 / (self.global_batch * D)
        p = self.prog = StepProgram(dev)
        xn, tn = dev.leaf(x), dev.leaf(t)
        params = {k: dev.leaf(v, True) for k, v in (("w1", w1), ("b1", b1), ("w2", w2), ("b2", b2))}
        for k, n in (("x", xn), ("t", tn), *params.items()):
            p.external(k, n)
        loss = W.mlp_loss(xn, params["w1"], params["b1"], params["w2"], params["b2"], tn, scale=scale)
        G.compute_gradients(loss)
        self.names = ["w1", "b1", "w2", "b2"]
        grads = {k: params[k].grad for k in self.names}
        if world == 1:
            ups = [W.sgd_update(params[k], lr) for k in self.names]
            p.add_phase([loss] + ups)
        else:
            # backward in two phases so the last layer's gradients travel while the first layer's are computed
            p.add_phase([loss, grads["w2"], grads["b2"]])
            p.add_phase([grads["w1"], grads["b1"]])
            g_leaves = {}
            for k in self.names:           # the update reads the summed gradients as plain inputs
                g_leaves[k] = G.Node(G.OpEnum.LEAF, data=grads[k].data)
                p.produced[id(g_leaves[k])] = p.produced[id(grads[k])]
            self._grad_ids = {k: id(grads[k]) for k in self.names}
            self._gleaf_ids = {k: id(g_leaves[k]) for k in self.names}
            lr_c = dev.const(lr)
            ups = [G.sub(params[k], G.mul(lr_c, g_leaves[k])) for k in self.names]
            p.add_phase(ups)
        self._loss_id = id(loss)
        self.loss_ptr = None
        self.steps_done = 0
        # the build pass above already ran one step worth of kernels but did not move the parameters
        dev.sync()

    def _allreduce(self, entries, overlap):
        n = len(entries)
        bufs = (ctypes.c_void_p * n)(*[e[0] for e in entries])
        counts = (ctypes.c_size_t * n)(*[e[1] // 4 for e in entries])
        check(lib.ormi_b200_allreduce_sum_f32(self.dev.handle, bufs, counts, n, 1 if overlap else 0))

    def step(self):
        p, dev = self.prog, self.dev
        outs: dict = {}
        if self.world == 1:
            res = p.run_phase(0, outs)
            new_params = {k: res[1 + i] for i, k in enumerate(self.names)}
            loss = res[0]
        else:
            res0 = p.run_phase(0, outs)
            loss = res0[0]
            self._allreduce([res0[1], res0[2], loss], self.overlap)
            res1 = p.run_phase(1, outs)
            self._allreduce([res1[0], res1[1]], self.overlap)
            if self.overlap:
                check(lib.ormi_b200_comm_join(dev.handle))
            for k in self.names:
                outs[self._gleaf_ids[k]] = outs[self._grad_ids[k]]
            res2 = p.run_phase(2, outs)
            new_params = {k: res2[i] for i, k in enumerate(self.names)}
        # parameters ping-pong; everything else this step produced goes back to the pool
        keep = {v[0] for v in new_params.values()} | {loss[0]}
        for k in self.names:
            old = p.ext_ptr[k]
            if self.steps_done > 0:
                dev.free(*old)
            p.ext_ptr[k] = new_params[k]
        for ptr, nbytes in outs.get("owned", []):
            if ptr not in keep:
                dev.free(ptr, nbytes)
        if self.loss_ptr is not None:
            dev.free(*self.loss_ptr)
        self.loss_ptr = loss
        self.steps_done += 1

    def loss(self) -> float:
        """Global loss of the last step (already summed over ranks when world > 1)."""
        out = np.empty(1, dtype=np.float32)
        self.dev.d2h(out, self.loss_ptr[0])
        return float(out[0])

    def parameter(self, name: str) -> np.ndarray:
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
