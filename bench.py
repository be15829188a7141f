#!/usr/bin/env python
"""Benchmark of the realize path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (configs[1] of the baseline description): row softmax and layernorm, forward plus the
autograd-generated backward, on x[16384, 4096] fp32 per GPU.  One step realizes both graphs once.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank owns its own 16384-row
shard (weak scaling); the only exchange is the all-reduce of the two [4096] parameter gradients.

Prints ONE JSON line (rank 0): the metric is algorithmic HBM traffic per second.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

R, C = 16384, 4096
METRIC, UNIT = "fused_graph_hbm_gbps", "GB/s"
WORKLOAD = "configs[1]: row softmax + layernorm, forward + autograd backward, x[16384,4096] fp32 per GPU"
# algorithmic bytes of one step (per GPU): softmax reads x, gy and writes y, dx; layernorm reads x, gy, g, b and
# writes y, dx, dg, db.  Nothing is saved between forward and backward: both run in one kernel per graph.
BYTES_SOFTMAX = 4 * R * C * 4
BYTES_LAYERNORM = 4 * R * C * 4 + 4 * C * 4
BYTES_STEP = BYTES_SOFTMAX + BYTES_LAYERNORM
# The two graphs read the same x and gy.  Realized in ONE call they become one kernel that reads each once: what that
# kernel must move is x, gy in and y, dx of both graphs out (plus g, b, dg, db).
BYTES_FUSED_KERNEL = 6 * R * C * 4 + 4 * C * 4
# DRAM traffic of the dominant kernel from its ncu capture (profiles/rows_softmax_layernorm_one_call_8192x4096.md), per
# launch over 8192 rows; the traffic is proportional to the rows, the bench launch covers 16384.
FUSED_READ_8192, FUSED_WRITE_8192 = 268_499_712, 482_261_760
STEP_TRAFFIC_BYTES = 2 * (FUSED_READ_8192 + FUSED_WRITE_8192)
STEP_TRAFFIC_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 8192 rows (750.8 MB), times 2 for 16384 rows"
STEP_KERNEL = ("one fused kernel for both graphs (rows template: softmax and layernorm forward+backward of the same x and gy, "
               "each read once) + its finalize launch (partials of dg and db)")


_REAL_STDOUT = None


def emit(obj):
    """The one JSON line of the run, on the process's original stdout."""
    text = (json.dumps(obj) + "\n").encode()
    sys.stdout.flush()
    os.write(_REAL_STDOUT if _REAL_STDOUT is not None else 1, text)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def build_graphs(G, W, leaf, rows=R, shard=0):
    """The two graphs of a step over `rows` rows; returns (roots, inputs) with inputs = dict of leaf nodes.
    x ~ N(0, 2) (variance 2), gy ~ N(0, 1), g ~ U(0.5, 1.5), b ~ N(0, 0.1); shard s draws x, gy from seeds 100 s + {0, 1}."""
    x = leaf(W.normal(100 * shard, (rows, C), math.sqrt(2.0)), True)
    gy = leaf(W.normal(100 * shard + 1, (rows, C)))
    g = leaf(W.uniform(2, (C,), 0.5, 1.5), True)
    b = leaf(W.normal(3, (C,), 0.1), True)
    y = W.softmax(x)
    y.grad = gy
    G.compute_gradients(y)
    sm_roots = [y, x.grad]
    x.grad = None
    y2 = W.layernorm(x, g, b)
    y2.grad = gy
    G.compute_gradients(y2)
    ln_roots = [y2, x.grad, g.grad, b.grad]
    return sm_roots, ln_roots, dict(x=x, gy=gy, g=g, b=b)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "samples": len(sm), "reasons": sorted(reasons)}


class StepRunner:
    """Realizes the two cached graphs through the C ABI, the way a host loop over the graph API does: the flattened
    graph is handed to ormi_b200_realize every step, results are dropped (returned to the pool) afterwards."""

    def __init__(self, dev, G, roots_list):
        from ormi_b200._lib import lib, check
        self.dev, self.lib, self.check, self.G = dev, lib, check, G
        self.graphs = []
        for roots in roots_list:
            order = G.topo_order(roots, stop_at_realized=True)
            dev.ensure_on_device(order)
            arr, order, ridx = G.flatten(roots, host_pointers=False, stop_at_realized=True)
            template = bytes(arr)
            self.graphs.append((arr, template, len(order), (ctypes.c_int * len(ridx))(*ridx), ridx, order))

    def run(self, which=None, keep=False):
        outs = []
        for gi, (arr, template, n, ridx, ridx_list, order) in enumerate(self.graphs):
            if which is not None and gi != which:
                continue
            ctypes.memmove(arr, template, len(template))
            self.check(self.lib.ormi_b200_realize(self.dev.handle, arr, n, ridx, len(ridx_list)))
            kept = {}
            for i in range(n):
                c = arr[i]
                if c.flags & self.G.NODE_OWNED:
                    if keep and i in ridx_list:
                        kept[i] = (c.data, c.data_bytes)
                    else:
                        self.dev.free(c.data, c.data_bytes)
            outs.extend(kept[i] for i in ridx_list if i in kept)      # in the order of the roots
        return outs


def timed(dev, torch, fn, steps, dist=None, after=None):
    stream = torch.cuda.ExternalStream(dev.stream)
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        fn()
    if after is not None:
        after()             # still inside the timed region (e.g. the wait for the last step's all-reduce)
    e1.record(stream)
    e1.synchronize()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


CPU_ROWS_PER_WORKER = 256      # rows of the configs[1] workload one CPU worker realizes per step


def _cpu_worker(arg):
    """One worker: `rows` rows of the step (softmax + layernorm, forward + backward) on the reference CPU backend —
    the unmodified reference from oracle/_ref, or its C restatement when that library is absent.  Returns the seconds
    spent in autograd + realize."""
    seed, rows = arg
    from ormi_b200 import graph as G, workloads as W
    from oracle import oracle as O
    x = G.leaf(W.normal(100 * seed, (rows, C), math.sqrt(2.0)), True)
    gy = G.leaf(W.normal(100 * seed + 1, (rows, C)))
    g = G.leaf(W.uniform(2, (C,), 0.5, 1.5), True)
    b = G.leaf(W.normal(3, (C,), 0.1), True)
    if O.ref_available():
        y = W.softmax(x)
        _, s1 = O.ref_run([(y, "value"), (x, "grad")], seeds=[(y, gy)], backward_root=y, caps=[rows * C] * 2)
        y2 = W.layernorm(x, g, b)
        _, s2 = O.ref_run([(y2, "value"), (x, "grad"), (g, "grad"), (b, "grad")], seeds=[(y2, gy)], backward_root=y2,
                          caps=[rows * C] * 4)
    else:
        sm, ln, _ = build_graphs(G, W, G.leaf, rows, shard=seed)
        _, s1 = O.port_run(sm)
        _, s2 = O.port_run(ln)
    return s1 + s2


class CpuReference:
    """The reference's CPU implementation of the path on the host cores of this machine.  Its realize path is single
    threaded (one interpreter loop per node), and rows are independent, so every core gets a worker process with its
    own rows: the aggregate is what the host can do with the reference code.  One step = workers x 256 rows."""

    def __init__(self, max_workers=None):
        from oracle import oracle as O
        import multiprocessing as mp
        self.kind = "reference" if O.ref_available() else "port"
        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        self.workers = max(1, min(cores, max_workers or 32))
        self.pool = None
        if self.workers > 1:
            try:
                self.pool = mp.get_context("fork").Pool(self.workers)
                self.pool.map(_cpu_worker, [(i, 8) for i in range(self.workers)])      # load libraries, touch memory
            except Exception:
                self.pool, self.workers = None, 1
        self.rows = self.workers * CPU_ROWS_PER_WORKER
        self.sample = (f"{self.workers} worker process(es) x {CPU_ROWS_PER_WORKER} rows = {self.rows} of {R} rows per step "
                       "(same graphs, seeded rows), autograd + realize on the reference CPU backend, wall clock over all workers")

    def step(self):
        """Runs one sample; returns (wall seconds, seconds of the slowest single worker)."""
        args = [(i, CPU_ROWS_PER_WORKER) for i in range(self.workers)]
        t0 = time.perf_counter()
        secs = self.pool.map(_cpu_worker, args) if self.pool else [_cpu_worker(a) for a in args]
        return time.perf_counter() - t0, max(secs)

    def gbps(self, wall):
        return BYTES_STEP * self.rows / R / wall / 1e9

    def close(self):
        if self.pool:
            self.pool.close()
            self.pool.join()


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cpu = CpuReference()
    for _ in range(args.warmup):
        cpu.step()
    t0 = time.perf_counter()
    one_core = []
    for _ in range(args.steps):
        _, slowest = cpu.step()
        one_core.append(slowest)
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    value = cpu.gbps(ms * 1e-3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": R, "cols": C, "cpu_sample": cpu.sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.workers, "kind": cpu.kind, "sample": cpu.sample,
                         "one_core_gbps": BYTES_STEP * CPU_ROWS_PER_WORKER / R / float(np.median(one_core)) / 1e9},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    cpu.close()
    emit(line)


def matmul_sweep(dev, torch, G, W, steps=5):
    """configs[2]: C = A @ B.  fp32 on the SIMT FFMA path through the graph; bf16 on the tcgen05 kernel with operands
    already in bf16 in HBM (the conversion pass is timed on its own) and through the graph (operands found in the
    context's bf16 cache, as in a loop that reuses them); the opt-in tf32 / 3xTF32 fp32 modes through the graph.
    cuBLAS (torch.matmul, TF32 off for fp32) on the same box is the comparator, never part of the product path."""
    from ormi_b200._lib import lib, check
    out = {}
    torch.backends.cuda.matmul.allow_tf32 = False
    P = ctypes.c_void_p
    for (M, N, K) in [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192), (8192, 1024, 8192)]:
        a = dev.leaf(W.normal(0, (M, K), 1 / math.sqrt(K)))
        b = dev.leaf(W.normal(1, (K, N), 1 / math.sqrt(K)))
        flop = 2.0 * M * N * K
        rec = {}
        n_slow = steps if flop < 3e11 else 2

        def through_graph(mode, n):
            dev.set_option("matmul", mode)
            runner = StepRunner(dev, G, [[G.matmul(a, b)]])
            for _ in range(3):
                runner.run()
            return flop / (timed(dev, torch, lambda: runner.run(), n) / n * 1e-3) / 1e12

        rec["fp32_ffma_tflops"] = through_graph("fp32", n_slow)
        rec["tf32_tflops"] = through_graph("tf32", 2 * steps)
        rec["3xtf32_tflops"] = through_graph("3xtf32", steps)
        rec["bf16_graph_tflops"] = through_graph("bf16", 2 * steps)
        a16, b16, c = dev.alloc(M * K * 2), dev.alloc(K * N * 2), dev.alloc(M * N * 4)
        h = dev.handle

        def cvt():
            check(lib.ormi_b200_cvt_bf16(h, P(a.data.dev_ptr), K, M, K, P(a16)))
            check(lib.ormi_b200_cvt_bf16(h, P(b.data.dev_ptr), N, K, N, P(b16)))

        def gemm():
            check(lib.ormi_b200_gemm_bf16(h, P(a16), 0, P(b16), 0, P(c), M, N, K))

        for _ in range(3):
            cvt(); gemm()
        rec["bf16_convert_ms"] = timed(dev, torch, cvt, steps) / steps
        rec["bf16_tcgen05_tflops"] = flop / (timed(dev, torch, gemm, 4 * steps) / (4 * steps) * 1e-3) / 1e12
        for ptr, nbytes in ((a16, M * K * 2), (b16, K * N * 2), (c, M * N * 4)):
            dev.free(ptr, nbytes)
        dev.sync()
        # comparators: cuBLAS through torch, same shapes, same box, same run
        for name, dt, n in (("cublas_bf16_tflops", torch.bfloat16, 4 * steps), ("cublas_sgemm_tflops", torch.float32, n_slow)):
            ta = torch.randn(M, K, device="cuda", dtype=dt) / math.sqrt(K)
            tb = torch.randn(K, N, device="cuda", dtype=dt) / math.sqrt(K)
            for _ in range(3):
                torch.matmul(ta, tb)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n):
                torch.matmul(ta, tb)
            e1.record()
            e1.synchronize()
            rec[name] = flop / (e0.elapsed_time(e1) / n * 1e-3) / 1e12
            del ta, tb
        out[f"{M}x{N}x{K}"] = rec
        del a, b
    dev.set_option("matmul", "fp32")
    return out


def rowsum_config0(dev, torch, G, W, peak, steps=20):
    """configs[0]: y = sum(relu(a*b + c) * exp(-|a|), axis=1) on [4096, 4096] fp32, one generated kernel.  Three input
    sets are rotated, so that no launch finds its 201 MB of operands left in L2 by the one before."""
    n = 4096
    sets = []
    for k in range(3):
        a, b, c = (dev.leaf(W.normal(10 * k + i, (n, n))) for i in range(3))
        sets.append(StepRunner(dev, G, [[W.fused_rowsum(a, b, c)]]))
    nbytes = 3 * n * n * 4 + n * 4
    state = {"i": 0}

    def run():
        sets[state["i"] % 3].run()
        state["i"] += 1

    for _ in range(6):
        run()
    ms = timed(dev, torch, run, 3 * steps) / (3 * steps)
    gbps = nbytes / (ms * 1e-3) / 1e9
    return {"gbps": gbps, "us_per_launch": ms * 1e3, "frac": gbps / peak, "algorithmic_bytes": nbytes,
            "l2": "3 input sets of 201 MB rotated", "shape": "a, b, c [4096,4096] fp32 -> y [4096]"}


def mlp_steps_per_s(dev, torch, W, batch, d_in, hidden, matmul, steps, rank=0, world=1, dist=None, global_batch=None):
    """configs[3] / configs[4]: full training step (forward, autograd backward, SGD update) of the 2-layer MLP."""
    from ormi_b200.train_step import MLPTrainer
    dev.set_option("matmul", matmul)
    # ONE seeded global batch whatever the number of ranks; this rank takes its rows of it
    rows = slice(rank * batch, (rank + 1) * batch)
    x = np.ascontiguousarray(W.normal(1000, (batch * world, d_in))[rows])
    t = np.ascontiguousarray(W.normal(2000, (batch * world, d_in))[rows])
    w1, w2 = W.kaiming_uniform(2, d_in, (d_in, hidden)), W.kaiming_uniform(3, hidden, (hidden, d_in))
    b1, b2 = np.zeros(hidden, np.float32), np.zeros(d_in, np.float32)
    tr = MLPTrainer(dev, x, t, w1, b1, w2, b2, lr=0.05, global_batch=global_batch or batch * world, world=world)
    for _ in range(3):
        tr.step()
    dev.sync()
    first = tr.loss()
    ms = timed(dev, torch, tr.step, steps, dist) / steps
    last = tr.loss()
    dev.set_option("matmul", "fp32")
    flop = 5 * 2.0 * batch * world * d_in * hidden
    return {"steps_per_s": 1e3 / ms, "ms_per_step": ms, "gemm_tflops_per_gpu": flop / world / (ms * 1e-3) / 1e12,
            "loss_first": first, "loss_last": last}


def mlp_sharded_vs_single(dev, W, rank, world, dist, d_in=2048, hidden=8192, rows_per_rank=512, steps=3):
    """Numerical parity of the sharded step: the N-rank trainer against a single-rank trainer fed the whole of the same
    reduced batch (configs[4] widths, rows_per_rank x N rows), after `steps` SGD steps.  Returns, on rank 0, the largest
    of |loss_N - loss_1| / |loss_1| and max|p_N - p_1| / max|p_1| over the four parameters."""
    from ormi_b200.train_step import MLPTrainer
    dev.set_option("matmul", "bf16")
    B = rows_per_rank * world
    x, t = W.normal(3000, (B, d_in)), W.normal(3001, (B, d_in))
    w1, w2 = W.kaiming_uniform(2, d_in, (d_in, hidden)), W.kaiming_uniform(3, hidden, (hidden, d_in))
    b1, b2 = W.normal(4, (hidden,), 0.1), W.normal(5, (d_in,), 0.1)
    rows = slice(rank * rows_per_rank, (rank + 1) * rows_per_rank)
    tr = MLPTrainer(dev, np.ascontiguousarray(x[rows]), np.ascontiguousarray(t[rows]), w1, b1, w2, b2, lr=0.05, global_batch=B, world=world)
    for _ in range(steps):
        tr.step()
    loss = tr.loss()
    params = [tr.parameter(n) for n in tr.names]
    err = None
    if rank == 0:
        solo = MLPTrainer(dev, x, t, w1, b1, w2, b2, lr=0.05)
        for _ in range(steps):
            solo.step()
        errs = [abs(loss - solo.loss()) / abs(solo.loss())]
        for n, got in zip(solo.names, params):
            want = solo.parameter(n)
            errs.append(float(np.abs(got - want).max() / np.abs(want).max()))
        err = max(errs)
        del solo
    del tr
    dist.barrier()
    dev.set_option("matmul", "fp32")
    return err


def run_mlp_sharded(args, rank, local_rank, world):
    """configs[4] alone, under torch.distributed.run: the global batch of --rows x world rows split over the ranks."""
    import torch
    import torch.distributed as dist
    from ormi_b200 import workloads as W
    from ormi_b200.runtime import Device
    from ormi_b200.train_step import init_comm
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = Device(local_rank)
    for item in filter(None, args.set.split(",")):
        k, v = item.split("=")
        dev.set_option(k, v)

    def bcast(payload):
        obj = [payload]
        dist.broadcast_object_list(obj, src=0)
        return obj[0]
    if world > 1:
        init_comm(dev, rank, world, bcast)
    res = mlp_steps_per_s(dev, torch, W, args.rows, 2048, 8192, "bf16", args.steps, rank, world, dist if world > 1 else None, args.rows * world)
    if rank == 0:
        emit(dict(res, only=args.only, rows_per_rank=args.rows, world=world, options=args.set))
    dist.destroy_process_group()
    dev.close()


def run_only(args):
    """One graph, a few launches, nothing else: the small case profilers attach to."""
    import torch
    from ormi_b200 import graph as G, workloads as W
    from ormi_b200.runtime import Device
    dev = Device(0)
    if args.only in ("mlp_bf16", "mlp_fp32"):
        # one rank's share of the MLP training step: --rows rows of the batch (8192 = one of 8 ranks of configs[4])
        wide = args.only == "mlp_bf16"
        res = mlp_steps_per_s(dev, torch, W, args.rows, 2048 if wide else 1024, 8192 if wide else 4096,
                              "bf16" if wide else "fp32", args.steps)
        emit((dict(res, only=args.only, rows=args.rows)))
        dev.close()
        return
    if args.only.startswith("gemm_"):
        # C = A @ B at M = N = K = --rows (default 8192 is too long under a profiler: use --rows 4096)
        n = args.rows
        a = dev.leaf(W.normal(0, (n, n), 1 / math.sqrt(n)))
        b = dev.leaf(W.normal(1, (n, n), 1 / math.sqrt(n)))
        dev.set_option("matmul", args.only[len("gemm_"):])      # fp32 | bf16 | tf32 | 3xtf32
        runner = StepRunner(dev, G, [[G.matmul(a, b)]])
        for _ in range(args.warmup):
            runner.run()
        ms = timed(dev, torch, lambda: runner.run(), args.steps)
        emit(({"only": args.only, "n": n, "ms_per_matmul": ms / args.steps,
                          "tflops_including_conversion": 2.0 * n ** 3 / (ms / args.steps * 1e-3) / 1e12}))
        dev.close()
        return
    if args.only == "rowsum":
        a, b, c = (dev.leaf(W.normal(i, (args.rows, C))) for i in range(3))
        roots, nbytes = [W.fused_rowsum(a, b, c)], 3 * args.rows * C * 4 + args.rows * 4
    elif args.only == "softmax_stable":
        # extension op MAX: the row maximum is subtracted first; forward + autograd backward, still one kernel
        x = dev.leaf(W.normal(0, (args.rows, C), math.sqrt(2.0)), True)
        y = W.softmax_stable(x)
        y.grad = dev.leaf(W.normal(1, (args.rows, C)))
        G.compute_gradients(y)
        roots, nbytes = [y, x.grad], 4 * args.rows * C * 4
    else:
        sm, ln, _ = build_graphs(G, W, lambda a, rg=False: dev.leaf(a, rg), rows=args.rows)
        roots = sm if args.only == "softmax" else (ln if args.only == "layernorm" else sm + ln)
        nbytes = (6 if args.only == "fused_step" else 4) * args.rows * C * 4
    runner = StepRunner(dev, G, [roots])
    for _ in range(args.warmup):
        runner.run()
    ms = timed(dev, torch, lambda: runner.run(), args.steps)
    emit(({"only": args.only, "rows": args.rows, "cols": C, "ms_per_launch": ms / args.steps,
                      "algorithmic_bytes": nbytes, "gbps": nbytes / (ms / args.steps * 1e-3) / 1e9}))
    dev.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default=None, choices=["softmax", "softmax_stable", "layernorm", "fused_step", "rowsum", "gemm_bf16", "gemm_fp32", "gemm_tf32", "gemm_3xtf32", "mlp_bf16", "mlp_fp32", "mlp_sharded"],
                    help="profiling aid: run just this graph --steps times on --rows rows and exit")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--no-extras", action="store_true", help="skip the matmul sweep and the MLP training steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--e2e-chunk", type=int, default=1024, help="rows per chunk of the pipelined end-to-end step (a divisor of 16384)")
    ap.add_argument("--set", default="", help="with --only mlp_sharded: backend options for the run, key=value,key=value")
    args = ap.parse_args()
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line there.  Everything but
    # that line goes to stderr.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    warmup = max(3, args.warmup)
    if args.only == "mlp_sharded":
        return run_mlp_sharded(args, rank, local_rank, world)
    if args.only:
        return run_only(args)

    # The CPU baseline leg runs first, before this process touches CUDA (its worker processes are forked): the
    # reference CPU backend on the same sample the reference arm steps over, best of a few repeats.
    cpu_rec = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = CpuReference()
        walls = [cpu.step()[0] for _ in range(6)]
        cpu_rec = {"value": cpu.gbps(min(walls)), "unit": UNIT, "cores": cpu.workers, "kind": cpu.kind,
                   "sample": cpu.sample + f"; best of {len(walls)} repeats ({sum(walls):.1f} s of wall clock in all)"}
        cpu.close()

    import torch
    from ormi_b200 import graph as G, workloads as W
    from ormi_b200.runtime import Device
    from ormi_b200._lib import lib, check

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod
    dev = Device(local_rank)

    # inputs resident in HBM; each rank draws its own shard (seed offset by rank)
    sm_roots, ln_roots, inputs = build_graphs(G, W, lambda a, rg=False: dev.leaf(a, rg), shard=rank)
    runner = StepRunner(dev, G, [sm_roots, ln_roots])            # the two graphs in separate calls (kernels timed alone)
    fused = StepRunner(dev, G, [sm_roots + ln_roots])           # the step: one realize call for all six results

    if dist is not None:
        from ormi_b200.train_step import init_comm

        def bcast(payload):
            obj = [payload]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        init_comm(dev, rank, world, bcast)

    pending = []        # results of the previous step whose all-reduce may still be in flight on the second stream

    def settle():
        """The compute stream waits for the previous step's all-reduce; its buffers go back to the pool."""
        if pending:
            check(lib.ormi_b200_comm_join(dev.handle))
            for ptr, nbytes in pending:
                dev.free(ptr, nbytes)
            pending.clear()

    def step():
        if dist is None:
            fused.run()
            return
        # cross-shard combine: dg, db (the last two roots) are summed over the ranks, in place, by NCCL on the second
        # stream.  Nothing of the next step reads them; the compute stream waits for the all-reduce (a latency of some
        # 25 us for 2 x 16 KB) before the next step's kernel, whose blocks have fixed row shares and must not find SMs
        # taken.  No host synchronisation inside a step.
        settle()
        outs = fused.run(keep=True)
        bufs = (ctypes.c_void_p * 2)(outs[-2][0], outs[-1][0])
        counts = (ctypes.c_size_t * 2)(C, C)
        check(lib.ormi_b200_allreduce_sum_f32(dev.handle, bufs, counts, 2, 1))
        pending.extend(outs)

    for _ in range(warmup):
        step()
        runner.run()            # the two graphs in calls of their own are timed further down: compiled and warm by then
    dev.sync()
    # The dominant kernel alone right after the warm-up, before the GPU has been under load for a second: the state the
    # copy-bandwidth peak was measured in (a burst).  `roofline.achieved` is the same measurement taken after the timed
    # region, under the power cap the long run settles into; both are reported.
    settle()
    fused.run()
    dev.sync()
    ms_fused_burst = timed(dev, torch, lambda: fused.run(), args.steps, dist)
    # nvidia-smi samples every 100 ms and the timed region lasts milliseconds, so the same step keeps the GPU under
    # load for about a second before and after the timed region: the clock samples bracket it.
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    load_steps = max(1, int(1.2 / 0.0008))
    for _ in range(load_steps):
        step()
    settle()
    dev.sync()
    launches0 = dev.counter("launches")
    ms_total = timed(dev, torch, step, args.steps, dist, after=settle)
    launches = dev.counter("launches") - launches0
    # the dominant kernel (with its finalize launch) alone, and the two graphs in calls of their own
    ms_fused = timed(dev, torch, lambda: fused.run(), args.steps, dist)
    ms_ln = timed(dev, torch, lambda: runner.run(which=1), args.steps, dist)
    ms_sm = timed(dev, torch, lambda: runner.run(which=0), args.steps, dist)
    for _ in range(300):
        step()
    settle()
    dev.sync()
    clocks = sampler.stop() if rank == 0 else None
    # the same step recorded once (ormi_b200_capture_begin / _end) and replayed with one call per step
    graph_ms = None
    if dist is None and not args.no_extras:
        with dev.capture() as captured:
            fused.run()
        for _ in range(3):
            captured.launch()
        graph_ms = timed(dev, torch, captured.launch, args.steps) / args.steps
        captured.destroy()

    # ------------------------------------------------------------------------------------------------ end to end
    # Host buffers in, host buffers out, through the public Device API, pipelined: the step is row independent, so it
    # runs in chunks of E2E_CHUNK rows — uploads on the upload stream, the kernels of chunk k as soon as its rows have
    # arrived, its results back on the download stream while later chunks upload and compute.  dg, db come back as one
    # partial per chunk and are added on the host (and, with N > 1, summed over the ranks on the device first).
    E2E_CHUNK = args.e2e_chunk
    n_chunks = R // E2E_CHUNK
    host_in = {k: torch.from_numpy(np.ascontiguousarray(v.data.host if v.data.host is not None else dev.download(v.data))).pin_memory()
               for k, v in inputs.items()}
    host_out = [torch.empty(R * C, dtype=torch.float32).pin_memory() for _ in range(4)]
    host_part = torch.empty(n_chunks * 2 * C, dtype=torch.float32).pin_memory()
    h2d = sum(t.numel() * 4 for t in host_in.values())
    d2h = sum(t.numel() * 4 for t in host_out) + host_part.numel() * 4
    # every chunk has device inputs of its own (together: the full-size x and gy), so the uploads of a step are all
    # queued at its start and run at the full one-direction rate; the kernels of chunk k wait for exactly chunk k's upload
    chunk_sets = []
    for _ in range(n_chunks):
        csm, cln, cin = build_graphs(G, W, lambda a, rg=False: dev.leaf(a, rg), rows=E2E_CHUNK, shard=rank)
        chunk_sets.append((StepRunner(dev, G, [csm + cln]), cin))
    np_in = {k: t.numpy() for k, t in host_in.items()}
    np_out = [t.numpy() for t in host_out]
    np_part = host_part.numpy()

    def upload(k):
        _, cin = chunk_sets[k]
        rows = slice(k * E2E_CHUNK * C, (k + 1) * E2E_CHUNK * C)
        # nothing on the device still reads these buffers: the previous step ended with the host waiting for its downloads
        dev.h2d_async(cin["x"].data.dev_ptr, np_in["x"].reshape(-1)[rows], False)
        dev.h2d_async(cin["gy"].data.dev_ptr, np_in["gy"].reshape(-1)[rows], False)
        dev.h2d_async(cin["g"].data.dev_ptr, np_in["g"].reshape(-1), False)
        dev.h2d_async(cin["b"].data.dev_ptr, np_in["b"].reshape(-1), False)
        dev.upload_mark(k)

    def e2e_step():
        held = []
        for k in range(n_chunks):
            upload(k)
        for k in range(n_chunks):
            dev.upload_wait(k)                   # the compute stream waits for chunk k's upload, not for the later ones
            outs = chunk_sets[k][0].run(keep=True)
            if dist is not None:
                bufs = (ctypes.c_void_p * 2)(outs[-2][0], outs[-1][0])
                counts = (ctypes.c_size_t * 2)(C, C)
                check(lib.ormi_b200_allreduce_sum_f32(dev.handle, bufs, counts, 2, 0))
            rows = slice(k * E2E_CHUNK * C, (k + 1) * E2E_CHUNK * C)
            for (ptr, nbytes), host in zip(outs[:4], np_out):
                dev.d2h_async(host[rows], ptr)
            dev.d2h_async(np_part[(2 * k) * C:(2 * k + 1) * C], outs[4][0])
            dev.d2h_async(np_part[(2 * k + 1) * C:(2 * k + 2) * C], outs[5][0])
            held.append(outs)
        dev.copy_wait(1)                         # the host waits for the downloads
        for outs in held:
            for ptr, nbytes in outs:
                dev.free(ptr, nbytes)
        part = np_part.reshape(n_chunks, 2, C)
        return part[:, 0].sum(axis=0), part[:, 1].sum(axis=0)

    def copy_rate(fn, nbytes):
        dev.sync()
        t0 = time.perf_counter()
        fn()
        return nbytes / (time.perf_counter() - t0) / 1e9

    big = dev.alloc(R * C * 4)
    h2d_gbps = copy_rate(lambda: (dev.h2d_async(big, np_in["x"].reshape(-1), False), dev.copy_wait(0), dev.sync()), R * C * 4)
    d2h_gbps = copy_rate(lambda: (dev.d2h_async(np_out[0], big), dev.copy_wait(1)), R * C * 4)
    dev.free(big, R * C * 4)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    dev.sync()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    dev.sync()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())

    # the other legs of the metric: configs[0], matmul TFLOP/s (configs[2]) and MLP training steps/s (configs[3], [4])
    extras = {}
    if graph_ms is not None:
        extras["step_graph_replay"] = {"ms_per_step": graph_ms, "gbps": BYTES_STEP / (graph_ms * 1e-3) / 1e9,
                                       "note": "the headline step captured into a CUDA graph and replayed: one host call per step (timed after a pause of the sustained load: compare with roofline.burst, not with value)"}
    peak, peak_src = peaks()
    if not args.no_extras:
        del runner, fused, host_in, host_out, host_part, np_in, np_out, np_part, chunk_sets
        for node in inputs.values():
            node.data = None
        inputs.clear()
        sm_roots.clear(); ln_roots.clear()
        import gc
        gc.collect()
        check(lib.ormi_b200_trim(dev.handle))
        if world == 1:
            extras["rowsum_config0"] = rowsum_config0(dev, torch, G, W, peak)
            check(lib.ormi_b200_trim(dev.handle))
            extras["matmul"] = matmul_sweep(dev, torch, G, W)
            gc.collect()
            check(lib.ormi_b200_trim(dev.handle))
            extras["mlp_fp32_config3"] = dict(mlp_steps_per_s(dev, torch, W, 8192, 1024, 4096, "fp32", 5),
                                              shape="B=8192, 1024->4096->1024, fp32 FFMA matmuls")
            gc.collect()
            check(lib.ormi_b200_trim(dev.handle))
        gb = 65536
        extras["mlp_bf16_config4"] = dict(mlp_steps_per_s(dev, torch, W, gb // world, 2048, 8192, "bf16", 10, rank, world, dist, gb),
                                          shape=f"global batch {gb} (one seeded batch, rows split over {world} GPU(s)), 2048->8192->2048, "
                                                "bf16 tcgen05 matmuls with fused epilogues, fp32 master weights, gradient all-reduce "
                                                "overlapped with backward",
                                          scaling="strong")
        if dist is not None:
            gc.collect()
            check(lib.ormi_b200_trim(dev.handle))
            err = mlp_sharded_vs_single(dev, W, rank, world, dist)
            extras["mlp_bf16_config4"]["sharded_vs_single_rel_err"] = err
            extras["mlp_bf16_config4"]["sharded_vs_single"] = (f"{world}-rank trainer against a single-rank trainer on the same {512 * world} rows, "
                                                                "3 SGD steps: largest relative error of loss and parameters")

    if rank == 0:
        ms_step = ms_total / args.steps
        value = world * BYTES_STEP / (ms_step * 1e-3) / 1e9
        ln_gbps = BYTES_LAYERNORM / (ms_ln / args.steps * 1e-3) / 1e9
        fused_gbps = BYTES_FUSED_KERNEL / (ms_fused / args.steps * 1e-3) / 1e9
        sm_gbps = BYTES_SOFTMAX / (ms_sm / args.steps * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": R, "cols": C,
                       "l2": "inputs larger than L2: x and gy are 268 MB each, the four results 268 MB each",
                       "step": "both graphs in one realize call: one fused kernel reads x and gy once (1.61 GB moved per step); "
                               "value counts the algorithmic bytes of the two graphs as separate fused passes (2.15 GB), as the reference arm does",
                       "exchange": "all-reduce of dg, db (2 x 4096 fp32) per step" if world > 1 else "none",
                       "cpu_sample": f"the reference arm and cpu_baseline step over workers x {CPU_ROWS_PER_WORKER} rows of the same workload"},
            "clocks": clocks,
            "e2e": {"value": world * BYTES_STEP / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "pipeline": f"{n_chunks} chunks of {E2E_CHUNK} rows: all uploads queued first | kernels k after upload k | download k behind kernels k",
                    "pinned_h2d_gbps": h2d_gbps, "pinned_d2h_gbps": d2h_gbps},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "kernel": STEP_KERNEL,
                         "achieved": fused_gbps, "peak": peak, "peak_source": peak_src, "unit": "GB/s", "frac": fused_gbps / peak,
                         "traffic": STEP_TRAFFIC_BYTES, "traffic_unit": "bytes per launch",
                         "traffic_source": STEP_TRAFFIC_SOURCE,
                         "algorithmic_bytes": BYTES_FUSED_KERNEL,
                         "burst": {"achieved": BYTES_FUSED_KERNEL / (ms_fused_burst / args.steps * 1e-3) / 1e9,
                                   "frac": BYTES_FUSED_KERNEL / (ms_fused_burst / args.steps * 1e-3) / 1e9 / peak,
                                   "note": "the same kernel timed right after the warm-up steps, before the sustained load"},
                         "graphs_in_calls_of_their_own": {
                             "softmax_kernel_gbps": sm_gbps, "layernorm_kernel_gbps": ln_gbps, "layernorm_frac": ln_gbps / peak,
                             "note": "each graph realized alone reads x and gy itself: 1 073.7 MB of algorithmic bytes per kernel"}},
        }
        if cpu_rec is not None:
            line["cpu_baseline"] = cpu_rec
        line["extra"] = extras
        emit(line)
    if dist is not None:
        dist.destroy_process_group()
    dev.close()


if __name__ == "__main__":
    main()
