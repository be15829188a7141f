"""Worker of the multi-rank tests (launched with torch.distributed.run).

mode "gloo":  CPU ranks.  Each rank evaluates the gradients of ITS row shard of the MLP loss with the oracle, the
              shards' gradients are summed with a gloo all-reduce, and rank 0 compares with the full-batch oracle.
              This pins the sharding rule the GPU trainer uses (local loss scaled by 1 / global batch).
mode "guard": CPU ranks and a TCP store.  Every rank announces each step (ormi_b200.guard.StepGuard) and then joins a gloo
              all-reduce; the last rank stops after two steps — once saying so (leave), once silently.  The others must
              get RankLost from the check of the third step, within the deadline, WITHOUT entering that step's collective.
mode "nccl_leave": one GPU per rank, NVLS off.  Two sharded trainer steps, then the last rank leaves between steps
              (nothing of its own in flight) and the others learn of it on the host before their next launch.
mode "nccl":  one GPU per rank.  MLPTrainer with world > 1 (NCCL all-reduce through the C ABI, overlapped with the
              backward phases) against a single-rank trainer fed the full batch, after three SGD steps.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ormi_b200 import graph as G            # noqa: E402
from ormi_b200 import workloads as W        # noqa: E402


def problem(B, D, H):
    x, t = W.normal(0, (B, D)), W.normal(1, (B, D))
    w1, b1 = W.kaiming_uniform(2, D, (D, H)), W.normal(4, (H,), 0.1)
    w2, b2 = W.kaiming_uniform(3, H, (H, D)), W.normal(5, (D,), 0.1)
    return x, t, w1, b1, w2, b2


def oracle_grads(x, t, params, scale):
    from oracle import oracle as O
    leaves = [G.leaf(p, True) for p in params]
    loss = W.mlp_loss(G.leaf(x), leaves[0], leaves[1], leaves[2], leaves[3], G.leaf(t), scale=scale)
    G.compute_gradients(loss)
    outs, _ = O.port_run([loss] + [l.grad for l in leaves])
    return outs


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    B, D, H = 64 * world, 32, 96
    x, t, *params = problem(B, D, H)
    rows = slice(rank * B // world, (rank + 1) * B // world)
    if mode == "guard":
        import datetime
        import time
        from ormi_b200.guard import StepGuard, RankLost
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
        store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=30))
        for variant, announce in (("says so", True), ("silent", False)):
            guard = StepGuard(store, rank, world, timeout_s=1.5, prefix=f"t/{variant}")
            entered = 0
            dist.barrier()                          # the ranks start the loop together (process start-up skews by seconds)
            try:
                for step in range(4):
                    if rank == world - 1 and step == 2:
                        if announce:
                            guard.leave()
                        break                       # this rank is gone: it joins no further collective
                    t0 = time.monotonic()
                    guard.check(step)
                    tt = torch.ones(4)
                    dist.all_reduce(tt)             # stands for the step's gradient all-reduce
                    entered += 1
                    assert float(tt[0]) == world
                assert rank == world - 1, "the survivors must not get through step 2"
            except RankLost as e:
                waited = time.monotonic() - t0
                assert rank != world - 1 and entered == 2 and waited < (0.5 if announce else 3.0), (entered, waited, str(e))
            time.sleep(2.0 if rank == world - 1 else 0.2)      # keep the store's master-side connections orderly
        if rank == 0:
            print("MULTI_RANK_OK guard", world)
        dist.destroy_process_group()
        return
    if mode == "nccl_leave":
        import datetime
        from ormi_b200.guard import StepGuard, RankLost
        from ormi_b200.runtime import Device
        from ormi_b200.train_step import MLPTrainer, init_comm
        local_rank = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local_rank)
        dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))     # host channel only: NCCL is driven by the library
        store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                              timeout=datetime.timedelta(seconds=30))
        dev = Device(local_rank)
        dev.set_option("comm_timeout_ms", "20000")

        def bcast(payload):
            obj = [payload]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        init_comm(dev, rank, world, bcast)
        tr = MLPTrainer(dev, x[rows], t[rows], *params, lr=0.1, global_batch=B, world=world)
        guard = StepGuard(store, rank, world, timeout_s=5.0)
        done, lost = 0, False
        dist.barrier()
        try:
            for step in range(4):
                if rank == world - 1 and step == 2:
                    tr.flush()
                    dev.sync()                      # nothing of this rank is in flight any more
                    guard.leave()
                    break
                guard.check(step)
                tr.step()
                done += 1
        except RankLost:
            lost = True
        dev.sync()                                  # the survivors' streams are clean: no collective was launched into the void
        assert done == 2 and (lost or rank == world - 1)
        assert np.isfinite(tr.loss())
        dev.close()
        import time
        time.sleep(1.0 if rank == world - 1 else 0.1)
        if rank == 0:
            print("MULTI_RANK_OK nccl_leave", world)
        dist.destroy_process_group()
        return
    if mode == "gloo":
        dist.init_process_group("gloo")
        local = oracle_grads(x[rows], t[rows], params, scale=1.0 / (B * D))
        summed = []
        for g in local:
            tt = torch.from_numpy(np.ascontiguousarray(g).reshape(-1).copy())
            dist.all_reduce(tt)
            summed.append(tt.numpy().reshape(g.shape))
        if rank == 0:
            full = oracle_grads(x, t, params, scale=1.0 / (B * D))
            for s, f in zip(summed, full):
                assert np.abs(s - f).max() <= 1e-5 * max(1e-30, np.abs(f).max()), np.abs(s - f).max()
            print("MULTI_RANK_OK gloo", world)
    else:
        from ormi_b200.runtime import Device
        from ormi_b200.train_step import MLPTrainer, init_comm
        local_rank = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dev = Device(local_rank)

        def bcast(payload):
            obj = [payload]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        init_comm(dev, rank, world, bcast)
        for overlap in (True, False):
            tr = MLPTrainer(dev, x[rows], t[rows], *params, lr=0.1, global_batch=B, world=world, overlap=overlap)
            for _ in range(3):
                tr.step()
            got_loss = tr.loss()
            got = [tr.parameter(n) for n in tr.names]
            if rank == 0:
                solo = MLPTrainer(dev, x, t, *params, lr=0.1)
                for _ in range(3):
                    solo.step()
                assert abs(got_loss - solo.loss()) <= 3e-5 * abs(solo.loss()), (got_loss, solo.loss())
                for n, g in zip(solo.names, got):
                    w = solo.parameter(n)
                    assert np.abs(g - w).max() <= 3e-5 * np.abs(w).max(), n
        dist.barrier()
        if rank == 0:
            print("MULTI_RANK_OK nccl", world)
        dev.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
