"""Worker of the multi-rank tests (launched with torch.distributed.run).

mode "gloo":  CPU ranks.  Each rank evaluates the gradients of ITS row shard of the MLP loss with the oracle, the
              shards' gradients are summed with a gloo all-reduce, and rank 0 compares with the full-batch oracle.
              This pins the sharding rule the GPU trainer uses (local loss scaled by 1 / global batch).
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
