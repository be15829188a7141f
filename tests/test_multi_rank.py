"""Multi-rank paths: gloo ranks on the CPU (always), NCCL ranks on GPUs (when the machine has at least two)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(mode, world, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_rank_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)


def test_sharded_gradients_sum_to_full_batch_gradients_gloo():
    out = launch("gloo", 2, 29533)
    assert out.returncode == 0 and "MULTI_RANK_OK gloo 2" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]


@pytest.mark.gpu
def test_sharded_training_step_nccl():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 4 if n >= 4 else 2
    out = launch("nccl", world, 29534)
    assert out.returncode == 0 and f"MULTI_RANK_OK nccl {world}" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]
