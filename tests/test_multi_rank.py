"""Multi-rank paths: gloo ranks on the CPU (always), NCCL ranks on GPUs (when the machine has at least two)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(mode, world, port, **extra_env):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "multi_rank_worker.py"), mode]
    env = dict(os.environ, OMP_NUM_THREADS="1", **extra_env)
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


def test_a_rank_that_leaves_is_noticed_on_the_host_before_the_next_collective_gloo():
    """Failure detection without any GPU: the last of three CPU ranks stops after two steps, once announcing it, once
    silently; the others' step guard raises within its deadline and they never enter the third collective."""
    out = launch("guard", 3, 29541)
    assert out.returncode == 0 and "MULTI_RANK_OK guard 3" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]


@pytest.mark.gpu
def test_a_rank_that_leaves_between_steps_nccl():
    """The same on GPUs: the rank leaves between steps with nothing in flight, the survivors learn of it on the host and
    launch nothing more.  NVLS is off (a rank whose memory is bound to a multicast object must not go away)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    out = launch("nccl_leave", 2, 29545, NCCL_NVLS_ENABLE="0")
    assert out.returncode == 0 and "MULTI_RANK_OK nccl_leave 2" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]
