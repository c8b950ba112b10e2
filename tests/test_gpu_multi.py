"""Multi-GPU checks: one process per GPU through torch.distributed.run.  Skipped on a machine with fewer
than two GPUs (the single-GPU run of the suite); the host-side sharding logic is covered on CPU by
tests/test_sharding_gloo.py."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("peer", [True, False])
def test_all_reduce_inside_the_row_kernel(peer):
    """An all-reduce requested on top of a reduction that rides along in a row kernel is done by that
    kernel over peer memory (peer=True) or, with WGF_NO_PEER_ALLREDUCE=1, by NCCL after it."""
    n = min(gpu_count(), 4)
    if n < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"      # plain peer memory only: no multicast objects in a test
    env.pop("WGF_NO_PEER_ALLREDUCE", None)
    if not peer:
        env["WGF_NO_PEER_ALLREDUCE"] = "1"
    port = 29540 + (0 if peer else 1)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "multi", "all_reduce_in_kernel_check.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=150)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("PASS") == n


def test_a_peer_that_sits_an_exchange_out_gives_a_timeout_status():
    """The wait for the peers' values has a limit (WGF_PEER_WAIT_MS): when a peer never posts, the settling
    kernel returns, the next synchronisation reports WGF_ERR_TIMEOUT and the communicator can be released."""
    if gpu_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    env["WGF_PEER_WAIT_MS"] = "50"
    env.pop("WGF_NO_PEER_ALLREDUCE", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29543", os.path.join(HERE, "multi", "peer_wait_runs_out.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=150)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("PASS") == 2
