"""Multi-GPU test of the data-parallel gradient exchanges (needs at least two GPUs in the box; skipped otherwise)."""
import os
import signal
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sharded_and_sparse_exchange_match_allreduce_exchange():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "mgpu_worker.py")]
    # the launcher and its workers form a process group of their own, so that a timeout ends all of them
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env, start_new_session=True)
    try:
        out, err = proc.communicate(timeout=600)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        out, err = proc.communicate()
        pytest.fail("multi-GPU worker timed out\n" + out[-2000:] + err[-4000:])
    assert proc.returncode == 0 and "MGPU_OK" in out, out[-2000:] + err[-4000:]
