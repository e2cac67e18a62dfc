"""The list launch over the row slices of two GPUs (bonsai_b200_chain_create_tp): needs two devices, skipped
otherwise.  The ranks run as child processes; nothing here waits on a GPU that cannot answer (every wait in the
kernel is bounded, and the workers run under a time limit)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_ranks_store_into_each_other(gpu):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "tp_worker.py")],
                         capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert "rank 0: ok=True status=0" in out.stdout and "rank 1: ok=True status=0" in out.stdout
