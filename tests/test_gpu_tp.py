"""The list launch over the row slices of several GPUs (bonsai_b200_chain_create_tp): needs two devices, skipped
otherwise.  The ranks run as child processes; nothing here waits on a GPU that cannot answer (every wait in the
kernel is bounded, and the workers run under a time limit)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ranks_store_into_each_other(gpu):
    """As many ranks as there are devices, 2, 4 or 8 (at rows / 8 an op leaves 1 - 4 tasks per CTA and many CTAs without
    rows: another geometry than at 2)."""
    import torch
    ndev = torch.cuda.device_count()
    if ndev < 2:
        pytest.skip("needs two GPUs")
    world = 8 if ndev >= 8 else 4 if ndev >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                          "--master-addr", "127.0.0.1", "--master-port", "29611", os.path.join(ROOT, "tests", "tp_worker.py")],
                         capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    for r in range(world):
        assert f"rank {r}: ok=True status=0" in out.stdout, (out.stdout + out.stderr)[-3000:]
