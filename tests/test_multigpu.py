"""Two-rank GPU checks (expert transport over peer memory, fused sharded optimizer, peer-store
broadcast), launched as child processes with torchrun. NVLS is switched off for the children."""

import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_two_rank_checks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(root, "tests", "multigpu", "check_two_ranks.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert out.returncode == 0 and "CHECKS PASSED" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
