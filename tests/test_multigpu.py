"""Multi-rank GPU checks (expert transport over peer memory, fused sharded optimizer, peer-store broadcast, context
and tensor parallel kernels), launched as child processes with torchrun on 2 GPUs, or on HALO_TEST_RANKS of them when
that is set (2, 4 or 8). NVLS is switched off for the children."""

import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def test_multi_rank_checks():
    import torch

    n = int(os.environ.get("HALO_TEST_RANKS", "2"))
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} CUDA devices")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(root, "tests", "multigpu", "check_ranks.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert out.returncode == 0 and "CHECKS PASSED" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
