"""Row-sharded SpMM / SDDMM on 2+ GPUs (one process per GPU, NCCL) against the CPU oracle.
Skipped where fewer than two GPUs are visible; the CPU-rank (gloo) tests cover the host logic."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_sharded_ops_match_the_oracle_on_every_rank():
    import torch
    n_gpus = torch.cuda.device_count()
    if n_gpus < 2:
        pytest.skip("needs at least two GPUs")
    import oracle
    oracle.build()
    world = min(n_gpus, 4)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MULTI_GPU_SMALL_OK world=%d" % world in r.stdout
    assert "MULTI_GPU_FULL_SIZE_OK world=%d" % world in r.stdout
    assert "MULTI_GPU_OK world=%d" % world in r.stdout
    print(r.stdout[-600:])
