"""Multi-process, multi-GPU parity (one process per GPU, real peer-mapped symmetric memory).
Runs on as many GPUs as the box has (2, 4 or 8); skipped on a single-GPU box, where the same protocol
is covered by the single-process harness in test_allgather_gpu.py."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_multiprocess_parity(capi, cuda):
    n = cuda.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)
    port = 32000 + (os.getpid() % 1000)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
         "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multigpu_worker.py")],
        capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK") == world
