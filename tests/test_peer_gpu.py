"""N-sharded linear with the all_gather fused into the matmul epilogue (peer stores), 2 GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs on one machine")
def test_sharded_matmul_allgather_two_ranks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541",
                          os.path.join(root, "tests", "peer_worker.py")], cwd=root, env=env, capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0 and res.stdout.count("PEER-OK") == 2, res.stdout[-3000:] + res.stderr[-3000:]
