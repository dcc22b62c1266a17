"""Row sharding over NCCL on two GPUs against the unsharded operators (skipped with fewer than two GPUs;
bench.py --gpus N carries the same comparison in its `shard_check` field for every N)."""
import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.timeout(600)
def test_two_gpu_sharding_matches_the_unsharded_operators():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "shard_nccl_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=540, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "rank 0: shard check ok" in proc.stdout and "rank 1: shard check ok" in proc.stdout
