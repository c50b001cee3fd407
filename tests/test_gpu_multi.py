"""Column-parallel and token-parallel linears on two GPUs (skipped on a single-GPU box): the NCCL all-gather
form and the fused epilogue-scatter form both reproduce the unsharded result bit for bit."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_linears_equal_unsharded_on_two_gpus():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(ROOT / "tests" / "multi_gpu_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
