"""Two processes on two GPUs: rows and gradients cross NVLink by direct stores into the peer's
memory.  Skipped unless at least two GPUs are visible."""

import socket
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("variant", ["l2", "distmult", "transh", "mlp"])
def test_two_processes_match_the_oracle(variant):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(ROOT / "tests" / "multi_gpu_worker.py"), variant]
    env = {**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"}
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert proc.stdout.count("MULTI_GPU_OK") == 2, proc.stdout[-3000:]
