"""Multi-GPU column-parallel parity (needs at least two GPUs; skipped otherwise): one process per
GPU under torchrun, fused in-kernel exchange and kernel + NCCL all-gather both checked against the
CPU oracle by tests/tp_worker.py."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_parallel_fused_and_nccl(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world), str(HERE / "tp_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert proc.returncode == 0 and "TP_WORKER_OK" in proc.stdout, (proc.stdout[-3000:], proc.stderr[-3000:])
