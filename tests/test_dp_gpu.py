"""Data-parallel step on real GPUs (needs at least two): shard gradients all-reduced over NCCL
from the segment hook equal the full-batch gradients. Host-side logic without GPUs is covered
by tests/test_dp_cpu.py (gloo, world size 2)."""
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_two_rank_gradients_match_full_batch():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    worker = Path(__file__).resolve().parent / "dp_worker.py"
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(worker)],
                         capture_output=True, text=True, timeout=600,
                         env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "OK" in res.stdout
