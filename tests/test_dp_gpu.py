"""Data-parallel step on real GPUs (needs at least two): shard gradients all-reduced over NCCL
during the backward pass equal the full-batch gradients -- through torch.distributed from the
Python segment hook, through the exchange inside the library (mt_dp_*, libpk's collective
group), and for a QLoRA model whose only gradients are the LoRA matrices (one flat collective).
Host-side logic without GPUs is covered by tests/test_dp_cpu.py (gloo, world size 2) and
tests/test_comm_cpu.py (time limit, abort)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("variant,port", [("torch", 29533), ("pk", 29534), ("qlora", 29535)])
def test_two_rank_gradients_match_full_batch(variant, port):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    worker = Path(__file__).resolve().parent / "dp_worker.py"
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(worker), variant],
                         capture_output=True, text=True, timeout=600, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "OK" in res.stdout
    print(res.stdout[-400:])


def test_cpp_only_two_rank_training():
    """The example trainer of paperkiln_b200/host/examples/dp_two_rank.cpp: C++ over the C driver
    ABI, no Python and no torch.distributed anywhere; the ranks end with identical weights."""
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    exe = Path(__file__).resolve().parent.parent / "paperkiln_b200" / "dp_two_rank"
    assert exe.exists(), "build the package first (python -m paperkiln_b200.build)"
    res = subprocess.run([str(exe), "2", "3"], capture_output=True, text=True, timeout=600,
                         env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    assert res.returncode == 0 and "OK: 2 ranks" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]
