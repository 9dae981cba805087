"""ZeRO-1 on two GPUs (skipped on a single-GPU box): one process per GPU over NCCL, run as child
processes; see tests/zero_multi_gpu_check.py for what is compared."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_fused_peer_store_gather_equals_nccl_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29541", os.path.join(HERE, "zero_multi_gpu_check.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-2000:]
    assert out.count(": OK") == 2 and "MISMATCH" not in out, out[-2000:]
