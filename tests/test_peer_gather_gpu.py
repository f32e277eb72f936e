"""The copy-engine gather (parallel.PeerGatherer) against the NCCL send/recv gather, on 2 GPUs of one box.
Skipped on a box with one GPU."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_peer_gather_equals_nccl_gather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from raptor_t_b200 import parallel
    if not parallel.PeerGatherer.available():
        pytest.skip("torch symmetric memory or the cuda-python driver bindings are missing")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", os.path.join(ROOT, "tests", "peer_gather_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "PEER GATHER OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
