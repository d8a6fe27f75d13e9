"""Multi-GPU parity of the library's own all-gather (peer stores + flag barrier); needs two GPUs on the node."""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_shard_gather_over_peer_memory():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    gpus = min(torch.cuda.device_count(), 4)
    if gpus < 2:
        pytest.skip("one GPU on this node: the peer all-gather needs two")
    script = Path(__file__).with_name("multi_gpu_gather.py")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
                          "--master-port", "29641", str(script)], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert "multi_gpu_gather ok" in run.stdout
