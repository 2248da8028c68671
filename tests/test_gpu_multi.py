"""Fused synchronisation across real GPUs (one process each, peer memory over NVLink) against the reference-style
NCCL path, and a two-rank SMA training run.  Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_sync_and_training_across_gpus():
    n = min(4, torch.cuda.device_count())
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(29700 + os.getpid() % 200), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if r.returncode != 0:                      # (shown by pytest with the failure; the assertion message itself is truncated)
        print(r.stdout[-3000:])
        print(r.stderr[-12000:])
    assert r.returncode == 0 and "MULTI_GPU_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])
