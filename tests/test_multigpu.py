"""Multi-GPU parity (needs >= 2 GPUs): ranks as child processes under torch.distributed.run, NCCL over NVLink."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_search_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(ROOT / "tests" / "mgpu_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("CASE_OK") == 10 and "SEARCH_OK" in out.stdout, out.stdout[-2000:]
    assert out.stdout.count("SCALE_OK") == 2 and "LATE_RANK_OK" in out.stdout, out.stdout[-2000:]
    assert "BALANCE_OK" in out.stdout, out.stdout[-2000:]
