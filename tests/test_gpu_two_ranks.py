"""Both multi-GPU partitionings on two real GPUs, one process per GPU (skipped on a one-GPU box)."""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_row_shards_and_key_range_shards_on_two_gpus():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    script = Path(__file__).with_name("two_rank_check.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
         "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
        capture_output=True, text=True, timeout=600, env=env,
    )
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert result.stdout.count("exact on own scores True") == 6
    assert result.stdout.count("64/64 rows equal") == 2
