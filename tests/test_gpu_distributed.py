"""Real multi-GPU run (one process per GPU, peer memory over NVLink) against the
unfused cuBLAS + NCCL path; needs at least two sm_100 GPUs."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _group_size() -> int:
    count = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return 8 if count >= 8 else 4 if count >= 4 else 2 if count >= 2 else 0


@pytest.mark.parametrize("handoff", ["lazy", "folded", "barriers"])
def test_fused_operators_match_cublas_plus_nccl(handoff: str) -> None:
    """Every slot hand-off protocol: one barrier kernel per operation with the second
    hand-off left to the next operation (the default), both hand-offs folded into the
    kernels, and two stand-alone barrier kernels per operation. The run
    covers every layout, the reference's multi-GPU shape matrix for this group size,
    the collective rejections, a hand-off that times out, and (--full) the
    Wan2.1-14B, Llama-3-8B, Llama-3-70B and edge-shape configurations on real peers."""

    import os

    up = _group_size()
    if up == 0:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, MEGA_UP_HANDOFF=handoff)
    command = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={up}",
        "--master-addr", "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "run_distributed.py"),
        "--full", "--stress", "20",
    ]
    result = subprocess.run(command, capture_output=True, text=True, timeout=1500, cwd=ROOT, env=env)
    lines = [line for line in result.stdout.splitlines() if line.startswith("[CORRECTNESS_RESULT]")]
    assert result.returncode == 0 and lines, result.stdout[-4000:] + result.stderr[-4000:]
    report = json.loads(lines[-1].split(" ", 1)[1])
    assert report["passed"], report["failures"]
