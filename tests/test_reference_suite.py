"""The reference's own CPU tests, run unmodified against this package through the
``mega_up`` import alias: its layout contract (tests/test_layout.py) and its shape
rule and tile-rotation tests (tests/test_shapes.py). Its PullConfigurationTest is
left out: it asserts the tuning tables of the reference's own pull kernel.

Needs a checkout of the reference; point ``MEGA_UP_REFERENCE_TREE`` at it. Nothing
is copied: the files are run where they lie, in a child process whose import
path starts with this repository. The reference's single-GPU pull-GEMM race
runner (tests/run_pull_gemm_contention.py) is driven the same way on a GPU; it
is also looked for in the reference install under ``baseline/_ref``.
"""

from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _reference_file(name: str) -> Path | None:
    candidates = []
    tree = os.environ.get("MEGA_UP_REFERENCE_TREE")
    if tree:
        candidates.append(Path(tree) / "tests" / name)
    candidates.append(ROOT / "baseline" / "_ref" / "reference_runners" / name)
    for candidate in candidates:
        if candidate.exists():
            return candidate
    return None


def test_reference_cpu_tests_pass_on_this_package() -> None:
    files = [_reference_file(name) for name in ("test_layout.py", "test_shapes.py")]
    if any(f is None for f in files):
        pytest.skip("the reference's tests are not available (set MEGA_UP_REFERENCE_TREE or run baseline/install_reference.sh)")
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    with tempfile.TemporaryDirectory() as scratch:
        where = subprocess.run(
            [sys.executable, "-c", "import mega_up; print(mega_up.__file__)"],
            capture_output=True, text=True, cwd=scratch, env=env, timeout=300,
        )
        assert where.returncode == 0, where.stderr
        assert Path(where.stdout.strip()).resolve().is_relative_to(ROOT), where.stdout
        result = subprocess.run(
            [sys.executable, "-m", "pytest", *map(str, files), "-q", "-p", "no:cacheprovider",
             "-k", "not PullConfiguration"],
            capture_output=True, text=True, cwd=scratch, env=env, timeout=900,
        )
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-2000:]
    assert " passed" in result.stdout


@pytest.mark.gpu
@pytest.mark.parametrize(
    "arguments",
    [
        ("--hidden", "2048", "--rows", "4096", "--iters", "20", "--contention", "--bias"),
        ("--hidden", "5120", "--rows", "4096", "--iters", "5", "--perf", "--perf-iters", "20"),
    ],
    ids=["contention_2048", "wan_5120_perf"],
)
def test_reference_pull_race_runner_passes_on_this_kernel(arguments: tuple[str, ...]) -> None:
    """The reference's single-GPU regression runner for its pull GEMM, unmodified,
    with ``mega_up.kernels.headshard_pull_gemm`` resolving to this package: eight
    emulated peers on one GPU, every call checked against a gather reference, a
    bitwise repeat check, and (first case) elementwise kernels on a side stream
    that share the SMs with the pull GEMM."""

    import json

    runner = _reference_file("run_pull_gemm_contention.py")
    if runner is None:
        pytest.skip("the reference's run_pull_gemm_contention.py is not available")
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    with tempfile.TemporaryDirectory() as scratch:
        result = subprocess.run(
            [sys.executable, str(runner), *arguments],
            capture_output=True, text=True, cwd=scratch, env=env, timeout=900,
        )
    tail = result.stdout[-3000:] + result.stderr[-2000:]
    assert result.returncode == 0, tail
    kernel_line = next(line for line in result.stdout.splitlines() if line.startswith("kernel="))
    assert Path(kernel_line.split("=", 1)[1]).resolve().is_relative_to(ROOT), kernel_line
    report = json.loads(
        next(line for line in result.stdout.splitlines() if line.startswith("[CONTENTION_RESULT]")).split(" ", 1)[1]
    )
    assert report["status"] == "passed" and report["race_events"] == 0 and report["dy_mismatches"] == 0, report
