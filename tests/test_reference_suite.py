"""The reference's own CPU tests, run unmodified against this package through the
``mega_up`` import alias: its layout contract (tests/test_layout.py) and its shape
rule and tile-rotation tests (tests/test_shapes.py). Its PullConfigurationTest is
left out: it asserts the tuning tables of the reference's own pull kernel.

Needs a checkout of the reference; point ``MEGA_UP_REFERENCE_TREE`` at it. Nothing
is copied: the files are run where they lie, in a child process whose import
path starts with this repository.
"""

from __future__ import annotations

import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_reference_cpu_tests_pass_on_this_package() -> None:
    tree = os.environ.get("MEGA_UP_REFERENCE_TREE")
    if not tree:
        pytest.skip("MEGA_UP_REFERENCE_TREE is not set")
    files = [Path(tree) / "tests" / name for name in ("test_layout.py", "test_shapes.py")]
    missing = [str(f) for f in files if not f.exists()]
    if missing:
        pytest.skip(f"not found: {missing}")
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
