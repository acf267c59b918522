"""Shared test configuration: the ``gpu`` marker, import paths, oracle build."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"
if str(GOLDEN) not in sys.path:
    sys.path.insert(0, str(GOLDEN))


def pytest_configure(config: pytest.Config) -> None:
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x")


@pytest.fixture(scope="session", autouse=True)
def _oracle_c_kernel() -> None:
    """Build the oracle's C kernel once (gcc); the oracle falls back to float32
    BLAS when it cannot be built, which is identical on integer-valued cases."""

    try:
        from oracle import build as oracle_build

        oracle_build.ensure_built()
    except Exception:  # noqa: BLE001 - the numpy path of the oracle still works
        pass


def pytest_collection_modifyitems(config: pytest.Config, items: list[pytest.Item]) -> None:
    try:
        import torch

        has_gpu = torch.cuda.is_available() and torch.cuda.get_device_capability(0)[0] == 10
    except Exception:  # noqa: BLE001
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="needs an sm_100 GPU")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
