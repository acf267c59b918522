"""The C-ABI library loads without a GPU and exports exactly what include/megaup.h declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from megaup_b200 import _native, build

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "megaup.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mup_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def library() -> ctypes.CDLL:
    build.ensure_built()
    return _native.lib()


def test_header_and_binding_list_the_same_symbols() -> None:
    assert declared_symbols() == sorted(_native.SIGNATURES)


def test_every_declared_symbol_is_exported(library: ctypes.CDLL) -> None:
    for name in declared_symbols():
        assert hasattr(library, name), name


def test_host_only_entry_points(library: ctypes.CDLL) -> None:
    assert library.mup_abi_version() == 1
    # shape rule: 0 = supported, else the first violated clause
    assert library.mup_shape_rule(5120, 8) == 0
    assert library.mup_shape_rule(2304, 2) == 0
    assert library.mup_shape_rule(4096, 3) == 1
    assert library.mup_shape_rule(2049, 2) == 2
    assert library.mup_shape_rule(1920, 2) == 3
    assert library.mup_shape_rule(1536, 8) == 4
    assert [library.mup_peer_n_rotation(r, 8, 5120, 256) for r in range(8)] == [0, 3, 5, 8, 10, 13, 15, 18]
    assert library.mup_pull_workspace_bytes(4096) == (16 + 1024 + 32) * 8
    assert library.mup_pull_workspace_bytes(0) == 0


def test_bad_arguments_are_rejected_without_a_gpu(library: ctypes.CDLL) -> None:
    plan = ctypes.c_void_p()
    code = library.mup_gather_rows(None, None, None, 4, 8, None)
    assert code == -1 and b"gather" in library.mup_last_error()
    code = library.mup_flag_barrier(None, 2, 0, 1, None, 1000, None)
    assert code == -1
    code = library.mup_peer_write_plan_create(
        ctypes.byref(plan), 0, 0, 256, 64, 2, 0, None, None, None, 0, None, 1000
    )
    assert code == -1 and not plan.value
