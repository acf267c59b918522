"""Host-side logic of the package on CPU: shape rule, layouts, slot arithmetic,
validation, and the multi-process (gloo, world_size 2) collective checks."""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import make_golden
import megaup_b200 as mega_up
from megaup_b200 import ops
from megaup_b200.kernels.peer_write_gemm import PEER_TILE_N, peer_n_rotation
from megaup_b200.runtime import MegaUPRuntime
from oracle import ulysses_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


# ----------------------------------------------------------------- shape rule


def test_shape_rule_matches_the_reference_strings() -> None:
    for width, up, reason in json.loads((GOLDEN / "shape_rule.json").read_text()):
        assert mega_up.unsupported_shape_reason(width, up) == reason
        assert mega_up.supports_shape(width, up) == (reason is None)


def test_head_dim_128_models_and_odd_tile_counts() -> None:
    for heads in (12, 16, 20, 24, 28, 32, 40, 48, 64):
        for up in (2, 4, 8):
            if heads % up == 0:
                assert mega_up.supports_shape(heads * 128, up)
    for hidden in (1280, 2304, 3328, 4864):
        assert mega_up.supports_shape(hidden, 2)


@pytest.mark.parametrize(
    "hidden,up,message",
    [
        (4096, 3, "UP must be one of"), (4096, 16, "UP must be one of"), (2049, 2, "divisible by UP"),
        (1920, 2, "multiple of 256"), (1536, 8, "head shard"), (1280, 8, "head shard"), (0, 2, "positive"),
    ],
)
def test_rejections_name_the_violated_constraint(hidden, up, message) -> None:
    assert message in mega_up.unsupported_shape_reason(hidden, up)
    assert not mega_up.supports_shape(hidden, up)


def test_rotation_matches_the_reference_tables() -> None:
    data = json.loads((GOLDEN / "rotation.json").read_text())
    assert data["tile_n"] == PEER_TILE_N
    for key, starts in data["starts"].items():
        hidden, up = map(int, key.split(","))
        assert [peer_n_rotation(r, up, hidden, PEER_TILE_N) for r in range(up)] == starts


# ----------------------------------------------------------------- THD layout


def test_thd_layouts_match_the_reference() -> None:
    with np.load(GOLDEN / "thd_layouts.npz") as data:
        for i in range(len(make_golden.THD_CASES)):
            cu = tuple(data[f"{i}/cu"].tolist())
            layout = ops._build_thd_layout(cu, up=int(data[f"{i}/up"]), device="cpu")
            assert np.array_equal(layout.to_thd_index.numpy(), data[f"{i}/to_thd"])
            assert np.array_equal(layout.to_source_major_index.numpy(), data[f"{i}/to_source_major"])
            assert layout.cu_seqlens_out == tuple(data[f"{i}/cu_out"].tolist())
            assert layout.fingerprint == bytes(data[f"{i}/fingerprint"]).decode()
            assert layout.num_samples == len(cu) - 1 and layout.tokens == cu[-1]


def test_thd_indices_are_mutually_inverse_permutations() -> None:
    layout = ops._build_thd_layout((0, 5, 5, 12, 13), up=3, device="cpu")
    assert (layout.tokens, layout.num_samples) == (13, 4)
    assert layout.cu_seqlens_out == (0, 15, 15, 36, 39)
    identity = torch.arange(39)
    assert torch.equal(layout.to_thd_index.sort().values, identity)
    assert torch.equal(layout.to_thd_index[layout.to_source_major_index], identity)
    assert torch.equal(layout.to_source_major_index[layout.to_thd_index], identity)


def test_thd_accepts_tensors_and_rejects_bad_boundaries() -> None:
    a = ops._build_thd_layout(torch.tensor([0, 4, 9], dtype=torch.int32), up=2, device="cpu")
    b = ops._build_thd_layout([0, 4, 9], up=2, device="cpu")
    assert torch.equal(a.to_thd_index, b.to_thd_index) and a.fingerprint == b.fingerprint
    for bad in ([0], [1, 5], [0, 5, 3], [0, 0], torch.zeros(2, 2, dtype=torch.int64), torch.tensor([0.0, 2.0])):
        with pytest.raises(ValueError):
            ops._build_thd_layout(bad, up=2, device="cpu")
    with pytest.raises(ValueError):
        ops._build_thd_layout([0, 4], up=0, device="cpu")


def test_equal_lengths_reduce_to_bshd() -> None:
    up, batch, seq, shard = 4, 3, 5, 16
    layout = ops._build_thd_layout([i * seq for i in range(batch + 1)], up=up, device="cpu")
    source_major = torch.arange(up * batch * seq * shard, dtype=torch.float32).view(up, batch * seq, shard)
    thd = ops._source_major_to_thd(source_major, layout, shard_heads=2, head_dim=8)
    bshd = ops._source_major_to_bshd(source_major, batch=batch, sequence=seq, shard_heads=2, head_dim=8)
    assert torch.equal(thd.view(batch, up * seq, 2, 8), bshd)


def test_layout_helpers_match_the_reference() -> None:
    with np.load(GOLDEN / "layout_helpers.npz") as data:
        up, batch, seq, sh, dim = data["meta"].tolist()
        sm = torch.arange(up * batch * seq * sh * dim, dtype=torch.float32).view(up, batch * seq, sh * dim)
        got = ops._source_major_to_bshd(sm, batch=batch, sequence=seq, shard_heads=sh, head_dim=dim)
        assert np.array_equal(got.numpy(), data["source_major_to_bshd"])
        hp = torch.arange(batch * up * seq * sh * dim, dtype=torch.float32).view(batch, up * seq, sh, dim)
        got = ops._bshd_to_destination_major(hp, up=up, sequence=seq)
        assert np.array_equal(got.numpy(), data["bshd_to_destination_major"])
        # round trip
        assert torch.equal(ops._source_major_to_bshd(got, batch=batch, sequence=seq, shard_heads=sh, head_dim=dim), hp)
        layout = ops._build_thd_layout(tuple(data["cu"].tolist()), up=up, device="cpu")
        smt = torch.arange(up * 16 * sh * dim, dtype=torch.float32).view(up, 16, sh * dim)
        got = ops._source_major_to_thd(smt, layout, shard_heads=sh, head_dim=dim)
        assert np.array_equal(got.numpy(), data["source_major_to_thd"])
        hpt = torch.arange(up * 16 * sh * dim, dtype=torch.float32).view(up * 16, sh, dim)
        got = ops._thd_to_destination_major(hpt, layout)
        assert np.array_equal(got.numpy(), data["thd_to_destination_major"])
    with pytest.raises(ValueError):
        ops._source_major_to_bshd(sm, batch=batch + 1, sequence=seq, shard_heads=sh, head_dim=dim)
    with pytest.raises(ValueError):
        ops._bshd_to_destination_major(hp, up=up, sequence=seq + 1)


# ----------------------------------------------------------------- runtime slot arithmetic


def cpu_runtime(up: int = 2, hidden: int = 512, max_rows: int = 64, rank: int = 0) -> MegaUPRuntime:
    arenas = tuple(
        torch.arange(up * max_rows * (hidden // up), dtype=torch.float32).view(up, max_rows, hidden // up) + 1e6 * r
        for r in range(up)
    )
    return MegaUPRuntime(
        group=None, arena=arenas[rank], handle=None, peer_buffers=arenas,
        peer_address_table=torch.zeros(up, dtype=torch.int64), max_rows=max_rows, hidden=hidden,
        local_rank=rank, up=up, emulated=True,
    )


def test_slots_are_densely_packed_from_offset_zero() -> None:
    runtime = cpu_runtime(up=2, hidden=512, max_rows=64, rank=1)
    assert runtime.shard_hidden == 256
    for rows, width in ((64, 512), (10, 512), (16, 1024), (7, 256)):
        shard = width // 2
        slots = runtime.slots(rows, width)
        assert tuple(slots.shape) == (2, rows, shard)
        flat = runtime.arena.view(-1)
        for p in range(2):
            assert torch.equal(slots[p].reshape(-1), flat[p * rows * shard : (p + 1) * rows * shard])
        views = runtime.remote_write_views(rows, width)
        for p, view in enumerate(views):
            start = runtime.local_rank * rows * shard
            assert torch.equal(view.reshape(-1), runtime.peer_buffers[p].view(-1)[start : start + rows * shard])
    assert tuple(runtime.slots(64).shape) == (2, 64, 256)


def test_capacity_rule() -> None:
    runtime = cpu_runtime(up=2, hidden=512, max_rows=64)
    runtime.check_capacity(64, 512)
    runtime.check_capacity(32, 1024)  # rows * width <= max_rows * hidden
    for rows, width in ((65, 512), (33, 1024), (0, 512), (4, 0), (4, 513)):
        with pytest.raises(ValueError):
            runtime.check_capacity(rows, width)


def test_validation_messages() -> None:
    runtime = cpu_runtime(up=2, hidden=512, max_rows=64)
    good = torch.zeros(512, 512, dtype=torch.bfloat16)
    assert ops._check_peer_weight(good, runtime, 64) == (512, 512)
    assert ops._check_pull_weight(good, runtime, 64) == (512, 512)
    with pytest.raises(ValueError, match="contiguous BF16"):
        ops._check_peer_weight(good.float(), runtime, 64)
    with pytest.raises(ValueError, match="contiguous BF16"):
        ops._check_peer_weight(torch.zeros(512, 1024, dtype=torch.bfloat16).t(), runtime, 64)  # transposed
    with pytest.raises(ValueError, match="peer-write out_features"):
        ops._check_peer_weight(torch.zeros(384, 512, dtype=torch.bfloat16), runtime, 64)
    with pytest.raises(ValueError, match="UP\\*head_dim"):
        ops._check_peer_weight(torch.zeros(512, 512, dtype=torch.bfloat16), runtime, 192)
    with pytest.raises(ValueError, match="multiple of 8"):
        ops._check_peer_weight(torch.zeros(512, 100, dtype=torch.bfloat16), runtime, 64)
    with pytest.raises(ValueError, match="pull in_features"):
        ops._check_pull_weight(torch.zeros(512, 384, dtype=torch.bfloat16), runtime, 64)
    with pytest.raises(ValueError, match="multiple of 256"):
        ops._check_pull_weight(torch.zeros(384, 512, dtype=torch.bfloat16), runtime, 64)
    with pytest.raises(ValueError, match="bias must have shape"):
        ops._check_bias(torch.zeros(5, dtype=torch.bfloat16), runtime, 512)
    with pytest.raises(ValueError, match="16-byte aligned"):
        ops._check_bias(torch.zeros(520, dtype=torch.bfloat16)[1:513], runtime, 512)
    with pytest.raises(TypeError):
        ops._check_layout(object(), runtime)
    layout = ops._build_thd_layout([0, 4], up=4, device="cpu")
    with pytest.raises(ValueError, match="UP=4"):
        ops._check_layout(layout, runtime)


def test_input_shape_checks() -> None:
    runtime = cpu_runtime(up=2, hidden=512, max_rows=64)
    x = torch.zeros(2, 8, 8, 64, dtype=torch.bfloat16)
    assert ops._peer_input_shape("bshd", x, runtime, None, n=512, k=512) == (2, 8, 8, 64)
    assert ops._peer_input_shape("sbhd", x, runtime, None, n=512, k=512) == (2, 8, 8, 64)
    assert ops._peer_input_shape("thd", x[0], runtime, None, n=512, k=512) == (8, 8, 64)
    with pytest.raises(ValueError, match=r"\[B,S,H,D\]"):
        ops._peer_input_shape("bshd", x[0], runtime, None, n=512, k=512)
    with pytest.raises(ValueError, match="heads\\*head_dim"):
        ops._peer_input_shape("bshd", x, runtime, None, n=512, k=256)
    with pytest.raises(ValueError, match="exceed the arena"):
        ops._peer_input_shape("bshd", torch.zeros(2, 64, 8, 64, dtype=torch.bfloat16), runtime, None, n=512, k=512)
    with pytest.raises(ValueError, match="contiguous BF16"):
        ops._peer_input_shape("bshd", x.float(), runtime, None, n=512, k=512)
    hx = torch.zeros(2, 16, 4, 64, dtype=torch.bfloat16)
    assert ops._pull_input_shape("bshd", hx, runtime, None, k=512) == (2, 8, 8, 64)
    assert ops._pull_input_shape("sbhd", hx, runtime, None, k=512) == (1, 16, 8, 64)
    assert ops._pull_input_shape("thd", hx[0], runtime, None, k=512) == (8, 8, 64)
    with pytest.raises(ValueError, match="divisible by UP"):
        ops._pull_input_shape("bshd", torch.zeros(2, 15, 4, 64, dtype=torch.bfloat16), runtime, None, k=512)
    layout = ops._build_thd_layout([0, 3, 7], up=2, device="cpu")
    with pytest.raises(ValueError, match="UP\\*T=14"):
        ops._pull_input_shape("thd", hx[0], runtime, layout, k=512)
    assert ops._exchanged_shape("bshd", (2, 8, 8, 64), 2, 4) == (2, 16, 4, 64)
    assert ops._exchanged_shape("sbhd", (8, 2, 8, 64), 2, 4) == (16, 2, 4, 64)
    assert ops._exchanged_shape("thd", (8, 8, 64), 2, 4) == (16, 4, 64)


def test_thd_token_resolution() -> None:
    runtime = cpu_runtime(up=2)
    layout = ops._build_thd_layout([0, 3, 7], up=2, device="cpu")
    assert ops._resolve_thd_tokens(None, layout, runtime) == 7
    assert ops._resolve_thd_tokens(7, layout, runtime) == 7
    with pytest.raises(ValueError, match="disagrees"):
        ops._resolve_thd_tokens(8, layout, runtime)
    with pytest.raises(ValueError, match="tokens is required"):
        ops._resolve_thd_tokens(None, None, runtime)


# ----------------------------------------------------------------- multi-process (gloo) checks


def _spawn(body: str, world: int = 2) -> None:
    import torch.multiprocessing as mp

    import _dist_workers

    port = 29600 + abs(hash(body)) % 300
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_dist_workers.run, args=(world, port, body, tmp), nprocs=world, join=True)
        for rank in range(world):
            verdict = Path(tmp, f"rank{rank}.txt").read_text()
            assert verdict == "ok", f"rank {rank}:\n{verdict}"


def test_collective_validation_world_size_2() -> None:
    _spawn("collective_validation")


def test_fd_exchange_world_size_2() -> None:
    _spawn("fd_exchange")


def test_exchange_semantics_over_gloo_world_size_2() -> None:
    _spawn("sharded_oracle_exchange")


def test_mega_up_alias_package_resolves_to_this_implementation() -> None:
    import mega_up as alias
    from mega_up.kernels.peer_write_gemm import PEER_TILE_N as tile
    from mega_up.ops import _build_thd_layout as build
    from mega_up.runtime import MegaUPRuntime as runtime_class

    assert alias.initialize_runtime is mega_up.initialize_runtime
    assert build is ops._build_thd_layout and runtime_class is MegaUPRuntime and tile == 256
    for name in (
        "initialize_runtime", "supports_shape", "unsupported_shape_reason", "prepare_thd_layout", "THDLayout",
        "prepare_peer_write_gemm_bshd", "prepare_peer_write_gemm_sbhd", "prepare_peer_write_gemm_thd",
        "prepare_headshard_pull_gemm_bshd", "prepare_headshard_pull_gemm_sbhd", "prepare_headshard_pull_gemm_thd",
        "peer_write_gemm_bshd", "peer_write_gemm_sbhd", "peer_write_gemm_thd",
        "headshard_pull_gemm_bshd", "headshard_pull_gemm_sbhd", "headshard_pull_gemm_thd",
        "MegaUPRuntime", "DEFAULT_MAX_ROWS", "SUPPORTED_UP_DEGREES",
    ):
        assert hasattr(alias, name), name


def test_secondary_surface_of_the_kernel_modules() -> None:
    """Names the reference's own tests and benchmarks import from its kernel modules
    (tests/test_shapes.py:50, benchmarks/bench_bshd.py:873, tests/run_pull_gemm_contention.py:225-254),
    describing this kernel: 16-byte lanes, tickets of at most 512 vectors."""

    import importlib

    pw = importlib.import_module("mega_up.kernels.peer_write_gemm")
    pull = importlib.import_module("mega_up.kernels.headshard_pull_gemm")
    assert pw.PEER_TILE_N == 256 and isinstance(pw.IMPLEMENTATION_REVISION, str)
    assert isinstance(pull.IMPLEMENTATION_REVISION, str)
    with pytest.raises(TypeError, match="BF16 A tensor"):
        pw.prepare_peer_write(None, None, None, ())
    assert pull.PULL_MAX_ELEMENTS_IN_FLIGHT == 4096
    # (shard width, rows per ticket, column segments of one row)
    for shard, rows, segments in ((128, 16, 1), (640, 4, 1), (1024, 4, 1), (1280, 2, 1), (2560, 1, 1), (4096, 1, 1), (6144, 1, 2), (8192, 1, 2)):
        assert pull._select_pull_elements_per_lane(shard) == 8
        assert pull._vector_pull_rows_per_ticket(16, shard) == rows
        assert pull._vector_pull_rows_per_ticket(2, shard) == min(rows, 2)
        assert pull._pull_column_chunks(shard, 1) == segments
        assert rows * shard // segments <= pull.PULL_MAX_ELEMENTS_IN_FLIGHT
    assert pull._pull_column_chunks(640, 8) == 2  # eight rows of 640 need two segments of 320
    with pytest.raises(ValueError):
        pull._select_pull_elements_per_lane(100)


def test_sync_points_skip_zero_when_the_32_bit_count_wraps() -> None:
    # 0 means "no wait / no signal" in a kernel's hand-off description, so the
    # wire value of a sync point is never 0 and stays strictly ordered by
    # signed distance across the wrap
    from megaup_b200.runtime import _wire_epoch

    assert _wire_epoch(0) == 0
    assert [_wire_epoch(c) for c in (1, 2, 3)] == [1, 2, 3]
    top = 0xFFFFFFFF
    around = [_wire_epoch(c) for c in range(top - 2, top + 4)]
    assert 0 not in around
    assert around == [top - 2, top - 1, top, 1, 2, 3]
    for earlier, later in zip(around, around[1:]):
        distance = (later - earlier) & 0xFFFFFFFF
        assert 0 < distance < 0x80000000  # "later" is ahead of "earlier" as the kernels compare them


def test_the_hand_off_protocol_is_validated_on_import() -> None:
    import subprocess
    import sys

    code = "import os; os.environ['MEGA_UP_HANDOFF']='sometimes'; import megaup_b200.runtime"
    repo = Path(__file__).resolve().parent.parent
    result = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(repo))
    assert result.returncode != 0 and "MEGA_UP_HANDOFF must be lazy, folded or barriers" in result.stderr
