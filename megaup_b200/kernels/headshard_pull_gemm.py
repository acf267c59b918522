"""Head-shard pull GEMM: pull warps gather every peer's head shard of each row
into the dense local input while the MMA warps already consume finished
128-row panels; ``out = bf16(dy @ W.T + bias)``.

Host handle of ``mup_pull_*`` in libmegaup.so; mirrors the seam of the
reference's ``mega_up/kernels/headshard_pull_gemm.py``
(``compile_headshard_pull_gemm`` at :2440-2777, ``CompiledHeadShardPullGemm``
at :2353-2438). The ticket cursor and the per-panel ready counts only ever
grow, so launches need no workspace reset in between; ``epoch`` and
``workspace_epochs`` keep the reference's meaning for callers that recycle.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch
from torch import Tensor

from .. import _native

IMPLEMENTATION_REVISION = "megaup-b200-cuda-r1"
TILE_N = 256
# BF16 elements one pull warp keeps in flight: a ticket is at most 512 16-byte vectors.
PULL_MAX_ELEMENTS_IN_FLIGHT = 512 * 8
WARP_SIZE = 32


def _ticket_shape(shard_k: int) -> tuple[int, int]:
    rows, segments = ctypes.c_int(), ctypes.c_int()
    try:
        _native.call("mup_pull_ticket_shape", int(shard_k), ctypes.byref(rows), ctypes.byref(segments))
    except _native.NativeError as error:
        raise ValueError(str(error)) from None
    return rows.value, segments.value


def _select_pull_elements_per_lane(shard_k: int) -> int:
    """BF16 elements per lane and load: this kernel always pulls with 16-byte
    vectors (the reference chooses 4, 8 or 16 elements by shard width,
    headshard_pull_gemm.py:137-142)."""

    _ticket_shape(shard_k)  # validates the shard width
    return 8


def _vector_pull_rows_per_ticket(pull_rows_per_ticket: int, shard_k: int) -> int:
    """Rows of one peer shard per ticket: the largest power of two, at most 16
    and at most ``pull_rows_per_ticket``, whose rows fit
    ``PULL_MAX_ELEMENTS_IN_FLIGHT`` (reference table: headshard_pull_gemm.py:166-182)."""

    rows, _ = _ticket_shape(shard_k)
    limit = max(1, int(pull_rows_per_ticket))
    while rows > limit:
        rows //= 2
    return rows


def _pull_column_chunks(shard_k: int, rows_in_flight: int) -> int:
    """Equal column segments a shard row is cut into so that ``rows_in_flight``
    rows of one segment fit a ticket (reference: headshard_pull_gemm.py:185-198).
    The kernel itself only cuts rows that exceed a ticket on their own."""

    _, segments = _ticket_shape(shard_k)
    rows = max(1, int(rows_in_flight))
    chunks = max(segments, -(-rows * shard_k // PULL_MAX_ELEMENTS_IN_FLIGHT))
    while shard_k % chunks or (shard_k // chunks) % 8:
        chunks += 1
    return chunks


class CompiledHeadShardPullGemm:
    """Bound pull kernel; call it with the stream to launch on."""

    def __init__(
        self,
        plan: ctypes.c_void_p,
        workspace: Tensor,
        keep_alive: tuple[object, ...],
        workspace_epochs: int,
        rows: int,
        rank: int,
        up: int,
    ) -> None:
        self._plan = plan
        self._workspace = workspace
        self._keep_alive = keep_alive
        self.workspace_epochs = int(workspace_epochs)
        self.epoch = 0
        self.logical_m = rows
        self.rank = rank
        self.up = up
        grid, group, smem, tile = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        launches = ctypes.c_uint64()
        _native.call(
            "mup_pull_plan_info", plan, ctypes.byref(grid), ctypes.byref(group),
            ctypes.byref(launches), ctypes.byref(smem), ctypes.byref(tile),
        )
        self.tile_n = tile.value
        self.grid_ctas = grid.value
        self.cta_group = group.value
        self.smem_bytes = smem.value
        # descriptors the reference's compiled object carries (run_pull_gemm_contention.py:225-254)
        # stage geometry of the widest work item (classes of 128, 256 and 512 columns)
        class_cols = 128 if self.tile_n <= 128 else 256 if self.tile_n <= 256 else 512
        stage_bytes = 128 * 64 * 2 + (class_cols // self.cta_group) * 64 * 2
        self.num_ab_stages = min(8, 196608 // stage_bytes)
        self.num_c_stages = 2
        self.enable_bulk_pull = False

    def describe_pull(self, shard_k: int) -> None:
        self.pull_rows_per_ticket, self.pull_col_chunks = _ticket_shape(shard_k)

    def reset_workspace(self, stream: torch.cuda.Stream | None = None) -> None:
        """Zero the counters on ``stream`` and restart the launch ordinal."""

        handle = (stream or torch.cuda.current_stream(self._workspace.device)).cuda_stream
        _native.call("mup_pull_plan_reset", self._plan, handle)
        self.epoch = 0

    def __call__(
        self,
        stream: torch.cuda.Stream | None = None,
        sync: "_native.MupSync | None" = None,
        stream_handle: int | None = None,
    ) -> None:
        if self.epoch >= self.workspace_epochs:
            raise RuntimeError(
                "pull workspace exhausted: call reset_workspace() before launching again"
            )
        if stream_handle is not None:
            handle = stream_handle
        else:
            handle = (stream or torch.cuda.current_stream(self._workspace.device)).cuda_stream
        if sync is None:
            _native.call("mup_pull_launch", self._plan, handle)
        else:
            # the hand-off with the staging peers is folded into the kernel
            _native.call("mup_pull_launch_synced", self._plan, handle, ctypes.byref(sync))
        self.epoch += 1

    def __del__(self) -> None:
        plan, self._plan = getattr(self, "_plan", None), None
        if plan:
            try:
                _native.lib().mup_pull_plan_destroy(plan)
            except Exception:
                pass


def compile_headshard_pull_gemm(
    peer_addresses: Tensor | Sequence[int],
    weight: Tensor,
    out: Tensor,
    dy: Tensor,
    *,
    logical_m: int,
    rank: int,
    up: int,
    bias: Tensor | None = None,
    workspace_epochs: int = 4096,
    peer_rows: int | None = None,
    enable_clc: bool = True,
    enable_bulk_pull: bool = True,
    hidden: int | None = None,
    max_active_ctas: int | None = None,
    num_c_stages: int | None = None,
    cta_group: int = 0,
    status_address: int = 0,
    timeout_ns: int = 5_000_000_000,
) -> CompiledHeadShardPullGemm:
    """Bind ``weight [N,K]``, ``bias``, the ``up`` staged peer arenas, the dense
    input buffer ``dy [rows,K]`` and the output buffer ``out [rows,N]``.

    ``peer_addresses`` holds the base address of every rank's arena (a device
    uint64 tensor such as ``MegaUPRuntime.peer_address_table``, read back to
    the host here, or a sequence of ints). ``enable_clc`` and
    ``enable_bulk_pull`` and ``num_c_stages`` are accepted for signature
    compatibility; this kernel has one scheduling and one pull strategy and
    always two accumulator slots. ``hidden``, when given, must be the pulled
    width K. ``max_active_ctas`` caps the grid so that the kernel stays fully
    resident next to other streams' kernels (the reference's runner leaves 16
    SMs free that way, tests/run_pull_gemm_contention.py:224-225 there).
    """

    del enable_clc, enable_bulk_pull, num_c_stages
    device = weight.device
    if hidden is not None and int(hidden) != int(weight.shape[1]):
        raise ValueError(f"hidden={hidden} must equal the weight's input width {int(weight.shape[1])}")
    if isinstance(peer_addresses, Tensor):
        addresses = [int(v) for v in peer_addresses.view(torch.int64).tolist()]
    else:
        addresses = [int(v) for v in peer_addresses]
    if len(addresses) != up:
        raise ValueError(f"expected {up} peer addresses, got {len(addresses)}")
    rows = int(logical_m)
    n, k = map(int, weight.shape)
    for name, tensor, shape in (("weight", weight, (n, k)), ("out", out, (rows, n)), ("dy", dy, (rows, k))):
        if (
            tensor.dtype != torch.bfloat16
            or tensor.device != device
            or not tensor.is_contiguous()
            or tuple(tensor.shape) != shape
        ):
            raise ValueError(f"{name} must be contiguous BF16 {shape} on {device}")
    if bias is not None and (
        bias.dtype != torch.bfloat16 or bias.device != device or tuple(bias.shape) != (n,)
        or not bias.is_contiguous()
    ):
        raise ValueError(f"bias must be contiguous BF16 ({n},) on {device}")
    if workspace_epochs <= 0:
        raise ValueError(f"workspace_epochs must be positive, got {workspace_epochs}")
    nbytes = int(_native.lib().mup_pull_workspace_bytes(rows))
    workspace = torch.zeros((nbytes + 127) // 128 * 16, dtype=torch.int64, device=device)
    if not cta_group:
        cta_group = int(os.environ.get("MEGA_UP_CTA_GROUP", "0"))
    plan = ctypes.c_void_p()
    _native.call("mup_set_max_active_ctas", int(max_active_ctas or 0))
    try:
        _native.call(
            "mup_pull_plan_create", ctypes.byref(plan), device.index, rows, n, k, int(up), int(rank),
            rows if peer_rows is None else int(peer_rows), weight.data_ptr(),
            None if bias is None else bias.data_ptr(), _native.pointer_array(addresses),
            dy.data_ptr(), out.data_ptr(), workspace.data_ptr(), int(cta_group),
            status_address or None, int(timeout_ns),
        )
    finally:
        _native.call("mup_set_max_active_ctas", 0)
    compiled = CompiledHeadShardPullGemm(
        plan, workspace, (weight, bias, out, dy), workspace_epochs, rows, int(rank), int(up)
    )
    compiled.describe_pull(k // int(up))
    return compiled
