"""Peer-write GEMM: ``bf16(A @ W.T + bias)`` whose column block ``p`` is stored
straight into rank ``p``'s arena slot by the kernel's epilogue.

Host handle of ``mup_peer_write_*`` in libmegaup.so; mirrors the seam of the
reference's ``mega_up/kernels/peer_write_gemm.py`` (``make_peer_write_launch``
at :2697-2930 returning a callable, ``peer_n_rotation`` at :977-993,
``PEER_TILE_N`` at :49-53). ``M`` (rows) is bound per launch object; nothing
is compiled at run time.
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch
from torch import Tensor

from .. import _native

IMPLEMENTATION_REVISION = "megaup-b200-cuda-r1"
PEER_TILE_N = 256


def peer_n_rotation(
    local_rank: int, num_peers: int, n_total: int, tile_n: int, cluster_n: int = 1
) -> int:
    """First N tile visited by ``local_rank``: every rank starts in its own
    column block, so at any moment the ranks of a group store into different
    destinations. Only the order of tiles changes, never a value."""

    n_tiles = -(-n_total // tile_n)
    n_clusters = -(-n_tiles // cluster_n)
    return (-(-(local_rank * n_clusters) // num_peers)) % n_clusters


def _as_2d(tensor: Tensor, name: str) -> Tensor:
    if tensor.ndim == 3 and tensor.shape[0] == 1:
        tensor = tensor[0]
    if tensor.ndim != 2:
        raise ValueError(f"{name} must be 2-D (or 3-D with a leading 1), got {tuple(tensor.shape)}")
    return tensor


def _check_bf16(tensor: Tensor, name: str, device: torch.device) -> None:
    if tensor.dtype != torch.bfloat16 or tensor.device != device or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous BF16 on {device}")


def _span(tensor: Tensor) -> tuple[int, int]:
    start = tensor.data_ptr()
    return start, start + tensor.numel() * tensor.element_size()


class PeerWriteLaunch:
    """Bound peer-write kernel: call it with ``A`` of the bound shape."""

    def __init__(
        self,
        plan: ctypes.c_void_p,
        weight: Tensor,
        bias: Tensor | None,
        peer_outs: tuple[Tensor, ...],
        rows: int,
        local_rank: int,
    ) -> None:
        self._plan = plan
        self.weight = weight
        self.bias = bias
        self.peer_outs = peer_outs
        self.rows = rows
        self.local_rank = local_rank
        self.out_features, self.in_features = map(int, weight.shape)
        grid, group, rotation, smem, tile = (ctypes.c_int() for _ in range(5))
        _native.call(
            "mup_peer_write_plan_info", plan, ctypes.byref(grid), ctypes.byref(group),
            ctypes.byref(rotation), ctypes.byref(smem), ctypes.byref(tile),
        )
        self.tile_n = tile.value
        self.grid_ctas = grid.value
        self.cta_group = group.value
        self.n_rotation = rotation.value
        self.smem_bytes = smem.value
        self._out_spans = tuple(_span(out) for out in peer_outs)

    def check(self, a: Tensor) -> Tensor:
        """The per-call contract on ``A`` (reference: PeerWriteLaunch.check,
        peer_write_gemm.py:2660-2675): BF16, the bound shape, contiguous, on the
        weight's device, not overlapping an output slot. Returns the 2-D view."""

        a = _as_2d(a, "A")
        if tuple(a.shape) != (self.rows, self.in_features):
            raise ValueError(
                f"A must have shape {(self.rows, self.in_features)}, got {tuple(a.shape)}"
            )
        _check_bf16(a, "A", self.weight.device)
        a_start, a_stop = _span(a)
        for start, stop in self._out_spans:
            if a_start < stop and start < a_stop:
                raise ValueError("A overlaps an output slot")
        return a

    def __call__(
        self, a: Tensor, sync: "_native.MupSync | None" = None, stream_handle: int | None = None
    ) -> None:
        a = self.check(a)
        stream = (
            stream_handle if stream_handle is not None else torch.cuda.current_stream(a.device).cuda_stream
        )
        if sync is None:
            _native.call("mup_peer_write_launch", self._plan, a.data_ptr(), stream)
        else:
            # the hand-off with the slots' owners is folded into the kernel
            _native.call(
                "mup_peer_write_launch_synced", self._plan, a.data_ptr(), stream, ctypes.byref(sync)
            )

    def __del__(self) -> None:
        plan, self._plan = getattr(self, "_plan", None), None
        if plan:
            try:
                _native.lib().mup_peer_write_plan_destroy(plan)
            except Exception:
                pass


def make_peer_write_launch(
    weight: Tensor,
    _unused: object,
    peer_outs: Sequence[Tensor],
    *,
    a_shape: Sequence[int],
    bias: Tensor | None = None,
    local_rank: int,
    cta_group: int = 0,
    status_address: int = 0,
    timeout_ns: int = 5_000_000_000,
) -> PeerWriteLaunch:
    """Bind ``weight [N,K]``, ``bias [N]`` and this rank's ``[rows, N/UP]`` slot
    in every peer arena; returns the launch callable.

    ``peer_outs[p]`` is the dense slot of this rank inside rank ``p``'s arena
    (``MegaUPRuntime.remote_write_views``). ``cta_group`` 1 or 2 selects the
    tcgen05 CTA pairing; 0 lets the library choose.
    """

    weight = _as_2d(weight, "weight")
    device = weight.device
    _check_bf16(weight, "weight", device)
    n, k = map(int, weight.shape)
    a_shape = tuple(int(v) for v in a_shape)
    if len(a_shape) == 3 and a_shape[0] == 1:
        a_shape = a_shape[1:]
    if len(a_shape) != 2 or a_shape[1] != k or a_shape[0] <= 0:
        raise ValueError(f"a_shape must be (rows, {k}), got {a_shape}")
    rows = a_shape[0]
    up = len(peer_outs)
    outs = tuple(_as_2d(out, "peer output") for out in peer_outs)
    if up == 0 or n % up:
        raise ValueError(f"out_features={n} must be divisible by the number of peers {up}")
    for out in outs:
        _check_bf16(out, "peer output", device)
        if tuple(out.shape) != (rows, n // up):
            raise ValueError(
                f"every peer output must be {(rows, n // up)}, got {tuple(out.shape)}"
            )
    if bias is not None:
        _check_bf16(bias, "bias", device)
        if tuple(bias.shape) != (n,):
            raise ValueError(f"bias must have shape ({n},), got {tuple(bias.shape)}")
    weight_span = _span(weight)
    for out in outs:
        start, stop = _span(out)
        if weight_span[0] < stop and start < weight_span[1]:
            raise ValueError("weight overlaps an output slot")
    if not cta_group:
        cta_group = int(os.environ.get("MEGA_UP_CTA_GROUP", "0"))
    plan = ctypes.c_void_p()
    _native.call(
        "mup_peer_write_plan_create", ctypes.byref(plan), device.index, rows, n, k, up,
        int(local_rank), weight.data_ptr(), None if bias is None else bias.data_ptr(),
        _native.pointer_array([out.data_ptr() for out in outs]), int(cta_group),
        status_address or None, int(timeout_ns),
    )
    return PeerWriteLaunch(plan, weight, bias, outs, rows, int(local_rank))


def prepare_peer_write(
    A: Tensor,
    B: Tensor,
    D: object,
    PeerOuts: Sequence[Tensor],
    *,
    bias: Tensor | None = None,
    local_rank: int = 0,
    **tile_options: object,
):
    """Bind a peer-write launch to one ``A``: returns a callable without
    arguments (reference: peer_write_gemm.py:2933-2980). The reference's tile and
    scheduler keywords are accepted and ignored: this kernel has one tile shape."""

    from functools import partial

    if not isinstance(A, Tensor):
        raise TypeError("peer_write requires a BF16 A tensor")
    del D, tile_options
    launch = make_peer_write_launch(
        B, None, PeerOuts, a_shape=tuple(A.shape), bias=bias, local_rank=local_rank
    )
    launch.check(A)
    return partial(launch, A)
