"""Helpers of the GPU tests: seeded inputs, conversions, and direct C-ABI
launches of the two kernels with single-process emulated peers."""

from __future__ import annotations

import ctypes

import numpy as np
import torch

from megaup_b200 import _native

DEVICE = torch.device("cuda", 0)
TIMEOUT_NS = 2_000_000_000


def to_gpu(values: np.ndarray | None) -> torch.Tensor | None:
    """float32 array of BF16-representable values -> BF16 tensor on the GPU."""

    if values is None:
        return None
    return torch.from_numpy(np.ascontiguousarray(values)).to(DEVICE).to(torch.bfloat16)


def to_host(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().float().cpu().numpy()


def seeded(shape, seed: int, *, ints: bool, scale: float = 1.0, lo: int = -4, hi: int = 5) -> torch.Tensor:
    """Seeded BF16 tensor on the GPU: small integers (every FP32 partial sum of a
    product with a ternary weight is then exact) or N(0, scale^2)."""

    gen = torch.Generator(device=DEVICE)
    gen.manual_seed(seed)
    if ints:
        return torch.randint(lo, hi, tuple(shape), device=DEVICE, generator=gen).to(torch.bfloat16)
    return (torch.randn(tuple(shape), device=DEVICE, generator=gen) * scale).to(torch.bfloat16)


class StatusWord:
    def __init__(self) -> None:
        self.host = ctypes.POINTER(ctypes.c_uint32)()
        self.device = ctypes.c_void_p()
        _native.call("mup_status_create", ctypes.byref(self.host), ctypes.byref(self.device))

    @property
    def value(self) -> int:
        return int(self.host[0])

    def close(self) -> None:
        _native.call("mup_status_destroy", self.host)


def stream_handle() -> int:
    return torch.cuda.current_stream(DEVICE).cuda_stream


def run_peer_write(x, weight, bias, *, up: int, rank: int, cta_group: int, guard_rows: int = 8):
    """Launch the peer-write kernel through the C ABI; ``up`` local buffers stand in
    for the slot of ``rank`` in every peer arena. Returns the slots and the
    rows behind them, which must stay NaN (no store beyond ``rows``)."""

    rows, k = x.shape
    n = weight.shape[0]
    shard = n // up
    slots = [torch.full((rows + guard_rows, shard), float("nan"), device=DEVICE, dtype=torch.bfloat16) for _ in range(up)]
    status = StatusWord()
    plan = ctypes.c_void_p()
    _native.call(
        "mup_peer_write_plan_create", ctypes.byref(plan), 0, rows, n, k, up, rank, weight.data_ptr(),
        None if bias is None else bias.data_ptr(),
        _native.pointer_array([s.data_ptr() for s in slots]), cta_group, status.device, TIMEOUT_NS,
    )
    try:
        _native.call("mup_peer_write_launch", plan, x.data_ptr(), stream_handle())
        torch.cuda.synchronize()
        assert status.value == 0, _native.decode_status(status.value)
    finally:
        _native.call("mup_peer_write_plan_destroy", plan)
        status.close()
    guards_clean = all(bool(torch.isnan(s[rows:]).all()) for s in slots)
    return [s[:rows] for s in slots], guards_clean


def run_pull(peers, weight, bias, *, rank: int, cta_group: int, launches: int = 1, guard_rows: int = 8):
    """Launch the pull kernel through the C ABI; ``peers[p]`` is rank ``p``'s staged
    arena ``[up(dest), rows, shard]``. Returns (dy, out, guards_clean)."""

    up = len(peers)
    _, rows, shard = peers[0].shape
    n, k = weight.shape
    dy = torch.full((rows, k), float("nan"), device=DEVICE, dtype=torch.bfloat16)
    out = torch.full((rows + guard_rows, n), float("nan"), device=DEVICE, dtype=torch.bfloat16)
    nbytes = int(_native.lib().mup_pull_workspace_bytes(rows))
    workspace = torch.zeros((nbytes + 127) // 128 * 16, dtype=torch.int64, device=DEVICE)
    status = StatusWord()
    plan = ctypes.c_void_p()
    _native.call(
        "mup_pull_plan_create", ctypes.byref(plan), 0, rows, n, k, up, rank, rows, weight.data_ptr(),
        None if bias is None else bias.data_ptr(),
        _native.pointer_array([p.data_ptr() for p in peers]), dy.data_ptr(), out.data_ptr(),
        workspace.data_ptr(), cta_group, status.device, TIMEOUT_NS,
    )
    try:
        for i in range(launches):
            if i:
                dy.fill_(float("nan"))
                out.fill_(float("nan"))
            _native.call("mup_pull_launch", plan, stream_handle())
        torch.cuda.synchronize()
        assert status.value == 0, _native.decode_status(status.value)
    finally:
        _native.call("mup_pull_plan_destroy", plan)
        status.close()
    return dy, out[:rows], bool(torch.isnan(out[rows:]).all())


def ulp_distance(a: torch.Tensor, b: torch.Tensor, floor: float = 2.0 ** -6) -> float:
    """Largest |a - b| in units of the BF16 ulp at max(|a|, |b|, floor).

    Two FP32 sums of the same products in different orders differ by an
    absolute error, so where the result cancels to (almost) zero the unit is
    the ulp at ``floor`` rather than the ulp of the tiny result itself.
    """

    a32, b32 = a.float(), b.float()
    scale = torch.maximum(torch.maximum(a32.abs(), b32.abs()), torch.full_like(a32, floor))
    ulp = torch.exp2(torch.floor(torch.log2(scale)) - 7)
    return float(((a32 - b32).abs() / ulp).max())


def representation_ulps(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance between two BF16 tensors counted in representable BF16
    values (the true ulp count, no floor): the bit patterns are mapped to
    integers that increase with the value, so neighbours differ by one whatever
    their magnitude. A result that cancels to almost zero can be many such ulps
    away from a differently ordered FP32 sum while being a tiny absolute error;
    `ulp_distance` (with its floor) is the pass/fail measure for those."""

    def ordered(t: torch.Tensor) -> torch.Tensor:
        bits = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        negative = bits >= 0x8000
        return torch.where(negative, 0x8000 - bits, bits)

    return int((ordered(a.to(torch.bfloat16)) - ordered(b.to(torch.bfloat16))).abs().max())
