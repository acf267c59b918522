"""The allocation-free pull entry point, called through the C ABI.

``mup_pull_gemm_noalloc`` serves callers that cannot allocate device memory
where they call it: code running while a memory pool is fully committed,
inside a region where a framework forbids allocator calls, or a host that may
only pass on buffers it was given. Its ticket cursor and ready counts live in
a fixed array inside the library's device image instead of a caller-provided
workspace. The result must equal, bit for bit, what the existing entry points
(``mup_pull_plan_create`` + ``mup_pull_launch``) produce from the same inputs
- on two calls in a row, because every call reuses the same array and has to
clear what the previous call left in it.

This file sorts last on purpose: a run that stops at the first failure has
already run every other test.
"""

from __future__ import annotations

import ctypes

import pytest
import torch

import _gpu_harness as h
from megaup_b200 import _native

pytestmark = pytest.mark.gpu

MAX_ROWS = 262144  # MUP_NOALLOC_MAX_ROWS in include/megaup.h


def _no_alloc_pull(peers, weight, bias, *, rank, cta_group, guard_rows=8, check_device_memory=False):
    up = len(peers)
    _, rows, shard = peers[0].shape
    n, k = weight.shape
    dy = torch.full((rows, k), float("nan"), device=h.DEVICE, dtype=torch.bfloat16)
    out = torch.full((rows + guard_rows, n), float("nan"), device=h.DEVICE, dtype=torch.bfloat16)
    status = h.StatusWord()
    # every buffer exists before the call; the call itself may not allocate
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(h.DEVICE)
    # torch's counter does not see a cudaMalloc made inside the library; the
    # driver's free-memory figure does (checked once the one-time set-up of the
    # first call on this device is behind us)
    free_before, _ = torch.cuda.mem_get_info(h.DEVICE)
    _native.call(
        "mup_pull_gemm_noalloc", h.DEVICE.index, rows, n, k, up, rank, rows, weight.data_ptr(),
        None if bias is None else bias.data_ptr(),
        _native.pointer_array([p.data_ptr() for p in peers]), dy.data_ptr(), out.data_ptr(),
        cta_group, status.device, h.TIMEOUT_NS, h.stream_handle(),
    )
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(h.DEVICE) == before
    if check_device_memory:
        assert torch.cuda.mem_get_info(h.DEVICE)[0] == free_before, "the call changed the device's free memory"
    assert status.value == 0, _native.decode_status(status.value)
    status.close()
    return dy, out[:rows], bool(torch.isnan(out[rows:]).all())


@pytest.mark.parametrize("cta_group", [0, 1])
def test_two_calls_in_a_row_match_the_plan_entry_points(cta_group: int) -> None:
    # the second call is smaller than the first: counts the first call left
    # behind in the shared array must not be taken for finished panels
    shapes = [(1000, 1024, 2048, 8, 3), (300, 512, 1024, 4, 1)]
    for rows, n, k, up, rank in shapes:
        weight = h.seeded((n, k), 81, ints=False, scale=k ** -0.5)
        bias = h.seeded((n,), 82, ints=False, scale=0.02)
        peers = [h.seeded((up, rows, k // up), 90 + p, ints=False) for p in range(up)]
        want_dy, want_out, _ = h.run_pull(peers, weight, bias, rank=rank, cta_group=cta_group or 2)
        dy, out, guards_clean = _no_alloc_pull(peers, weight, bias, rank=rank, cta_group=cta_group)
        assert guards_clean, "a store went past the last row"
        assert torch.equal(dy, want_dy)
        assert torch.equal(out, want_out)  # same kernel, same inputs: bit-exact
    # and the very same call twice
    dy2, out2, _ = _no_alloc_pull(peers, weight, bias, rank=rank, cta_group=cta_group, check_device_memory=True)
    assert torch.equal(dy2, want_dy) and torch.equal(out2, want_out)


def test_a_call_for_another_device_than_the_current_one_is_rejected() -> None:
    lib = _native.lib()
    dummy = torch.zeros(8, device=h.DEVICE, dtype=torch.bfloat16)
    peers = _native.pointer_array([dummy.data_ptr()] * 2)
    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second device ordinal to name")
    other = (h.DEVICE.index + 1) % torch.cuda.device_count()
    code = lib.mup_pull_gemm_noalloc(
        other, 64, 256, 256, 2, 0, 64, dummy.data_ptr(), None, peers, dummy.data_ptr(), dummy.data_ptr(),
        0, None, 1000, None,
    )
    assert code == -1 and b"current device" in lib.mup_last_error()


def test_sizes_beyond_the_built_in_scratch_are_rejected_with_a_clear_error() -> None:
    lib = _native.lib()
    dummy = torch.zeros(8, device=h.DEVICE, dtype=torch.bfloat16)
    peers = _native.pointer_array([dummy.data_ptr()] * 2)
    code = lib.mup_pull_gemm_noalloc(
        h.DEVICE.index, MAX_ROWS + 1, 256, 256, 2, 0, MAX_ROWS + 1, dummy.data_ptr(), None, peers,
        dummy.data_ptr(), dummy.data_ptr(), 0, None, 1000, None,
    )
    assert code == -1
    message = lib.mup_last_error().decode()
    assert "MUP_NOALLOC_MAX_ROWS" in message and str(MAX_ROWS) in message
    # other contract violations are rejected before anything is launched
    assert lib.mup_pull_gemm_noalloc(
        h.DEVICE.index, 64, 256, 384, 2, 0, 64, dummy.data_ptr(), None, peers, dummy.data_ptr(), dummy.data_ptr(),
        0, None, 1000, None,
    ) == -1
    torch.cuda.synchronize()
