"""Parity of the two CUDA kernels, called through the C ABI with emulated peers:
bit-exact against the CPU oracle on integer-valued inputs (every partial sum
exact, so the result does not depend on summation order), bit-exact against
cuBLAS (F.linear on the same GPU) on random inputs wherever cuBLAS does not
split K, within 1 BF16 ulp where it does."""

from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import _gpu_harness as h
from oracle import ulysses_oracle as oracle

pytestmark = pytest.mark.gpu

# (rows, N, K, UP, rank): shapes of the reference's configurations and edge cases
PEER_SHAPES = [
    (128, 256, 64, 2, 0),          # one tile, one K step
    (200, 1024, 1040, 8, 3),       # K % 64 != 0, shard (128) narrower than a tile, ragged M
    (17, 512, 512, 2, 1),          # fewer rows than one epilogue warp
    (512, 2304, 2304, 2, 1),       # odd number of 256-column tiles
    (1024, 2048, 2048, 8, 6),      # LTX-shaped, head_dim 64
    (64, 1024, 4096, 8, 2),        # Llama-3-8B K projection, small M (cuBLAS splits K)
    (256, 1536, 1536, 2, 0),       # CPU plumbing configuration of the reference
    (4096, 5120, 5120, 8, 5),      # Wan2.1-14B Q projection, 640-column shards straddle tiles
    (4096, 5120, 5120, 4, 3),
    (4096, 5120, 5120, 2, 1),
    (8192, 6144, 4096, 8, 7),      # Llama-3-8B fused QKV
]
PULL_SHAPES = [
    (128, 256, 256, 2, 0),
    (200, 512, 1024, 8, 3),        # shard 128, ragged M
    (17, 256, 512, 2, 1),
    (512, 2304, 2304, 2, 0),
    (1024, 2048, 2048, 8, 6),
    (4096, 5120, 5120, 8, 5),      # Wan2.1-14B O projection
    (4096, 5120, 5120, 4, 0),
    (4096, 5120, 5120, 2, 1),
    (16384, 8192, 8192, 8, 4),     # Llama-3-70B O projection
    (256, 256, 16384, 2, 1),       # a shard row (16 KB) wider than one pull ticket: two column segments
    (130, 512, 12288, 2, 0),       # 12 KB shard rows, two segments of 6 KB, ragged M
]


def _weights(n, k, seed, ints, bias=True):
    w = h.seeded((n, k), seed, ints=ints, scale=k ** -0.5, lo=-1, hi=2)
    b = h.seeded((n,), seed + 1, ints=ints, scale=0.02, lo=-3, hi=4) if bias else None
    return w, b


def _oracle_linear(x, w, b, max_rows=1024):
    """Oracle rows: all of them for small problems, a spread sample otherwise."""

    rows = x.shape[0]
    pick = np.arange(rows) if rows <= max_rows else np.unique(
        np.concatenate([np.arange(0, 160), np.arange(rows - 160, rows), np.arange(0, rows, max(1, rows // 640))])
    )
    xs = h.to_host(x)[pick]
    return pick, oracle.linear(xs, h.to_host(w), None if b is None else h.to_host(b), use_c=False)


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("rows,n,k,up,rank", PEER_SHAPES)
def test_peer_write_kernel(rows, n, k, up, rank, cta_group) -> None:
    shard = n // up
    # integer-valued: bit-exact against the CPU oracle, routed per peer_write_route
    w, b = _weights(n, k, 11, True)
    x = h.seeded((rows, k), 12, ints=True)
    slots, guards_clean = h.run_peer_write(x, w, b, up=up, rank=rank, cta_group=cta_group)
    assert guards_clean, "a store went past the last row"
    pick, want = _oracle_linear(x, w, b)
    got = torch.cat(slots, dim=1)
    assert np.array_equal(h.to_host(got)[pick], want)
    for col in range(0, n, 64):
        dst, lcol = oracle.peer_write_route(col, shard)
        assert torch.equal(slots[dst][:, lcol : lcol + 64], got[:, col : col + 64])
    # random-valued, with and without bias: bit-exact against cuBLAS
    for bias in (True, False):
        w, b = _weights(n, k, 21, False, bias)
        x = h.seeded((rows, k), 22, ints=False)
        slots, guards_clean = h.run_peer_write(x, w, b, up=up, rank=rank, cta_group=cta_group)
        assert guards_clean
        got = torch.cat(slots, dim=1)
        ref = F.linear(x, w, b)
        if torch.equal(got, ref):
            continue
        # cuBLAS splits K for small M: then compare with the same rows of a
        # 4096-row cuBLAS call (bit-exact) and with the small call (<= 1 ulp)
        assert rows < 256, "cuBLAS and the kernel differ on a large-M problem"
        padded = torch.zeros((4096, k), device=h.DEVICE, dtype=torch.bfloat16)
        padded[:rows] = x
        assert torch.equal(got, F.linear(padded, w, b)[:rows])
        assert h.ulp_distance(got, ref) <= 1


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("rows,n,k,up,rank", PULL_SHAPES)
def test_pull_kernel(rows, n, k, up, rank, cta_group) -> None:
    shard = k // up
    for ints in (True, False):
        w, b = _weights(n, k, 31 + ints, ints)
        peers = [h.seeded((up, rows, shard), 40 + p, ints=ints) for p in range(up)]
        dy, out, guards_clean = h.run_pull(peers, w, b, rank=rank, cta_group=cta_group, launches=2)
        assert guards_clean, "a store went past the last row"
        # the pulled dense input is a pure gather: always bit-exact
        want_dy = torch.cat([p[rank] for p in peers], dim=1)
        assert torch.equal(dy, want_dy)
        if rows <= 4096:
            host = oracle.pull_gather([h.to_host(p).reshape(-1) for p in peers], rank, rows, shard)
            assert np.array_equal(h.to_host(dy), host)
        if ints:
            pick, want = _oracle_linear(want_dy, w, b)
            assert np.array_equal(h.to_host(out)[pick], want)
        else:
            ref = F.linear(want_dy, w, b)
            if not torch.equal(out, ref):
                # only outputs too small to fill the GPU, where cuBLAS splits K
                assert rows < 256 or rows * n <= 256 * 512
                assert h.ulp_distance(out, ref) <= 1


@pytest.mark.parametrize("rows,n,k,up,rank", [(4096, 5120, 5120, 8, 5), (640, 2304, 1024, 2, 1), (200, 1024, 1040, 8, 3)])
def test_the_schedule_never_changes_a_bit(rows, n, k, up, rank, monkeypatch) -> None:
    """Item width, the cut-up last round, the issue sequence and whether the CTAs
    draw their items from a feed or have them assigned only decide which SM
    computes which columns when: every K loop stays whole and ascending, so all
    variants must give identical bits."""

    x = h.seeded((rows, k), 71, ints=False)
    w, b = _weights(n, k, 72, False)
    # the pull GEMM contracts over the exchanged width, which must obey the shape rule: use n
    peers = [h.seeded((up, rows, n // up), 80 + p, ints=False) for p in range(up)]
    w_pull, b_pull = _weights(n, n, 73, False)
    results = []
    variants = [
        {}, {"MEGA_UP_SPLIT_TAIL": "0"}, {"MEGA_UP_ITEM_UNITS": "2"}, {"MEGA_UP_ITEM_UNITS": "3", "MEGA_UP_KERNEL_FLAGS": "2"},
        {"MEGA_UP_ITEM_UNITS": "8"}, {"MEGA_UP_ITEM_FEED": "1"}, {"MEGA_UP_ITEM_FEED": "1", "MEGA_UP_ITEM_UNITS": "7"},
        {"MEGA_UP_ITEM_FEED": "0", "MEGA_UP_ITEM_UNITS": "1"}, {"MEGA_UP_BAND": "1"}, {"MEGA_UP_BAND": "4", "MEGA_UP_BAND_INTERLEAVE": "0"},
        {"MEGA_UP_PULL_PACE_NS": "5"},
    ]
    names = ("MEGA_UP_SPLIT_TAIL", "MEGA_UP_ITEM_UNITS", "MEGA_UP_KERNEL_FLAGS", "MEGA_UP_ITEM_FEED", "MEGA_UP_BAND",
             "MEGA_UP_BAND_INTERLEAVE", "MEGA_UP_PULL_PACE_NS")
    for env in variants:
        for name in names:
            monkeypatch.delenv(name, raising=False)
        for name, value in env.items():
            monkeypatch.setenv(name, value)
        slots, clean = h.run_peer_write(x, w, b, up=up, rank=rank, cta_group=2)
        _, out, clean_pull = h.run_pull(peers, w_pull, b_pull, rank=rank, cta_group=2)
        assert clean and clean_pull
        results.append((torch.cat(slots, dim=1), out))
    for got_pw, got_pull in results[1:]:
        assert torch.equal(got_pw, results[0][0])
        assert torch.equal(got_pull, results[0][1])


def test_pull_kernel_is_bit_stable_across_many_launches_under_contention() -> None:
    """Every launch reuses the same monotonically increasing counters; a side
    stream keeps SMs busy so CTAs start at different times."""

    rows, n, k, up, rank = 1000, 1024, 2048, 8, 3
    w, b = _weights(n, k, 51, False)
    peers = [h.seeded((up, rows, k // up), 60 + p, ints=False) for p in range(up)]
    side = torch.cuda.Stream()
    noise = torch.randn(4096, 4096, device=h.DEVICE)
    with torch.cuda.stream(side):
        for _ in range(20):
            noise = torch.nn.functional.gelu(noise @ noise.t() * 1e-3)
    dy, out, guards_clean = h.run_pull(peers, w, b, rank=rank, cta_group=2, launches=50)
    side.synchronize()
    assert guards_clean
    want_dy = torch.cat([p[rank] for p in peers], dim=1)
    assert torch.equal(dy, want_dy)
    assert torch.equal(out, F.linear(want_dy, w, b))


def test_layout_copy_kernels() -> None:
    import ctypes

    from megaup_b200 import _native

    up, batch, seq, shard = 4, 3, 37, 384
    src = h.seeded((up * batch * seq, shard), 70, ints=False)
    dst = torch.empty_like(src)
    _native.call("mup_regroup_rows", dst.data_ptr(), src.data_ptr(), up, batch, seq, shard, 1, h.stream_handle())
    want = oracle.copy_peer_written(h.to_host(src).reshape(-1), up, batch, seq, shard)
    assert np.array_equal(h.to_host(dst).reshape(want.shape), want)
    back = torch.empty_like(src)
    _native.call("mup_regroup_rows", back.data_ptr(), dst.data_ptr(), up, batch, seq, shard, 0, h.stream_handle())
    assert torch.equal(back, src)
    staged = oracle.stage_head_parallel(h.to_host(dst).reshape(batch, up * seq, 1, shard), up)
    assert np.array_equal(h.to_host(back).reshape(-1), staged)
    layout = oracle.thd_layout((0, 5, 5, 40, 111), up)
    index = torch.from_numpy(layout["to_thd_index"]).to(h.DEVICE)
    gathered = torch.empty_like(src)
    _native.call("mup_gather_rows", gathered.data_ptr(), src.data_ptr(), index.data_ptr(), src.shape[0], shard, h.stream_handle())
    torch.cuda.synchronize()
    assert np.array_equal(h.to_host(gathered), h.to_host(src)[layout["to_thd_index"]])
    # misaligned buffers and ragged widths are rejected, not truncated
    lib = _native.lib()
    assert lib.mup_gather_rows(gathered.data_ptr() + 2, src.data_ptr(), None, 4, shard, None) == -1
    assert lib.mup_gather_rows(gathered.data_ptr(), src.data_ptr(), None, 4, 12, None) == -1


def test_a_flag_nobody_raises_times_out_and_the_context_survives() -> None:
    """A bounded wait that runs out must end the kernel with a status code."""

    import ctypes

    from megaup_b200 import _native

    flags = [torch.zeros(8, dtype=torch.int32, device=h.DEVICE) for _ in range(2)]
    status = h.StatusWord()
    _native.call(
        "mup_flag_barrier", _native.pointer_array([f.data_ptr() for f in flags]), 2, 0, 1,
        status.device, 20_000_000, h.stream_handle(),
    )
    torch.cuda.synchronize()
    assert status.value >> 24 == 7 and status.value & 0xFFFFFF == 1  # waited for rank 1
    assert int(flags[0][0]) == 1 and int(flags[1][0]) == 1  # own arrival was published everywhere
    # the context is intact: a barrier whose peer has arrived completes
    status.host[0] = 0
    flags[0][1] = 2
    _native.call(
        "mup_flag_barrier", _native.pointer_array([f.data_ptr() for f in flags]), 2, 0, 2,
        status.device, 20_000_000, h.stream_handle(),
    )
    torch.cuda.synchronize()
    assert status.value == 0
    status.close()


def test_a_pull_whose_hand_off_never_comes_gives_up_and_the_plan_recovers() -> None:
    """The pull workers wait (bounded) for the peers' staging hand-off. Nobody
    raises the flag here: the launch must end with the hand-off status code, and
    after a plan reset the same plan must run bit-exactly."""

    import ctypes

    from megaup_b200 import _native

    rows, n, k, up, rank = 300, 512, 1024, 2, 1
    w, b = _weights(n, k, 91, False)
    peers = [h.seeded((up, rows, k // up), 95 + p, ints=False) for p in range(up)]
    dy = torch.full((rows, k), float("nan"), device=h.DEVICE, dtype=torch.bfloat16)
    out = torch.full((rows, n), float("nan"), device=h.DEVICE, dtype=torch.bfloat16)
    nbytes = int(_native.lib().mup_pull_workspace_bytes(rows))
    workspace = torch.zeros((nbytes + 127) // 128 * 16, dtype=torch.int64, device=h.DEVICE)
    status = h.StatusWord()
    plan = ctypes.c_void_p()
    _native.call(
        "mup_pull_plan_create", ctypes.byref(plan), h.DEVICE.index, rows, n, k, up, rank, rows, w.data_ptr(),
        b.data_ptr(), _native.pointer_array([p.data_ptr() for p in peers]), dy.data_ptr(), out.data_ptr(),
        workspace.data_ptr(), 2, status.device, h.TIMEOUT_NS,
    )
    try:
        flags = [torch.zeros(8, dtype=torch.int32, device=h.DEVICE) for _ in range(up)]
        flag_array = _native.pointer_array([f.data_ptr() for f in flags])
        sync = _native.MupSync(
            peer_flags=flag_array, up=up, rank=rank, wait_epoch=1, signal_epoch=0, done_counter=None,
            done_before=0, done_after=0, status_device_ptr=status.device, timeout_ns=20_000_000,
        )
        _native.call("mup_pull_launch_synced", plan, h.stream_handle(), ctypes.byref(sync))
        torch.cuda.synchronize()
        assert status.value >> 24 == 7, _native.decode_status(status.value)
        # recover: clear the word, zero the counters, launch normally
        status.host[0] = 0
        _native.call("mup_pull_plan_reset", plan, h.stream_handle())
        _native.call("mup_pull_launch", plan, h.stream_handle())
        torch.cuda.synchronize()
        assert status.value == 0, _native.decode_status(status.value)
        want_dy = torch.cat([p[rank] for p in peers], dim=1)
        assert torch.equal(dy, want_dy)
        assert torch.equal(out, F.linear(want_dy, w, b))
    finally:
        _native.call("mup_pull_plan_destroy", plan)
        status.close()


def test_plan_creation_rejects_what_the_kernels_cannot_run() -> None:
    import ctypes

    from megaup_b200 import _native

    lib = _native.lib()
    w = torch.zeros(512, 512, device=h.DEVICE, dtype=torch.bfloat16)
    slots = [torch.zeros(8, 256, device=h.DEVICE, dtype=torch.bfloat16) for _ in range(2)]
    ptrs = _native.pointer_array([s.data_ptr() for s in slots])
    plan = ctypes.c_void_p()
    args = lambda **kw: (  # noqa: E731
        ctypes.byref(plan), 0, kw.get("rows", 8), kw.get("n", 512), kw.get("k", 512), kw.get("up", 2),
        kw.get("rank", 0), w.data_ptr(), kw.get("bias"), ptrs, kw.get("g", 0), None, 1000,
    )
    assert lib.mup_peer_write_plan_create(*args(up=3)) == -1
    assert lib.mup_peer_write_plan_create(*args(n=384)) == -1
    assert lib.mup_peer_write_plan_create(*args(k=100)) == -1
    assert lib.mup_peer_write_plan_create(*args(rank=2)) == -1
    assert lib.mup_peer_write_plan_create(*args(bias=w.data_ptr() + 2)) == -1
    assert lib.mup_peer_write_plan_create(*args(g=3)) == -1
    assert lib.mup_peer_write_plan_create(*args()) == 0
    assert lib.mup_peer_write_launch(plan, w.data_ptr() + 2, None) == -1  # misaligned A
    lib.mup_peer_write_plan_destroy(plan)
