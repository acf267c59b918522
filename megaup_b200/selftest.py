"""Run ONE kernel configuration on the current GPU with single-process emulated peers:
check it bit for bit against cuBLAS (``F.linear``) and time it with CUDA events.

    python -m megaup_b200.selftest --mode peer_write --rows 4096 --n 5120 --k 5120 --up 8 --rank 5
    python -m megaup_b200.selftest --mode pull --rows 4096 --n 5120 --k 5120 --up 8 --iters 20

The peers are ``up`` local buffers (the way the reference's
``tests/run_pull_gemm_contention.py`` emulates a UP group on one GPU), so the
kernel does all of its work - the GEMM plus the routed stores or the pulls -
without NVLink. Prints one ``[SELFTEST] {json}`` line; exits non-zero on a
mismatch or a device-side status code. Small enough to run under a profiler.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import sys

import torch
import torch.nn.functional as F

from . import _native


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--mode", choices=("peer_write", "pull"), default="peer_write")
    parser.add_argument("--rows", type=int, default=4096)
    parser.add_argument("--n", type=int, default=5120)
    parser.add_argument("--k", type=int, default=5120)
    parser.add_argument("--up", type=int, default=8)
    parser.add_argument("--rank", type=int, default=0)
    parser.add_argument("--cta-group", type=int, default=0)
    parser.add_argument("--no-bias", action="store_true")
    parser.add_argument("--iters", type=int, default=0, help="timed launches (0: correctness only)")
    parser.add_argument("--seed", type=int, default=1)
    parser.add_argument("--trace", action="store_true", help="report in-kernel cycle counters of the last launch")
    args = parser.parse_args()

    device = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=device).manual_seed(args.seed)

    def randn(shape, scale=1.0):
        return (torch.randn(shape, device=device, generator=gen) * scale).to(torch.bfloat16)

    rows, n, k, up, rank = args.rows, args.n, args.k, args.up, args.rank
    weight = randn((n, k), k ** -0.5)
    bias = None if args.no_bias else randn((n,), 0.02)
    host_status = ctypes.POINTER(ctypes.c_uint32)()
    device_status = ctypes.c_void_p()
    _native.call("mup_status_create", ctypes.byref(host_status), ctypes.byref(device_status))
    stream = torch.cuda.current_stream(device).cuda_stream
    timeout_ns = 2_000_000_000
    plan = ctypes.c_void_p()
    grid, group, smem, tile = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    report: dict[str, object] = {
        "mode": args.mode, "rows": rows, "n": n, "k": k, "up": up, "rank": rank, "bias": bias is not None,
    }

    if args.mode == "peer_write":
        x = randn((rows, k))
        shard = n // up
        slots = [torch.full((rows, shard), float("nan"), device=device, dtype=torch.bfloat16) for _ in range(up)]
        _native.call(
            "mup_peer_write_plan_create", ctypes.byref(plan), device.index, rows, n, k, up, rank,
            weight.data_ptr(), None if bias is None else bias.data_ptr(),
            _native.pointer_array([s.data_ptr() for s in slots]), args.cta_group, device_status, timeout_ns,
        )
        rotation = ctypes.c_int()
        _native.call(
            "mup_peer_write_plan_info", plan, ctypes.byref(grid), ctypes.byref(group),
            ctypes.byref(rotation), ctypes.byref(smem), ctypes.byref(tile),
        )

        def launch() -> None:
            _native.call("mup_peer_write_launch", plan, x.data_ptr(), stream)

        launch()
        torch.cuda.synchronize(device)
        got = torch.cat(slots, dim=1)
        want = F.linear(x, weight, bias)
        report["exchange_exact"] = True  # routing is part of `got`: column block p came from slot p
    else:
        shard = k // up
        peers = [randn((up, rows, shard)) for _ in range(up)]
        dy = torch.full((rows, k), float("nan"), device=device, dtype=torch.bfloat16)
        out = torch.full((rows, n), float("nan"), device=device, dtype=torch.bfloat16)
        nbytes = int(_native.lib().mup_pull_workspace_bytes(rows))
        workspace = torch.zeros((nbytes + 127) // 128 * 16, dtype=torch.int64, device=device)
        _native.call(
            "mup_pull_plan_create", ctypes.byref(plan), device.index, rows, n, k, up, rank, rows,
            weight.data_ptr(), None if bias is None else bias.data_ptr(),
            _native.pointer_array([p.data_ptr() for p in peers]), dy.data_ptr(), out.data_ptr(),
            workspace.data_ptr(), args.cta_group, device_status, timeout_ns,
        )
        launches = ctypes.c_uint64()
        _native.call(
            "mup_pull_plan_info", plan, ctypes.byref(grid), ctypes.byref(group),
            ctypes.byref(launches), ctypes.byref(smem), ctypes.byref(tile),
        )

        def launch() -> None:
            _native.call("mup_pull_launch", plan, stream)

        launch()
        torch.cuda.synchronize(device)
        gathered = torch.cat([p[rank] for p in peers], dim=1)
        report["exchange_exact"] = bool(torch.equal(dy, gathered))
        got = out
        want = F.linear(gathered, weight, bias)

    status = int(host_status[0])
    report.update(
        grid_ctas=grid.value, cta_group=group.value, tile_n=tile.value, smem_bytes=smem.value, status=status,
        status_text=_native.decode_status(status),
        bitwise_vs_cublas=bool(torch.equal(got, want)),
        mismatches=int((got != want).sum()),
        max_abs_diff=float(torch.nan_to_num((got.float() - want.float()).abs(), nan=1e9).max()),
    )
    trace = None
    if args.trace:
        trace = torch.zeros((grid.value, 16), dtype=torch.int64, device=device)
        setter = "mup_peer_write_plan_set_trace" if args.mode == "peer_write" else "mup_pull_plan_set_trace"
        _native.call(setter, plan, trace.data_ptr())
    if args.iters and status == 0:
        for _ in range(3):
            launch()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        start.record()
        for _ in range(args.iters):
            launch()
        stop.record()
        torch.cuda.synchronize(device)
        us = start.elapsed_time(stop) * 1e3 / args.iters
        report["us_per_launch"] = us
        report["tflops"] = 2.0 * rows * n * k / us / 1e6
        report["status_after_timing"] = int(host_status[0])
    if trace is not None:
        trace.zero_()
        launch()
        torch.cuda.synchronize(device)
        t = trace.cpu().double()
        cycles = t[:, 1] - t[:, 0]
        ns = t[:, 7] - t[:, 6]
        leaders = t[:: max(group.value, 1)]
        report["trace"] = {
            "cta_cycles_max": float(cycles.max()), "cta_cycles_mean": float(cycles.mean()),
            "kernel_ns": float(t[:, 7].max() - t[:, 6].min()),
            "sm_mhz": float((cycles / ns).mean() * 1e3),
            "mma_wait_operands_mean": float(leaders[:, 2].mean()), "mma_wait_operands_max": float(leaders[:, 2].max()),
            "mma_wait_accumulator_mean": float(leaders[:, 3].mean()),
            "producer_wait_stage_mean": float(t[:, 4].mean()),
            "epilogue_wait_mean": float(t[:, 5].mean()),
            "setup_done_us_mean_max": [float(t[:, 12].mean()) / 1e3, float(t[:, 12].max()) / 1e3],
            "first_operands_us_min_mean_max": [
                float(leaders[:, 14].min()) / 1e3, float(leaders[:, 14].mean()) / 1e3, float(leaders[:, 14].max()) / 1e3,
            ],
            "items_per_cta_min_max": [float(leaders[:, 15].min()), float(leaders[:, 15].max())],
        }
        if args.mode == "pull":
            report["trace"]["pull_done_us_after_start"] = float(t[:, 8].max() - t[:, 6].min()) / 1e3
            report["trace"]["pull_tickets_min_max"] = [float(t[:, 9].min()), float(t[:, 9].max())]
            report["trace"]["first_ticket_stored_us_min_mean_max"] = [
                float(t[:, 13].min()) / 1e3, float(t[:, 13].mean()) / 1e3, float(t[:, 13].max()) / 1e3,
            ]
            gate = t[:, 10] / 1e3
            report["trace"]["first_gate_open_us_min_mean_max"] = [float(gate.min()), float(gate.mean()), float(gate.max())]
            report["trace"]["gate_cycles_mean"] = float(t[:, 11].mean())
    print("[SELFTEST] " + json.dumps(report), flush=True)
    ok = status == 0 and report["exchange_exact"] and (report["bitwise_vs_cublas"] or rows < 256)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
