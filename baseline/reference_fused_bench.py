"""Time the reference's OWN fused kernels (its CuTe-DSL peer-write GEMM and
head-shard pull GEMM, unmodified, from the install under baseline/_ref) on ONE
GPU with emulated peers, the way its tests/run_pull_gemm_contention.py does:
``up`` local buffers stand in for the peers' arenas, so every tensor map and
every load of the reference's kernels stays inside this GPU's memory.

    python baseline/reference_fused_bench.py --mode pull --rows 4096 --n 5120 --k 5120 --up 8

Prints one ``[REFERENCE_FUSED] {json}`` line: kernel time (CUDA events around
back-to-back launches, median of per-launch events as well), a cuBLAS
``F.linear`` of the same shape timed the same way, and whether the result
matches cuBLAS bit for bit. Single process, single GPU only; install the
reference first with baseline/install_reference.sh. Nothing of this repository's
own package is imported here.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE / "_ref"))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--mode", choices=("peer_write", "pull"), required=True)
    parser.add_argument("--rows", type=int, default=4096)
    parser.add_argument("--n", type=int, default=5120)
    parser.add_argument("--k", type=int, default=5120)
    parser.add_argument("--up", type=int, default=8)
    parser.add_argument("--rank", type=int, default=5)
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--no-bias", action="store_true")
    args = parser.parse_args()

    import mega_up  # the reference package

    if not Path(mega_up.__file__).resolve().is_relative_to(HERE / "_ref"):
        raise SystemExit(f"imported {mega_up.__file__}, not the reference install under {HERE / '_ref'}")
    device = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=device).manual_seed(1)

    def randn(shape, scale=1.0):
        return (torch.randn(shape, device=device, generator=gen) * scale).to(torch.bfloat16)

    rows, n, k, up, rank = args.rows, args.n, args.k, args.up, args.rank
    weight = randn((n, k), k ** -0.5)
    bias = None if args.no_bias else randn((n,), 0.02)
    report: dict[str, object] = {
        "mode": args.mode, "rows": rows, "n": n, "k": k, "up": up, "rank": rank, "bias": bias is not None,
        "package": str(Path(mega_up.__file__).parent),
    }
    started = time.perf_counter()
    if args.mode == "peer_write":
        from mega_up.kernels import peer_write_gemm as module

        x = randn((rows, k))
        slots = [torch.full((rows, n // up), float("nan"), device=device, dtype=torch.bfloat16) for _ in range(up)]
        # the reference binds [1, rows, .] views (mega_up/ops.py:677-714 there)
        bound = module.make_peer_write_launch(
            weight.unsqueeze(0), None, tuple(slot.unsqueeze(0) for slot in slots), a_shape=(1, rows, k), bias=bias,
            local_rank=rank,
        )
        x3d = x.unsqueeze(0)

        def launch() -> None:
            bound(x3d)

        launch()
        torch.cuda.synchronize(device)
        got = torch.cat(slots, dim=1)
        want = F.linear(x, weight, bias)

        def cublas() -> None:
            F.linear(x, weight, bias)
    else:
        from mega_up.kernels import headshard_pull_gemm as module

        shard = k // up
        peers = [randn((up, rows, shard)) for _ in range(up)]
        table = torch.tensor([p.data_ptr() for p in peers], dtype=torch.uint64, device=device)
        dy = torch.full((rows, k), float("nan"), device=device, dtype=torch.bfloat16)
        out = torch.full((rows, n), float("nan"), device=device, dtype=torch.bfloat16)
        epochs = 4096
        compiled = module.compile_headshard_pull_gemm(
            table, weight, out, dy, logical_m=rows, rank=rank, up=up, hidden=k, bias=bias,
            workspace_epochs=epochs, peer_rows=rows,
        )
        compiled()
        torch.cuda.synchronize(device)
        gathered = torch.cat([p[rank] for p in peers], dim=1)
        report["exchange_exact"] = bool(torch.equal(dy, gathered))
        got, want = out, F.linear(gathered, weight, bias)

        def launch() -> None:
            compiled()

        def cublas() -> None:
            F.linear(gathered, weight, bias)

    report["revision"] = getattr(module, "IMPLEMENTATION_REVISION", None)
    report["compile_s"] = round(time.perf_counter() - started, 1)
    report["bitwise_vs_cublas"] = bool(torch.equal(got, want))
    report["max_abs_diff"] = float((got.float() - want.float()).abs().max())

    def timed(fn) -> tuple[float, float]:
        for _ in range(3):
            fn()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        start.record()
        for _ in range(args.iters):
            fn()
        stop.record()
        torch.cuda.synchronize(device)
        back_to_back = start.elapsed_time(stop) * 1e3 / args.iters
        singles = []
        for _ in range(args.iters):
            start.record()
            fn()
            stop.record()
            stop.synchronize()
            singles.append(start.elapsed_time(stop) * 1e3)
        return back_to_back, statistics.median(singles)

    kernel_us, kernel_single_us = timed(launch)
    cublas_us, cublas_single_us = timed(cublas)
    report.update(
        us_per_launch=kernel_us, us_per_launch_isolated_median=kernel_single_us,
        cublas_us=cublas_us, cublas_isolated_median_us=cublas_single_us,
        tflops=2.0 * rows * n * k / kernel_us / 1e6, kernel_over_cublas=kernel_us / cublas_us,
    )
    print("[REFERENCE_FUSED] " + json.dumps(report), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
