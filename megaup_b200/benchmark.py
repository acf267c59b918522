"""Benchmark of the fused operators over the shapes of the reference's benchmark, one
Ulysses group per run (same paths and timing protocol as the reference's
``benchmarks/bench_bshd.py``: fused prepared API, kernel only, the unfused
torch pipeline - cuBLAS + permute + NCCL ``all_to_all_single`` + output copy -
and the dense cuBLAS GEMM; warm-ups, per-iteration CUDA events, rank-max per
sample, path order rotated every iteration, medians).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node U --master-addr 127.0.0.1 \
        --master-port 29540 -m megaup_b200.benchmark [--configs wan_q,wan_o,...] [--iters 30]

With one process (no torchrun) a UP=8 group is emulated on the GPU and only the
kernel / cuBLAS columns are real exchanges-free numbers. Rank 0 prints one
``[BENCH_RESULT] {json}`` line per configuration and a table at the end.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

import megaup_b200 as mega_up
from megaup_b200.kernels import peer_write_gemm

NVLINK_BYTES_PER_S = 665e9  # measured: peer loads with every rank reading at once (nvlink_probe)

# name -> (direction, layout, rows-defining dims, N, K, head_dim, bias, scale of W, only_up)
CONFIGS = {
    # Wan2.1-14B-shaped attention: Q projection (peer-write) and O projection (pull)
    "wan_q": ("pw", "bshd", dict(batch=1, sequence=4096), 5120, 5120, 128, True, None, None),
    "wan_o": ("pull", "bshd", dict(batch=1, sequence=4096), 5120, 5120, 128, True, None, None),
    # Llama-3-8B fused QKV, sequence-first, no bias
    "llama8b_qkv": ("pw", "sbhd", dict(sequence=8192, batch=1), 6144, 4096, 128, False, 1 / 64, None),
    # Llama-3-70B O projection, packed THD with a split-sample layout, UP = 8 only
    "llama70b_o": ("pull", "thd", dict(tokens=16384), 8192, 8192, 128, False, None, 8),
    # the point the reference's README quotes its ratios on: hidden 5120, packed THD with a split-sample
    # layout, 65 536 tokens per rank (run these two alone: they need a runtime of their own size)
    "ref64k_q": ("pw", "thd", dict(tokens=65536), 5120, 5120, 128, False, None, None),
    "ref64k_o": ("pull", "thd", dict(tokens=65536), 5120, 5120, 128, False, None, None),
    # shape-edge sweep
    "edge_2304_b4": ("pw", "bshd", dict(batch=4, sequence=128), 2304, 2304, 128, True, None, 2),
    "edge_ltx_2048": ("pw", "bshd", dict(batch=1, sequence=1024), 2048, 2048, 64, True, None, 8),
    "edge_kproj_m64": ("pw", "bshd", dict(batch=1, sequence=64), 1024, 4096, 128, True, None, 8),
}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--configs", default=",".join(name for name in CONFIGS if not name.startswith("ref64k")))
    parser.add_argument("--iters", type=int, default=30)
    parser.add_argument("--warmup", type=int, default=10)
    args = parser.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        dist.init_process_group("nccl", device_id=device)
    up = world if distributed else 8
    peak = 1647.8
    peaks_file = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(peaks_file):
        peak = float(json.load(open(peaks_file))["bf16_tflops"])

    def randn(shape, seed, scale=1.0):
        gen = torch.Generator(device=device).manual_seed(seed)
        return (torch.randn(shape, device=device, generator=gen) * scale).to(torch.bfloat16)

    def rank_max(values: list[float]) -> list[float]:
        if not distributed:
            return values
        t = torch.tensor(values, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def sync_all() -> None:
        torch.cuda.synchronize(device)
        if distributed:
            dist.barrier()
            torch.cuda.synchronize(device)

    def time_paths(paths: dict[str, object]) -> dict[str, float]:
        """Median over iterations of the rank-max time of each path, order rotated."""

        names = list(paths)
        for _ in range(args.warmup):
            for name in names:
                paths[name]()
        sync_all()
        samples: dict[str, list[float]] = {name: [] for name in names}
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(args.iters):
            order = names[it % len(names):] + names[: it % len(names)]
            for name in order:
                if distributed:
                    dist.barrier()
                start.record()
                paths[name]()
                stop.record()
                stop.synchronize()
                samples[name].append(start.elapsed_time(stop) * 1e3)
        return {name: statistics.median(rank_max(values)) for name, values in samples.items()}

    results = []
    for name in args.configs.split(","):
        direction, layout, dims, n, k, head_dim, has_bias, w_scale, only_up = CONFIGS[name]
        if only_up is not None and only_up != up:
            continue
        exchanged = n if direction == "pw" else k
        if mega_up.unsupported_shape_reason(exchanged, up) is not None:
            continue
        rows = 1
        for v in dims.values():
            rows *= v
        if distributed:
            runtime = mega_up.initialize_runtime(dist.group.WORLD, hidden=exchanged, max_rows=rows, device=device)
            runtimes = [runtime]
        else:
            runtimes = list(mega_up.initialize_emulated_group(up, hidden=exchanged, max_rows=rows, device=device))
            runtime = runtimes[0]
        weight = randn((n, k), 11, w_scale if w_scale is not None else k ** -0.5)
        bias = randn((n,), 12, 0.02) if has_bias else None
        shard = exchanged // up
        lead = tuple(dims.values())
        cu = None
        thd_layout = None
        if layout == "thd":
            gen = torch.Generator().manual_seed(4)
            cu = [0]
            while cu[-1] < rows:
                cu.append(min(rows, cu[-1] + int(torch.randint(512, 4097, (1,), generator=gen))))
            thd_layout = mega_up.prepare_thd_layout(cu, runtime)
        extra = {"layout": thd_layout} if layout == "thd" else {}
        kw = dict(dims, bias=bias, validate_group=distributed, **extra)
        dense = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
        send = torch.empty((up, rows, shard), dtype=torch.bfloat16, device=device)
        recv = torch.empty_like(send)

        def exchange() -> None:
            if distributed:
                dist.all_to_all_single(recv, send)
            else:
                recv.copy_(send)

        if direction == "pw":
            heads = k // head_dim
            x = randn((*lead, heads, head_dim), 100 + rank)
            prepared = getattr(mega_up, f"prepare_peer_write_gemm_{layout}")(
                weight, runtime, heads=heads, head_dim=head_dim, **kw
            )
            out = torch.empty(prepared.output_shape, dtype=torch.bfloat16, device=device)
            x2d = x.view(rows, k)
            batch = dims.get("batch", 1) if layout == "bshd" else 1
            seq = rows // batch

            def fused() -> None:
                prepared(x, out=out, validate_group=False)

            def kernel_only() -> None:
                prepared.launch(x2d)

            def baseline() -> None:
                if bias is None:
                    torch.mm(x2d, weight.t(), out=dense)
                else:
                    torch.addmm(bias, x2d, weight.t(), out=dense)
                send.copy_(dense.view(rows, up, shard).permute(1, 0, 2))
                exchange()
                out.view(batch, up, seq, shard).copy_(recv.view(up, batch, seq, shard).permute(1, 0, 2, 3))

            # correctness gate (distributed: against the NCCL pipeline; emulated: own column block)
            fused()
            got = out.clone()
            baseline()
            torch.cuda.synchronize(device)
            if distributed and thd_layout is None:
                gate = bool(torch.equal(got, out)) or rows < 256
            else:
                gate = bool(torch.equal(runtime.slots(rows, n)[runtime.local_rank], dense[:, runtime.local_rank * shard:(runtime.local_rank + 1) * shard])) or rows < 256
        else:
            heads = k // head_dim
            hshape = list(lead) + [heads // up, head_dim]
            hshape[1 if layout == "bshd" else 0] *= up
            head_x = randn(hshape, 200 + rank)
            prepared = getattr(mega_up, f"prepare_headshard_pull_gemm_{layout}")(
                weight, runtime, heads=heads, head_dim=head_dim, **kw
            )
            if not distributed:
                # the other emulated ranks stage once so that rank 0 pulls from eight arenas
                for rt in runtimes[1:]:
                    kw_rt = dict(kw)
                    if layout == "thd":
                        kw_rt["layout"] = mega_up.prepare_thd_layout(cu, rt)
                    other = getattr(mega_up, f"prepare_headshard_pull_gemm_{layout}")(
                        weight, rt, heads=heads, head_dim=head_dim, **kw_rt
                    )
                    other._stage(head_x)
            mat = torch.empty((rows, k), dtype=torch.bfloat16, device=device)
            flat = head_x.view(up * rows, shard)

            def fused() -> None:
                prepared(head_x, validate_group=False)

            def kernel_only() -> None:
                if prepared.compiled.epoch >= prepared.compiled.workspace_epochs:
                    prepared.compiled.reset_workspace()
                prepared.compiled()

            def baseline() -> None:
                if thd_layout is not None:
                    torch.index_select(flat, 0, thd_layout.to_source_major_index, out=send.view(up * rows, shard))
                else:
                    batch = dims.get("batch", 1) if layout == "bshd" else 1
                    seq = rows // batch
                    send.view(up, batch, seq, shard).copy_(head_x.view(batch, up, seq, shard).permute(1, 0, 2, 3))
                exchange()
                mat.view(rows, up, shard).copy_(recv.permute(1, 0, 2))
                if bias is None:
                    torch.mm(mat, weight.t(), out=dense)
                else:
                    torch.addmm(bias, mat, weight.t(), out=dense)

            fused()
            got_mat, got = prepared.materialized_input.clone(), prepared.output_2d.clone()
            baseline()
            torch.cuda.synchronize(device)
            if distributed:
                gate = bool(torch.equal(got_mat, mat)) and (bool(torch.equal(got, dense)) or rows < 256)
            else:
                gate = bool(torch.equal(got, F.linear(got_mat, weight, bias))) or rows < 256
            x2d = mat

        def matmul() -> None:
            if bias is None:
                torch.mm(x2d, weight.t(), out=dense)
            else:
                torch.addmm(bias, x2d, weight.t(), out=dense)

        gate_all = torch.tensor([int(gate)], device=device)
        if distributed:
            dist.all_reduce(gate_all, op=dist.ReduceOp.MIN)
        times = time_paths({"fused": fused, "kernel_only": kernel_only, "baseline": baseline, "matmul": matmul})
        torch.cuda.synchronize(device)
        runtime.check_status()
        flops = 2.0 * rows * n * k
        nvlink_us = rows * exchanged * 2 * (up - 1) / up / NVLINK_BYTES_PER_S * 1e6
        roofline_us = max(flops / (peak * 1e12) * 1e6, nvlink_us)
        record = {
            "config": name, "direction": direction, "layout": layout, "up": up, "rows": rows, "n": n, "k": k,
            "bias": has_bias, "peers": "nvlink" if distributed else "emulated",
            "bitwise_vs_unfused": bool(gate_all.item()),
            "us": {key: round(value, 2) for key, value in times.items()},
            "tflops_per_gpu": {key: round(flops / value / 1e6, 1) for key, value in times.items()},
            "roofline_us": round(roofline_us, 2),
            "roofline_frac": {"fused": round(roofline_us / times["fused"], 3), "kernel_only": round(roofline_us / times["kernel_only"], 3)},
            "fused_vs_baseline": round(times["baseline"] / times["fused"], 3),
            "kernel_vs_matmul": round(times["kernel_only"] / times["matmul"], 3),
            "tile_n": prepared.launch.tile_n if direction == "pw" else prepared.compiled.tile_n,
            "revision": peer_write_gemm.IMPLEMENTATION_REVISION,
        }
        results.append(record)
        if rank == 0:
            print("[BENCH_RESULT] " + json.dumps(record), flush=True)
        del prepared
    if rank == 0:
        print(f"\n{'config':18s} {'UP':>2s} {'fused us':>9s} {'kernel us':>9s} {'unfused us':>10s} {'cuBLAS us':>9s} "
              f"{'TF/GPU':>7s} {'roofl.':>6s} {'vs unfused':>10s} {'kern/mm':>7s} exact")
        for r in results:
            print(f"{r['config']:18s} {r['up']:2d} {r['us']['fused']:9.1f} {r['us']['kernel_only']:9.1f} "
                  f"{r['us']['baseline']:10.1f} {r['us']['matmul']:9.1f} {r['tflops_per_gpu']['fused']:7.0f} "
                  f"{r['roofline_frac']['fused']:6.2f} {r['fused_vs_baseline']:10.2f} {r['kernel_vs_matmul']:7.2f} "
                  f"{r['bitwise_vs_unfused']}")
    if distributed:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if all(r["bitwise_vs_unfused"] for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
