"""Where the time of one fused operation goes on real peers: CUDA events between the
launches of a peer-write call (GEMM with routed stores | copy-out of the slots)
and of a pull call (staging copy | pull + GEMM), on the Wan2.1-14B-shaped
projection, next to the kernels timed alone and the whole call.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node U --master-addr 127.0.0.1 \
        --master-port 29545 -m megaup_b200.handoff_profile [--iters 30]

Run it once per hand-off protocol (``MEGA_UP_HANDOFF=lazy``, the default: one
barrier kernel per operation, the second hand-off signalled from the tail of
the operation's last kernel; ``folded``: both inside the kernels; ``barriers``:
two stand-alone barrier kernels per operation; barrier kernels show up inside
the segment of the launch they precede). The
report ends with the pull kernel's own trace words over real peers (first panel
gate of every CTA, first ticket stored, all rows pulled). An
event between two launches takes away their programmatic overlap, so the
segments add up to a little more than the call timed as a whole; the
difference is printed. Every figure is the maximum over the ranks of the
rank's median. Rank 0 prints one ``[HANDOFF_PROFILE] {json}`` line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

import megaup_b200 as mega_up
from megaup_b200 import _native

HIDDEN, HEADS, HEAD_DIM, TOKENS = 5120, 40, 128, 4096


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--iters", type=int, default=30)
    args = parser.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    up = world
    runtime = mega_up.initialize_runtime(dist.group.WORLD, hidden=HIDDEN, max_rows=TOKENS, device=device)
    gen = torch.Generator(device=device).manual_seed(99 + rank)

    def randn(shape, scale=1.0):
        return (torch.randn(shape, device=device, generator=gen) * scale).to(torch.bfloat16)

    w, b = randn((HIDDEN, HIDDEN), HIDDEN ** -0.5), randn((HIDDEN,), 0.02)
    x = randn((1, TOKENS, HEADS, HEAD_DIM))
    hx = randn((1, up * TOKENS, HEADS // up, HEAD_DIM))
    out = torch.empty((1, up * TOKENS, HEADS // up, HEAD_DIM), dtype=torch.bfloat16, device=device)
    kw = dict(batch=1, sequence=TOKENS, heads=HEADS, head_dim=HEAD_DIM, bias=b)
    writer = mega_up.prepare_peer_write_gemm_bshd(w, runtime, **kw)
    puller = mega_up.prepare_headshard_pull_gemm_bshd(w, runtime, **kw)
    events = [torch.cuda.Event(enable_timing=True) for _ in range(2)]

    def sync_all() -> None:
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)

    def reduce_max(values: list[float]) -> list[float]:
        t = torch.tensor(values, dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def median_us(samples: list[list[float]]) -> list[float]:
        return reduce_max([statistics.median(column) for column in zip(*samples)])

    def whole(call) -> float:
        for _ in range(3):
            call()
        sync_all()
        events[0].record()
        for _ in range(args.iters):
            call()
        events[1].record()
        sync_all()
        return reduce_max([events[0].elapsed_time(events[1]) * 1e3 / args.iters])[0]

    def segments(first, second) -> list[float]:
        """[first launch, second launch] of one operation, an event in between; the
        calls are enqueued back to back (as in the whole-call timing) and the
        events read afterwards."""

        total = args.iters + 3
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(total)]
        sync_all()
        for it in range(total):
            with torch.no_grad(), runtime.lease():
                marks[it][0].record()
                first()
                marks[it][1].record()
                second()
                marks[it][2].record()
        sync_all()
        samples = [
            [m[0].elapsed_time(m[1]) * 1e3, m[1].elapsed_time(m[2]) * 1e3] for m in marks[3:]
        ]
        return median_us(samples)

    x2d = x.view(TOKENS, HIDDEN)
    report: dict[str, object] = {
        "up": up,
        "handoff": runtime.handoff,
    }
    report["peer_write_call_us"] = whole(lambda: writer(x, out=out, validate_group=False))
    report["pull_call_us"] = whole(lambda: puller(hx, validate_group=False))
    report["peer_write_kernel_alone_us"] = whole(lambda: writer.launch(x2d))

    def pull_alone() -> None:
        if puller.compiled.epoch >= puller.compiled.workspace_epochs:
            puller.compiled.reset_workspace()
        puller.compiled()

    report["pull_kernel_alone_us"] = whole(pull_alone)
    sync_all()
    gemm_us, copy_out_us = segments(lambda: writer._launch(x), lambda: writer._materialize(out))
    stage_us, pull_us = segments(lambda: (puller._refresh_workspace(), puller._stage(hx)), puller._launch)
    report["peer_write_segments_us"] = {"gemm_with_routed_stores": gemm_us, "copy_out_with_its_waits": copy_out_us}
    report["pull_segments_us"] = {"staging_copy_with_its_waits": stage_us, "pull_gemm_with_its_waits": pull_us}
    report["event_overhead_us"] = {
        "peer_write": gemm_us + copy_out_us - report["peer_write_call_us"],
        "pull": stage_us + pull_us - report["pull_call_us"],
    }
    report["call_minus_kernel_us"] = {
        "peer_write": report["peer_write_call_us"] - report["peer_write_kernel_alone_us"],
        "pull": report["pull_call_us"] - report["pull_kernel_alone_us"],
    }
    # ---- every launch of the reference's two-barrier protocol on its own (GEMM | barrier | copy |
    # barrier and copy | barrier | GEMM | barrier), whatever protocol the runtime itself uses: what
    # a barrier kernel and a copy cost on this box next to the GEMMs
    def launches(steps) -> list[float]:
        total = args.iters + 3
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(steps) + 1)] for _ in range(total)]
        sync_all()
        for it in range(total):
            with torch.no_grad(), runtime.lease():
                marks[it][0].record()
                for index, step in enumerate(steps):
                    step()
                    marks[it][index + 1].record()
        sync_all()
        samples = [[m[i].elapsed_time(m[i + 1]) * 1e3 for i in range(len(steps))] for m in marks[3:]]
        return median_us(samples)

    shard = HIDDEN // up
    slots = runtime.slots(TOKENS, HIDDEN)
    stream = lambda: runtime._stream()  # noqa: E731

    def copy_out() -> None:
        _native.call("mup_gather_rows", out.data_ptr(), slots.data_ptr(), None, up * TOKENS, shard, stream())

    def stage() -> None:
        _native.call("mup_gather_rows", slots.data_ptr(), hx.data_ptr(), None, up * TOKENS, shard, stream())

    names = ("gemm", "barrier_written", "copy_out", "barrier_reusable")
    report["peer_write_launches_two_barrier_protocol_us"] = dict(
        zip(names, launches([lambda: writer.launch(x2d, stream_handle=stream()), runtime.barrier, copy_out, runtime.barrier]))
    )
    names = ("staging_copy", "barrier_staged", "pull_gemm", "barrier_reusable")

    def pull_launch() -> None:
        if puller.compiled.epoch >= puller.compiled.workspace_epochs:
            puller.compiled.reset_workspace()
        puller.compiled(stream_handle=stream())

    report["pull_launches_two_barrier_protocol_us"] = dict(
        zip(names, launches([stage, runtime.barrier, pull_launch, runtime.barrier]))
    )

    # ---- the pull kernel's own trace words over real peers (per CTA; see mup_pull_plan_set_trace)
    sync_all()
    trace = torch.zeros((puller.compiled.grid_ctas, 16), dtype=torch.int64, device=device)
    _native.call("mup_pull_plan_set_trace", puller.compiled._plan, trace.data_ptr())
    gates, stored, done, kernel = [], [], [], []
    for _ in range(4):
        trace.zero_()
        sync_all()
        puller(hx, validate_group=False)
        torch.cuda.synchronize(device)
        t = trace.cpu().double()
        first_gate = t[:, 10][t[:, 10] > 0] / 1e3
        gates.append([float(first_gate.min()), float(first_gate.mean()), float(first_gate.max())])
        stored.append(float(t[:, 13][t[:, 13] > 0].mean()) / 1e3)
        done.append(float(t[:, 8].max() - t[:, 6].min()) / 1e3)
        kernel.append(float(t[:, 7].max() - t[:, 6].min()) / 1e3)
    _native.call("mup_pull_plan_set_trace", puller.compiled._plan, None)
    gate_min, gate_mean, gate_max = median_us(gates)
    report["pull_kernel_trace"] = {
        "first_gate_open_us_min_mean_max": [gate_min, gate_mean, gate_max],
        "first_ticket_stored_us": reduce_max([statistics.median(stored)])[0],
        "all_rows_pulled_us": reduce_max([statistics.median(done)])[0],
        "kernel_us": reduce_max([statistics.median(kernel)])[0],
    }
    torch.cuda.synchronize(device)
    runtime.check_status()
    if rank == 0:
        print("[HANDOFF_PROFILE] " + json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
