"""Measure the peer-memory path the fused operators use, with the library's own
kernels over the runtime's peer-mapped arenas (no NCCL on the data path):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29544 -m megaup_b200.nvlink_probe [--mib 512]

* peer-load and peer-store bandwidth of a plain 16-byte-vector copy kernel
  (``mup_gather_rows``), one direction (rank 0 alone) and all ranks at once
  (every rank reads from / writes to its right-hand neighbour);
* round-trip time of dependent 8-byte loads from a peer (``mup_probe_load_latency``)
  next to the same loads from local memory.

Rank 0 prints one ``[NVLINK_PROBE] {json}`` line. The reference measures
nothing of the kind; its README quotes the 900 GB/s NVLink 5 figure.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from . import _native
from .runtime import initialize_runtime


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--mib", type=int, default=512, help="bytes moved per copy, in MiB")
    parser.add_argument("--iters", type=int, default=10)
    args = parser.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    hidden = 4096
    rows = args.mib * (1 << 20) // (hidden * 2)
    runtime = initialize_runtime(dist.group.WORLD, hidden=hidden, max_rows=rows, device=device)
    neighbour = runtime.peer_buffers[(rank + 1) % world]
    local = torch.zeros(rows * hidden, dtype=torch.bfloat16, device=device)
    nbytes = rows * hidden * 2
    stream = torch.cuda.current_stream(device).cuda_stream
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def copy(dst: torch.Tensor, src: torch.Tensor) -> None:
        _native.call("mup_gather_rows", dst.data_ptr(), src.data_ptr(), None, rows, hidden, stream)

    def timed_gbs(dst: torch.Tensor, src: torch.Tensor, active: bool) -> float:
        """GB/s of this rank's copies (0 when it sits the test out); all ranks start together."""

        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        if not active:
            dist.barrier()
            return 0.0
        for _ in range(2):
            copy(dst, src)
        start.record()
        for _ in range(args.iters):
            copy(dst, src)
        stop.record()
        torch.cuda.synchronize(device)
        dist.barrier()
        return nbytes * args.iters / (start.elapsed_time(stop) * 1e-3) / 1e9

    def reduce(value: float, op) -> float:
        t = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=op)
        return float(t.item())

    results: dict[str, object] = {"up": world, "mib_per_copy": args.mib}
    results["local_copy_gbs_read_plus_write"] = 2 * reduce(timed_gbs(local, runtime.arena.view(-1), True), dist.ReduceOp.MIN)
    results["peer_load_one_direction_gbs"] = reduce(timed_gbs(local, neighbour.view(-1), rank == 0), dist.ReduceOp.MAX)
    results["peer_store_one_direction_gbs"] = reduce(timed_gbs(neighbour.view(-1), local, rank == 0), dist.ReduceOp.MAX)
    results["peer_load_all_ranks_gbs_min"] = reduce(timed_gbs(local, neighbour.view(-1), True), dist.ReduceOp.MIN)
    results["peer_store_all_ranks_gbs_min"] = reduce(timed_gbs(neighbour.view(-1), local, True), dist.ReduceOp.MIN)

    # dependent-load round trips (the arena's first bytes are zeroed for the chase)
    out_ns = torch.zeros(1, dtype=torch.int64, device=device)
    runtime.arena.view(-1)[:4096].zero_()
    torch.cuda.synchronize(device)
    dist.barrier()
    chase = 2000
    for name, target in (("local", runtime.arena), ("peer", neighbour)):
        _native.call("mup_probe_load_latency", target.data_ptr(), chase, out_ns.data_ptr(), stream)
        torch.cuda.synchronize(device)
        results[f"{name}_load_round_trip_ns"] = reduce(float(out_ns.item()) / chase, dist.ReduceOp.MAX)
    torch.cuda.synchronize(device)
    runtime.check_status()
    if rank == 0:
        print("[NVLINK_PROBE] " + json.dumps(results), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
