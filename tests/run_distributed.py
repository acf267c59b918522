"""torchrun runner: the fused operators over REAL peer memory (one process per GPU)
against the unfused torch path on the same GPUs - cuBLAS ``F.linear`` + permute
+ NCCL ``all_to_all_single`` - plus the collective-rejection checks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node U --master-addr 127.0.0.1 \
        --master-port 29533 tests/run_distributed.py [--full]

Rank 0 prints one ``[CORRECTNESS_RESULT] {json}`` line; every rank exits non-zero
on a mismatch. NCCL carries only the baseline's exchange and host metadata.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

import megaup_b200 as mega_up  # noqa: E402

sys.path.insert(0, str(ROOT / "tests"))
from _gpu_harness import ulp_distance  # noqa: E402


def a2a(send: torch.Tensor) -> torch.Tensor:
    send = send.contiguous()
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send)
    return received


def regroup_thd(source_major, cu):
    up = source_major.shape[0]
    return torch.cat([source_major[r, a:b] for a, b in zip(cu, cu[1:]) for r in range(up)], dim=0)


def split_thd(flat, cu, up):
    tokens = cu[-1]
    send = torch.empty((up, tokens, flat.shape[1]), dtype=flat.dtype, device=flat.device)
    for a, b in zip(cu, cu[1:]):
        for d in range(up):
            begin = up * a + d * (b - a)
            send[d, a:b] = flat[begin : begin + (b - a)]
    return send


def baseline_peer_write(kind, x, w, b, up, cu):
    """linear + permute + all_to_all_single (+ slice regroup for THD layouts)."""

    k = w.shape[1]
    rows = x.numel() // k
    dense = F.linear(x.reshape(rows, k), w, b)
    shard = w.shape[0] // up
    if kind == "bshd":
        batch, seq = x.shape[0], x.shape[1]
        send = dense.view(batch, seq, up, shard).permute(2, 0, 1, 3)
        return a2a(send).permute(1, 0, 2, 3).reshape(batch, up * seq, shard).contiguous()
    received = a2a(dense.view(rows, up, shard).permute(1, 0, 2))
    if kind == "thd" and cu is not None:
        return regroup_thd(received, cu)
    return received.reshape(up * rows, shard)


def baseline_pull(kind, head_x, w, b, up, cu):
    """all_to_all_single + permute + linear; returns (dense input, output)."""

    k = w.shape[1]
    shard = k // up
    if kind == "bshd":
        batch, gseq = head_x.shape[0], head_x.shape[1]
        seq = gseq // up
        received = a2a(head_x.reshape(batch, up, seq, shard).permute(1, 0, 2, 3))
        mat = received.permute(1, 2, 0, 3).reshape(batch * seq, k).contiguous()
    else:
        flat = head_x.reshape(-1, shard)
        rows = flat.shape[0] // up
        send = split_thd(flat, cu, up) if (kind == "thd" and cu is not None) else flat.view(up, rows, shard)
        mat = a2a(send).permute(1, 0, 2).reshape(rows, k).contiguous()
    return mat, F.linear(mat, w, b)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--full", action="store_true", help="also run the Wan2.1-14B-shaped configuration")
    parser.add_argument(
        "--stress", type=int, default=0,
        help="with --full: this many extra back-to-back peer-write + pull rounds on fresh inputs, every result checked",
    )
    args = parser.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    group = dist.group.WORLD
    up = world
    failures: list[str] = []
    report: dict[str, object] = {"up": up, "cases": {}}

    def randn(shape, seed, scale=1.0):
        gen = torch.Generator(device=device).manual_seed(seed)
        return (torch.randn(shape, device=device, generator=gen) * scale).to(torch.bfloat16)

    def check(name, got, want, exact=True):
        """Bit-exact, or (where cuBLAS splits K for a small M) within 1 BF16 ulp; on all ranks."""

        same = torch.equal(got.reshape(want.shape), want)
        ulps = 0.0 if same else max(ulp_distance(got.reshape(want.shape), want), 1e-3)
        worst = torch.tensor([ulps], device=device, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        report["cases"][name] = {"bitwise": float(worst[0]) == 0.0, "max_ulp": round(float(worst[0]), 3)}
        if float(worst[0]) > (0.0 if exact else 1.0):
            failures.append(name)

    heads, dim = 8 * up // 2, 128  # hidden = heads * 128: shards of 4*128 = 512 columns
    hidden = heads * dim
    runtime = mega_up.initialize_runtime(group, hidden=hidden, max_rows=256, device=device)
    again = mega_up.initialize_runtime(group, hidden=hidden, max_rows=256, device=device)
    if again is not runtime:
        failures.append("one runtime per (group, hidden)")
    w = randn((hidden, hidden), 1, hidden ** -0.5)
    b = randn((hidden,), 2, 0.02)

    shapes = {
        "bshd": [(1, 64), (2, 17)],
        "sbhd": [(64, 2), (17, 3)],
        "thd": [(33, None), (31, None), (17, (0, 5, 5, 12, 17)), (16, (0, 1, 16))],
    }
    for kind, cases in shapes.items():
        for lead in cases:
            cu = lead[1] if kind == "thd" else None
            lead_dims = (lead[0],) if kind == "thd" else lead
            rows = 1
            for v in lead_dims:
                rows *= v
            layout = mega_up.prepare_thd_layout(cu, runtime) if cu is not None else None
            tag = f"{kind}{lead_dims}{'+layout' if cu else ''}"
            extra = {"layout": layout} if kind == "thd" else {}
            # ---- peer-write: one-shot, then prepared on two inputs
            x = randn((*lead_dims, heads, dim), 100 + rank)
            one_shot = getattr(mega_up, f"peer_write_gemm_{kind}")(x, w, runtime, bias=b, **extra)
            check(f"pw one-shot {tag}", one_shot, baseline_peer_write(kind, x, w, b, up, cu), exact=rows >= 256)
            names = ("batch", "sequence") if kind == "bshd" else ("sequence", "batch") if kind == "sbhd" else ("tokens",)
            dims = dict(zip(names, lead_dims), heads=heads, head_dim=dim)
            prepared = getattr(mega_up, f"prepare_peer_write_gemm_{kind}")(w, runtime, bias=b, **dims, **extra)
            for trial in range(2):
                x = randn((*lead_dims, heads, dim), 200 + 10 * trial + rank)
                got = prepared(x, validate_group=(trial == 0))
                check(f"pw prepared {tag} #{trial}", got, baseline_peer_write(kind, x, w, b, up, cu), exact=rows >= 256)
            # ---- pull: prepared, three calls on alternating streams with a workspace recycle
            seq_axis = 1 if kind == "bshd" else 0
            hshape = list(lead_dims) + [heads // up, dim]
            hshape[seq_axis] *= up
            pull = getattr(mega_up, f"prepare_headshard_pull_gemm_{kind}")(
                w, runtime, bias=b, workspace_epochs=2, **dims, **extra
            )
            streams = [torch.cuda.Stream(device), torch.cuda.Stream(device)]
            for trial in range(3):
                hx = randn(hshape, 400 + 10 * trial + rank)
                torch.cuda.synchronize(device)
                with torch.cuda.stream(streams[trial % 2]):
                    out = pull(hx, validate_group=(trial == 0))
                torch.cuda.synchronize(device)
                mat, want = baseline_pull(kind, hx, w, b, up, cu)
                check(f"pull input {tag} #{trial}", pull.materialized_input, mat)
                check(f"pull output {tag} #{trial}", out, want, exact=rows >= 256)
            hx = randn(hshape, 500 + rank)
            out = getattr(mega_up, f"headshard_pull_gemm_{kind}")(hx, w, runtime, bias=b, **extra)
            mat, want = baseline_pull(kind, hx, w, b, up, cu)
            check(f"pull one-shot {tag}", out, want, exact=rows >= 256)
            torch.cuda.synchronize(device)
            runtime.check_status()

    # ---- collective rejection: a rank-local fault raises ValueError on EVERY rank
    def expect(name, error_type, fn):
        try:
            fn()
        except error_type:
            raised = 1
        except Exception as error:  # noqa: BLE001
            raised = 0
            report.setdefault("unexpected", []).append(f"{name}: {type(error).__name__}: {error}")
        else:
            raised = 0
        flag = torch.tensor([raised], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if not int(flag[0]):
            failures.append(f"rejection: {name}")

    good = randn((1, 64, heads, dim), 600 + rank)
    bad_dtype = good.float() if rank == 0 else good
    expect("rank-local dtype", ValueError, lambda: mega_up.peer_write_gemm_bshd(bad_dtype, w, runtime, bias=b))
    bad_shape = good[:, :32].contiguous() if rank == 0 else good
    expect("rank-local shape", ValueError, lambda: mega_up.peer_write_gemm_bshd(bad_shape, w, runtime, bias=b))
    bad_bias = b[: hidden // 2].contiguous() if rank == 0 else b
    expect("rank-local bias", ValueError, lambda: mega_up.peer_write_gemm_bshd(good, w, runtime, bias=bad_bias))
    transposed = randn((hidden, 2 * hidden), 7).t()[:, :hidden]
    expect("transposed weight", ValueError, lambda: mega_up.peer_write_gemm_bshd(good, transposed, runtime))
    expect(
        "hidden mismatch",
        ValueError,
        lambda: mega_up.initialize_runtime(group, hidden=hidden if rank else 2 * hidden, max_rows=256, device=device),
    )
    expect(
        "changed max_rows", RuntimeError,
        lambda: mega_up.initialize_runtime(group, hidden=hidden, max_rows=512, device=device),
    )
    expect(
        "invalid ordinal on rank 0", ValueError,
        lambda: mega_up.initialize_runtime(group, hidden=2 * hidden, max_rows=64, device=f"cuda:{97 if rank == 0 else local_rank}"),
    )
    cu_a, cu_b = (0, 5, 17), (0, 6, 17)
    layout = mega_up.prepare_thd_layout(cu_a if rank else cu_b, runtime)
    x17 = randn((17, heads, dim), 700 + rank)
    expect("THD fingerprint mismatch", ValueError, lambda: mega_up.peer_write_gemm_thd(x17, w, runtime, layout=layout))
    # the runtime still works after the rejected calls
    x = randn((1, 64, heads, dim), 800 + rank)
    check("pw after rejections", mega_up.peer_write_gemm_bshd(x, w, runtime, bias=b), baseline_peer_write("bshd", x, w, b, up, None), exact=False)

    # ---- a peer that does not show up: the bounded flag wait runs out, the host raises,
    # the context survives, and the group realigns once the late rank arrives
    torch.cuda.synchronize(device)
    dist.barrier()
    if rank == 0:
        runtime.barrier(timeout_s=0.05)
        torch.cuda.synchronize(device)
        try:
            runtime.check_status()
            failures.append("flag timeout was not reported")
        except RuntimeError as error:
            if "slot hand-off flag" not in str(error):
                failures.append(f"unexpected timeout message: {error}")
    dist.barrier()  # host-side: the late ranks arrive only after rank 0 has given up
    if rank != 0:
        runtime.barrier()
    torch.cuda.synchronize(device)
    runtime.check_status()
    x = randn((1, 64, heads, dim), 850 + rank)
    check("pw after a timed-out hand-off", mega_up.peer_write_gemm_bshd(x, w, runtime, bias=b), baseline_peer_write("bshd", x, w, b, up, None), exact=False)

    # ---- a second runtime with another hidden has its own arena
    other = mega_up.initialize_runtime(group, hidden=2 * hidden, max_rows=64, device=device)
    if other is runtime or other.arena.data_ptr() == runtime.arena.data_ptr():
        failures.append("distinct arenas per hidden")

    if args.full:
        tokens, big, big_heads = 4096, 5120, 40
        big_rt = mega_up.initialize_runtime(group, hidden=big, max_rows=tokens, device=device)
        wq, bq = randn((big, big), 11, big ** -0.5), randn((big,), 12, 0.02)
        x = randn((1, tokens, big_heads, 128), 900 + rank)
        got = mega_up.peer_write_gemm_bshd(x, wq, big_rt, bias=bq)
        check("pw Wan2.1-14B Q", got, baseline_peer_write("bshd", x, wq, bq, up, None))
        hx = randn((1, up * tokens, big_heads // up, 128), 950 + rank)
        pull = mega_up.prepare_headshard_pull_gemm_bshd(wq, big_rt, batch=1, sequence=tokens, heads=big_heads, head_dim=128, bias=bq)
        out = pull(hx)
        mat, want = baseline_pull("bshd", hx, wq, bq, up, None)
        check("pull Wan2.1-14B O input", pull.materialized_input, mat)
        check("pull Wan2.1-14B O", out, want)
        torch.cuda.synchronize(device)
        big_rt.check_status()
        # back-to-back rounds on fresh inputs: the slots are reused immediately, so a
        # hand-off that lets a rank run ahead would show up as stale or torn rows
        if args.stress:
            writer = mega_up.prepare_peer_write_gemm_bshd(
                wq, big_rt, batch=1, sequence=tokens, heads=big_heads, head_dim=128, bias=bq
            )
            bad_rounds = 0
            for round_index in range(args.stress):
                x = randn((1, tokens, big_heads, 128), 2000 + 16 * round_index + rank)
                hx = randn((1, up * tokens, big_heads // up, 128), 6000 + 16 * round_index + rank)
                got_pw = writer(x, validate_group=False)
                got_pull = pull(hx, validate_group=False).clone()
                got_mat = pull.materialized_input.clone()
                want_pw = baseline_peer_write("bshd", x, wq, bq, up, None)
                mat, want_pull = baseline_pull("bshd", hx, wq, bq, up, None)
                same = (
                    torch.equal(got_pw.reshape(want_pw.shape), want_pw)
                    and torch.equal(got_mat, mat)
                    and torch.equal(got_pull.reshape(want_pull.shape), want_pull)
                )
                bad_rounds += 0 if same else 1
            worst = torch.tensor([bad_rounds], device=device)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            report["stress"] = {"rounds": args.stress, "bad_rounds": int(worst[0])}
            if int(worst[0]):
                failures.append("stress rounds")
            torch.cuda.synchronize(device)
            big_rt.check_status()

    torch.cuda.synchronize(device)
    report["failures"] = failures
    report["passed"] = not failures
    if rank == 0:
        print("[CORRECTNESS_RESULT] " + json.dumps(report), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == "__main__":
    main()
