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
from _gpu_harness import representation_ulps, ulp_distance  # noqa: E402


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
    parser.add_argument("--no-matrix", action="store_true", help="skip the reference's (heads, UP, bias) shape matrix")
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
        true_ulps = 0 if same else representation_ulps(got.reshape(want.shape), want)
        worst = torch.tensor([ulps, float(true_ulps)], device=device, dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        # max_ulp: in units of the BF16 ulp at max(|a|, |b|, 2^-6), the pass/fail measure (an output
        # that cancels to almost zero carries an absolute FP32 error); max_true_ulp: representable
        # BF16 values between the two results, no floor
        report["cases"][name] = {
            "bitwise": float(worst[0]) == 0.0, "max_ulp": round(float(worst[0]), 3), "max_true_ulp": int(worst[1]),
        }
        if float(worst[0]) > (0.0 if exact else 1.0):
            failures.append(name)

    def layout_suite(label, peer_rt, pull_rt, w_pw, b_pw, w_pull, b_pull, in_heads, pull_in_heads, dim):
        """Every layout of both operators on one pair of projections: peer-write
        x[..., in_heads, dim] @ w_pw^T, pull head_x[..., pull_in_heads / up, dim] @ w_pull^T."""

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
                tag = f"{label}{kind}{lead_dims}{'+layout' if cu else ''}"
                names = ("batch", "sequence") if kind == "bshd" else ("sequence", "batch") if kind == "sbhd" else ("tokens",)
                # ---- peer-write: one-shot, then prepared on two inputs
                layout = mega_up.prepare_thd_layout(cu, peer_rt) if cu is not None else None
                extra = {"layout": layout} if kind == "thd" else {}
                x = randn((*lead_dims, in_heads, dim), 100 + rank)
                one_shot = getattr(mega_up, f"peer_write_gemm_{kind}")(x, w_pw, peer_rt, bias=b_pw, **extra)
                check(f"pw one-shot {tag}", one_shot, baseline_peer_write(kind, x, w_pw, b_pw, up, cu), exact=rows >= 256)
                dims = dict(zip(names, lead_dims), heads=in_heads, head_dim=dim)
                prepared = getattr(mega_up, f"prepare_peer_write_gemm_{kind}")(w_pw, peer_rt, bias=b_pw, **dims, **extra)
                for trial in range(2):
                    x = randn((*lead_dims, in_heads, dim), 200 + 10 * trial + rank)
                    got = prepared(x, validate_group=(trial == 0))
                    check(f"pw prepared {tag} #{trial}", got, baseline_peer_write(kind, x, w_pw, b_pw, up, cu), exact=rows >= 256)
                # ---- pull: prepared, three calls on alternating streams with a workspace recycle
                layout = mega_up.prepare_thd_layout(cu, pull_rt) if cu is not None else None
                extra = {"layout": layout} if kind == "thd" else {}
                seq_axis = 1 if kind == "bshd" else 0
                hshape = list(lead_dims) + [pull_in_heads // up, dim]
                hshape[seq_axis] *= up
                dims = dict(zip(names, lead_dims), heads=pull_in_heads, head_dim=dim)
                pull = getattr(mega_up, f"prepare_headshard_pull_gemm_{kind}")(
                    w_pull, pull_rt, bias=b_pull, workspace_epochs=2, **dims, **extra
                )
                streams = [torch.cuda.Stream(device), torch.cuda.Stream(device)]
                for trial in range(3):
                    hx = randn(hshape, 400 + 10 * trial + rank)
                    torch.cuda.synchronize(device)
                    with torch.cuda.stream(streams[trial % 2]):
                        out = pull(hx, validate_group=(trial == 0))
                    torch.cuda.synchronize(device)
                    mat, want = baseline_pull(kind, hx, w_pull, b_pull, up, cu)
                    check(f"pull input {tag} #{trial}", pull.materialized_input, mat)
                    check(f"pull output {tag} #{trial}", out, want, exact=rows >= 256)
                hx = randn(hshape, 500 + rank)
                out = getattr(mega_up, f"headshard_pull_gemm_{kind}")(hx, w_pull, pull_rt, bias=b_pull, **extra)
                mat, want = baseline_pull(kind, hx, w_pull, b_pull, up, cu)
                check(f"pull one-shot {tag}", out, want, exact=rows >= 256)
                torch.cuda.synchronize(device)
                peer_rt.check_status()
                pull_rt.check_status()

    # One runtime per exchanged width for the whole run; the widths the --full
    # configurations use get their capacity from the start.
    capacity = {5120: 4096, 6144: 8192, 8192: 16384, 2304: 512, 2048: 1024, 1024: 256} if args.full else {}

    def runtime_for(width):
        return mega_up.initialize_runtime(group, hidden=width, max_rows=capacity.get(width, 256), device=device)

    heads, dim = 8 * up // 2, 128  # hidden = heads * 128: shards of 4*128 = 512 columns
    hidden = heads * dim
    runtime = runtime_for(hidden)
    again = runtime_for(hidden)
    if again is not runtime:
        failures.append("one runtime per (group, hidden)")
    w = randn((hidden, hidden), 1, hidden ** -0.5)
    b = randn((hidden,), 2, 0.02)
    layout_suite("", runtime, runtime, w, b, w, b, heads, heads, dim)

    # ---- the shape matrix of the reference's multi-GPU test (tests/test_distributed.py:21-59 there):
    # six square (heads, UP, bias) projections and five rectangular ones, each tied to one UP degree
    # (input heads, peer-write output heads, pull input heads, pull output heads, head_dim, UP, bias, runtime per width)
    matrix = [
        (16, 16, 16, 16, 128, 8, False, False),   # hidden 2048: 256-column shards, two peers per 512 columns
        (40, 40, 40, 40, 128, 8, True, False),    # hidden 5120: 640-column shards straddle 256-column blocks
        (10, 10, 10, 10, 128, 2, True, False),    # hidden 1280
        (32, 32, 32, 32, 128, 4, False, False),   # hidden 4096
        (18, 18, 18, 18, 128, 2, True, False),    # hidden 2304: odd number of 256-column blocks
        (64, 64, 64, 64, 128, 2, False, False),   # hidden 8192: 4096-column shards pulled in segments
        (32, 48, 32, 32, 128, 8, True, False),    # fused GQA QKV [6144, 4096]; pull [4096, 4096]
        (16, 8, 8, 16, 128, 2, True, False),      # K/V [1024, 2048]; pull [2048, 1024]
        (16, 64, 64, 16, 128, 4, False, False),   # [8192, 2048]; pull [2048, 8192]
        (13, 32, 32, 16, 80, 2, False, False),    # [2560, 1040], K not a multiple of 64; pull [1280, 2560]
        (16, 48, 16, 48, 128, 4, True, True),     # packed QKV [6144, 2048] both ways, one runtime per exchanged width
    ]
    if not args.no_matrix:
        for index, (in_heads, peer_out, pull_in, pull_out, hd, case_up, bias_on, per_width) in enumerate(matrix):
            if case_up != up:
                continue
            peer_width, pull_width = peer_out * hd, pull_in * hd
            wide = max(peer_width, pull_width)
            peer_rt = runtime_for(peer_width if per_width else wide)
            pull_rt = runtime_for(pull_width if per_width else wide)
            if (peer_rt is pull_rt) != (peer_rt.hidden == pull_rt.hidden):
                failures.append(f"matrix {index}: one runtime per hidden")
            w_pw = randn((peer_out * hd, in_heads * hd), 31 + index, (in_heads * hd) ** -0.5)
            w_pull = randn((pull_out * hd, pull_in * hd), 61 + index, (pull_in * hd) ** -0.5)
            b_pw = randn((peer_out * hd,), 41 + index, 0.02) if bias_on else None
            b_pull = randn((pull_out * hd,), 71 + index, 0.02) if bias_on else None
            layout_suite(f"[{peer_out * hd}x{in_heads * hd}|{pull_out * hd}x{pull_in * hd}] ", peer_rt, pull_rt,
                         w_pw, b_pw, w_pull, b_pull, in_heads, pull_in, hd)
        report["matrix_cases"] = [i for i, case in enumerate(matrix) if case[5] == up]

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
        lambda: mega_up.initialize_runtime(
            group, hidden=hidden if rank else 2 * hidden, max_rows=capacity.get(hidden, 256), device=device
        ),
    )
    expect(
        "changed max_rows", RuntimeError,
        lambda: mega_up.initialize_runtime(group, hidden=hidden, max_rows=capacity.get(hidden, 256) + 1, device=device),
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
    other = runtime_for(2 * hidden)
    if other is runtime or other.arena.data_ptr() == runtime.arena.data_ptr():
        failures.append("distinct arenas per hidden")

    if args.full:
        tokens, big, big_heads = 4096, 5120, 40
        big_rt = runtime_for(big)
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

        # Llama-3-8B fused GQA QKV: peer-write, sequence-first, no bias, W[6144, 4096], 8192 tokens per rank
        rt = runtime_for(6144)
        w_qkv = randn((6144, 4096), 13, 1.0 / 64)
        x = randn((8192, 1, 32, 128), 1000 + rank)
        got = mega_up.peer_write_gemm_sbhd(x, w_qkv, rt)
        check("pw Llama-3-8B QKV sbhd", got, baseline_peer_write("sbhd", x, w_qkv, None, up, None))
        del x, got, w_qkv
        if up == 8:
            # Llama-3-70B O projection: pull, packed THD with a layout, no bias, W[8192, 8192],
            # 16384 tokens per rank in variable-length samples (512..4096 tokens, the last one cut)
            rt = runtime_for(8192)
            lengths, total = [], 0
            length_gen = torch.Generator().manual_seed(70)
            while total < 16384:
                length = int(torch.randint(512, 4097, (1,), generator=length_gen))
                length = min(length, 16384 - total)
                lengths.append(length)
                total += length
            cu = [0]
            for length in lengths:
                cu.append(cu[-1] + length)
            layout = mega_up.prepare_thd_layout(tuple(cu), rt)
            w_o = randn((8192, 8192), 14, 8192 ** -0.5)
            hx = randn((up * 16384, 64 // up, 128), 1100 + rank)
            pull70 = mega_up.prepare_headshard_pull_gemm_thd(w_o, rt, tokens=16384, heads=64, head_dim=128, layout=layout)
            out = pull70(hx)
            mat, want = baseline_pull("thd", hx, w_o, None, up, tuple(cu))
            check("pull Llama-3-70B O thd+layout input", pull70.materialized_input, mat)
            check("pull Llama-3-70B O thd+layout", out, want)
            del hx, out, mat, want, w_o, pull70
            # LTX-shaped W[2048, 2048], 32 heads of 64, 1024 tokens per rank
            rt = runtime_for(2048)
            w_l, b_l = randn((2048, 2048), 15, 2048 ** -0.5), randn((2048,), 16, 0.02)
            x = randn((1, 1024, 32, 64), 1200 + rank)
            check("pw LTX 2048 D=64", mega_up.peer_write_gemm_bshd(x, w_l, rt, bias=b_l),
                  baseline_peer_write("bshd", x, w_l, b_l, up, None))
            hx = randn((1, up * 1024, 32 // up, 64), 1250 + rank)
            out = mega_up.headshard_pull_gemm_bshd(hx, w_l, rt, bias=b_l)
            check("pull LTX 2048 D=64", out, baseline_pull("bshd", hx, w_l, b_l, up, None)[1])
            # Llama-3-8B K projection W[1024, 4096], 64 tokens per rank: cuBLAS splits K for so few rows
            rt = runtime_for(1024)
            w_k, b_k = randn((1024, 4096), 17, 1.0 / 64), randn((1024,), 18, 0.02)
            x = randn((1, 64, 32, 128), 1300 + rank)
            check("pw Llama-3-8B K proj M=64", mega_up.peer_write_gemm_bshd(x, w_k, rt, bias=b_k),
                  baseline_peer_write("bshd", x, w_k, b_k, up, None), exact=False)
        if up == 2:
            # 2304 wide (an odd number of 256-column blocks), B=4 x S=128: the strided regroup copies
            rt = runtime_for(2304)
            w_e, b_e = randn((2304, 2304), 19, 2304 ** -0.5), randn((2304,), 20, 0.02)
            x = randn((4, 128, 18, 128), 1400 + rank)
            check("pw 2304 B=4", mega_up.peer_write_gemm_bshd(x, w_e, rt, bias=b_e),
                  baseline_peer_write("bshd", x, w_e, b_e, up, None))
            hx = randn((4, up * 128, 18 // up, 128), 1450 + rank)
            out = mega_up.headshard_pull_gemm_bshd(hx, w_e, rt, bias=b_e)
            check("pull 2304 B=4", out, baseline_pull("bshd", hx, w_e, b_e, up, None)[1])
        torch.cuda.synchronize(device)
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
