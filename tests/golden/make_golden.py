"""Generate the golden fixtures in this directory by RUNNING the reference.

Needs a checkout of the reference (pass its path as the first argument); it is
imported, never copied. Outputs are small compressed files committed next to
this script. Inputs are not stored: tests regenerate them with
``golden_inputs`` below (numpy PCG64 streams, identical on every platform).

    python tests/golden/make_golden.py /path/to/reference

What is pinned:
  shape_rule.json       unsupported_shape_reason over a (width, UP) sweep
  rotation.json         peer_n_rotation tables
  thd_layouts.npz       THDLayout permutations, boundaries, fingerprints
  layout_helpers.npz    the four layout-contract helpers on arange tensors
  unfused_ws2.npz       the reference's F.linear + permute + all_to_all_single
                        baselines under gloo, world_size 2, for BSHD / SBHD /
                        THD (slab and split), integer-valued (exact) inputs and
                        one random-valued case
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

SHAPE_WIDTHS = (0, 128, 256, 384, 640, 1024, 1280, 1536, 1920, 2048, 2049, 2304, 3328, 4096, 4864, 5120, 6144, 8192)
SHAPE_UPS = (1, 2, 3, 4, 8, 16)
ROTATION_CASES = ((2048, 8), (3072, 4), (4096, 2), (5120, 8), (5120, 4), (5120, 2), (2304, 2), (6144, 8), (1024, 8))
THD_CASES = (
    ((0, 5, 5, 12, 13), 3),
    ((0, 3, 10, 11, 16), 4),
    ((0, 17), 2),
    ((0, 5, 5, 12, 17), 2),
    ((0, 1, 2, 3, 4, 33), 8),
    ((0, 0, 7, 7, 31), 4),
)

# name -> (layout, dims, up, N, K, head_dim_out, bias, integer_valued, cu)
UNFUSED_CASES = {
    "bshd_cfg1_small": ("bshd", (1, 16, 12, 128), 2, 1536, 1536, 128, True, True, None),
    "bshd_b2_s17": ("bshd", (2, 17, 8, 64), 2, 512, 512, 64, True, True, None),
    "bshd_rect_nobias": ("bshd", (1, 33, 4, 64), 2, 768, 256, 128, False, True, None),
    "sbhd_s17_b3": ("sbhd", (17, 3, 8, 64), 2, 512, 512, 64, True, True, None),
    "thd_slab_33": ("thd", (33, 8, 64), 2, 512, 512, 64, True, True, None),
    "thd_split_17": ("thd", (17, 8, 64), 2, 512, 512, 64, False, True, (0, 5, 5, 12, 17)),
    "bshd_random": ("bshd", (1, 24, 8, 64), 2, 512, 512, 64, True, False, None),
    "bshd_cfg1_full": ("bshd", (1, 256, 12, 128), 2, 1536, 1536, 128, True, True, None),
}
HASH_ONLY = ("bshd_cfg1_full",)


def _bf16_round(values: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = (bits + (np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def golden_inputs(name: str) -> dict[str, object]:
    """Seeded inputs of an unfused case as float32 arrays of BF16-representable values.

    peer-write inputs ``x[r]`` and pull inputs ``head_x[r]`` per rank, the
    weight for each direction (``w_pw`` is [N,K], ``w_pull`` is [K_out=N,K_in=N']
    with the exchanged width on the input side) and biases.
    """

    layout, dims, up, n, k, dim_out, has_bias, ints, cu = UNFUSED_CASES[name]
    seed = int.from_bytes(hashlib.sha1(name.encode()).digest()[:4], "little")
    rng = np.random.default_rng(seed)

    def tensor(shape, scale=1.0, lo=-4, hi=5):
        if ints:
            return rng.integers(lo, hi, size=shape).astype(np.float32)
        return _bf16_round((rng.standard_normal(shape) * scale).astype(np.float32))

    w_pw = tensor((n, k), scale=k ** -0.5, lo=-1, hi=2)
    b_pw = tensor((n,), scale=0.02, lo=-3, hi=4) if has_bias else None
    xs = [tensor(dims) for _ in range(up)]
    # pull direction: exchanged width is the INPUT width n; output width k_out = k rounded to 256
    n_out = max(256, (k + 255) // 256 * 256)
    w_pull = tensor((n_out, n), scale=n ** -0.5, lo=-1, hi=2)
    b_pull = tensor((n_out,), scale=0.02, lo=-3, hi=4) if has_bias else None
    shard_heads = n // (up * dim_out)
    if layout == "bshd":
        batch, seq = dims[0], dims[1]
        hshape = (batch, up * seq, shard_heads, dim_out)
    elif layout == "sbhd":
        seq, batch = dims[0], dims[1]
        hshape = (up * seq, batch, shard_heads, dim_out)
    else:
        hshape = (up * dims[0], shard_heads, dim_out)
    head_xs = [tensor(hshape) for _ in range(up)]
    return {
        "layout": layout, "up": up, "cu": cu, "xs": xs, "head_xs": head_xs,
        "w_pw": w_pw, "b_pw": b_pw, "w_pull": w_pull, "b_pull": b_pull,
    }


def _to_bits(t) -> np.ndarray:
    import torch

    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def _worker(rank: int, world: int, port: int, ref_root: str, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import run_distributed_correctness as ref  # the reference's own runner module

    def bf(a):
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16)

    results: dict[str, np.ndarray] = {}
    for name, (layout, dims, up, n, k, dim_out, has_bias, ints, cu) in UNFUSED_CASES.items():
        g = golden_inputs(name)
        x, hx = bf(g["xs"][rank]), bf(g["head_xs"][rank])
        w_pw, b_pw, w_pull, b_pull = bf(g["w_pw"]), bf(g["b_pw"]), bf(g["w_pull"]), bf(g["b_pull"])
        group = dist.group.WORLD
        if layout == "bshd":
            pw = ref.baseline_peer_write(x, w_pw, b_pw, up=up, group=group)
            mat, out = ref.baseline_pull_gemm(hx, w_pull, b_pull, up=up, group=group)
        elif layout == "sbhd":
            pw = ref.baseline_peer_write_sbhd(x, w_pw, b_pw, up=up, group=group)
            mat, out = ref.baseline_pull_gemm_sbhd(hx, w_pull, b_pull, up=up, group=group)
        else:
            pw = ref.baseline_peer_write_thd(x, w_pw, b_pw, cu, up=up, group=group)
            mat, out = ref.baseline_pull_gemm_thd(hx, w_pull, b_pull, cu, up=up, group=group)
        results[f"{name}/pw/{rank}"] = _to_bits(pw)
        results[f"{name}/pull_mat/{rank}"] = _to_bits(mat)
        results[f"{name}/pull_out/{rank}"] = _to_bits(out)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **results)
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    import torch
    import torch.multiprocessing as mp

    from mega_up import unsupported_shape_reason
    from mega_up.kernels.peer_write_gemm import PEER_TILE_N, peer_n_rotation
    from mega_up.ops import (
        _bshd_to_destination_major,
        _build_thd_layout,
        _source_major_to_bshd,
        _source_major_to_thd,
        _thd_to_destination_major,
    )

    shape_rows = [[w, u, unsupported_shape_reason(w, u)] for w in SHAPE_WIDTHS for u in SHAPE_UPS]
    (HERE / "shape_rule.json").write_text(json.dumps(shape_rows, indent=0))

    rotation = {
        f"{hidden},{up}": [peer_n_rotation(r, up, hidden, PEER_TILE_N) for r in range(up)]
        for hidden, up in ROTATION_CASES
    }
    (HERE / "rotation.json").write_text(json.dumps({"tile_n": PEER_TILE_N, "starts": rotation}, indent=0))

    thd: dict[str, np.ndarray] = {}
    for i, (cu, up) in enumerate(THD_CASES):
        layout = _build_thd_layout(cu, up=up, device="cpu")
        thd[f"{i}/cu"] = np.asarray(cu, dtype=np.int64)
        thd[f"{i}/up"] = np.asarray(up, dtype=np.int64)
        thd[f"{i}/to_thd"] = layout.to_thd_index.numpy()
        thd[f"{i}/to_source_major"] = layout.to_source_major_index.numpy()
        thd[f"{i}/cu_out"] = np.asarray(layout.cu_seqlens_out, dtype=np.int64)
        thd[f"{i}/fingerprint"] = np.frombuffer(layout.fingerprint.encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "thd_layouts.npz", **thd)

    helpers: dict[str, np.ndarray] = {}
    up, batch, seq, sh, dim = 4, 3, 5, 2, 8
    sm = torch.arange(up * batch * seq * sh * dim, dtype=torch.float32).view(up, batch * seq, sh * dim)
    helpers["source_major_to_bshd"] = _source_major_to_bshd(
        sm, batch=batch, sequence=seq, shard_heads=sh, head_dim=dim
    ).numpy()
    hp = torch.arange(batch * up * seq * sh * dim, dtype=torch.float32).view(batch, up * seq, sh, dim)
    helpers["bshd_to_destination_major"] = _bshd_to_destination_major(hp, up=up, sequence=seq).numpy()
    cu = (0, 3, 10, 11, 16)
    layout = _build_thd_layout(cu, up=up, device="cpu")
    smt = torch.arange(up * 16 * sh * dim, dtype=torch.float32).view(up, 16, sh * dim)
    helpers["source_major_to_thd"] = _source_major_to_thd(smt, layout, shard_heads=sh, head_dim=dim).numpy()
    hpt = torch.arange(up * 16 * sh * dim, dtype=torch.float32).view(up * 16, sh, dim)
    helpers["thd_to_destination_major"] = _thd_to_destination_major(hpt, layout).numpy()
    helpers["meta"] = np.asarray([up, batch, seq, sh, dim], dtype=np.int64)
    helpers["cu"] = np.asarray(cu, dtype=np.int64)
    np.savez_compressed(HERE / "layout_helpers.npz", **helpers)

    import tempfile

    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(2, 29541, ref_root, tmp), nprocs=2, join=True)
        merged: dict[str, np.ndarray] = {}
        for rank in range(2):
            with np.load(os.path.join(tmp, f"rank{rank}.npz")) as data:
                for key in data.files:
                    case = key.split("/")[0]
                    if case in HASH_ONLY:
                        digest = hashlib.sha256(data[key].tobytes()).hexdigest()
                        merged[key + "/sha256"] = np.frombuffer(digest.encode(), dtype=np.uint8)
                        merged[key + "/shape"] = np.asarray(data[key].shape, dtype=np.int64)
                    else:
                        merged[key] = data[key]
        np.savez_compressed(HERE / "unfused_ws2.npz", **merged)
    for f in sorted(HERE.glob("*.np*")) + sorted(HERE.glob("*.json")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
