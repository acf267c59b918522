"""Worker bodies for the multi-process (gloo, CPU) tests."""

from __future__ import annotations

import os
import sys
import traceback
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _init(rank: int, world: int, port: int) -> None:
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def run(rank: int, world: int, port: int, body: str, out_dir: str) -> None:
    """Run ``body`` (a function name in this module) and record its verdict."""

    import torch.distributed as dist

    verdict = "ok"
    try:
        _init(rank, world, port)
        globals()[body](rank, world)
    except Exception:  # noqa: BLE001 - reported through the file
        verdict = traceback.format_exc()
    finally:
        Path(out_dir, f"rank{rank}.txt").write_text(verdict)
        if dist.is_initialized():
            dist.destroy_process_group()


class _FakeRuntime:
    """Just enough of MegaUPRuntime for the host-side collective checks."""

    def __init__(self, rank: int, world: int) -> None:
        import torch
        import torch.distributed as dist

        self.group = dist.group.WORLD
        self.up = world
        self.local_rank = rank
        self.device = torch.device("cpu")
        self.hidden = 512
        self.max_rows = 64


def collective_validation(rank: int, world: int) -> None:
    from megaup_b200.ops import _collective_validate

    runtime = _FakeRuntime(rank, world)
    # agreeing ranks pass
    _collective_validate(runtime, "op", ("meta", 1), None)
    # a rank-local error raises on every rank, naming the failing rank
    try:
        _collective_validate(runtime, "op", ("meta", 1), "ValueError: bad" if rank == 1 else None)
    except ValueError as error:
        assert "collective validation failed" in str(error) and "(1, 'ValueError: bad')" in str(error)
    else:
        raise AssertionError("a rank-local error must raise everywhere")
    # diverging metadata raises on every rank
    try:
        _collective_validate(runtime, "op", ("meta", rank), None)
    except ValueError as error:
        assert "identical" in str(error)
    else:
        raise AssertionError("diverging metadata must raise everywhere")
    # diverging operations raise too
    try:
        _collective_validate(runtime, f"op{rank}", ("meta",), None)
    except ValueError:
        pass
    else:
        raise AssertionError("diverging operations must raise everywhere")


def fd_exchange(rank: int, world: int) -> None:
    import torch.distributed as dist

    from megaup_b200.runtime import exchange_fds

    fd = os.memfd_create(f"rank{rank}")
    os.write(fd, f"payload-of-rank-{rank}".encode())
    received = exchange_fds(dist.group.WORLD, fd)
    assert len(received) == world and received[rank] == fd
    for peer, peer_fd in enumerate(received):
        os.lseek(peer_fd, 0, os.SEEK_SET)
        assert os.read(peer_fd, 64) == f"payload-of-rank-{peer}".encode()
    # a second exchange in the same processes works too (fresh socket names)
    again = exchange_fds(dist.group.WORLD, fd)
    assert len(again) == world


def sharded_oracle_exchange(rank: int, world: int) -> None:
    """The package's layout helpers over a REAL all_to_all_single (gloo) equal the
    single-process oracle - the N>1 exchange semantics, on CPU."""

    import numpy as np
    import torch
    import torch.distributed as dist

    from megaup_b200.ops import _bshd_to_destination_major, _source_major_to_bshd
    from oracle import ulysses_oracle as oracle

    batch, seq, shard_heads, dim = 2, 5, 2, 8
    rng = np.random.default_rng(3)
    dense = [rng.integers(-8, 9, (batch * seq, world * shard_heads * dim)).astype(np.float32) for _ in range(world)]
    mine = torch.from_numpy(dense[rank])
    send = mine.view(batch * seq, world, shard_heads * dim).permute(1, 0, 2).contiguous()
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send)
    got = _source_major_to_bshd(received, batch=batch, sequence=seq, shard_heads=shard_heads, head_dim=dim)
    want = oracle.copy_peer_written(
        np.concatenate([d.reshape(batch * seq, world, -1)[:, rank] for d in dense]).reshape(-1),
        world, batch, seq, shard_heads * dim,
    )
    assert np.array_equal(got.numpy().reshape(want.shape), want)
    # and back: destination-major staging + all_to_all = the pulled dense input
    staged = _bshd_to_destination_major(got, up=world, sequence=seq)
    back = torch.empty_like(staged)
    dist.all_to_all_single(back, staged)
    dy = back.permute(1, 0, 2).reshape(batch * seq, -1)
    staged_all = [None] * world
    dist.all_gather_object(staged_all, staged.numpy().reshape(-1))
    want_dy = oracle.pull_gather(staged_all, rank, batch * seq, shard_heads * dim)
    assert np.array_equal(dy.numpy(), want_dy)
