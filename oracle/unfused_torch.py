"""TEST INFRASTRUCTURE - the reference's unfused CPU path, restated with torch CPU ops
for timing: ``F.linear`` + permute + equal-split all-to-all (the peer-write
baseline) and all-to-all + permute + ``F.linear`` (the pull baseline), as in
tests/run_distributed_correctness.py:236-336 and benchmarks/bench_bshd.py:225-494
of the reference. One process plays one rank; the blocks it would exchange
with its peers are memory copies of the same size (a gloo all_to_all_single
on one host is a set of copies through shared memory as well).

``reference_baselines()`` returns the reference's own ``baseline_peer_write`` /
``baseline_pull_gemm`` when its runner has been installed next to the repo
(``baseline/install_reference.sh``), else restatements of them; both take a
process group and run a real ``all_to_all_single`` (gloo on the host).

Only the bench's CPU-baseline / reference legs and the tests may import this.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path
from typing import Callable

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor

_RUNNER = Path(__file__).resolve().parent.parent / "baseline" / "_ref" / "reference_runners" / "run_distributed_correctness.py"
# names the reference's runner imports from its package at module level; the
# unfused baselines use none of them
_PACKAGE_NAMES = (
    "SUPPORTED_UP_DEGREES", "initialize_runtime", "peer_write_gemm_bshd", "peer_write_gemm_sbhd",
    "peer_write_gemm_thd", "prepare_headshard_pull_gemm_bshd", "prepare_headshard_pull_gemm_sbhd",
    "prepare_headshard_pull_gemm_thd", "prepare_peer_write_gemm_bshd", "prepare_peer_write_gemm_sbhd",
    "prepare_peer_write_gemm_thd", "prepare_thd_layout",
)


def port_baseline_peer_write(x: Tensor, weight: Tensor, bias: Tensor | None, *, up: int, group) -> Tensor:
    """``F.linear`` + permute + ``all_to_all_single`` of ``[B,S,H,D]``
    (restates tests/run_distributed_correctness.py:236-258 of the reference)."""

    batch, sequence, heads, head_dim = map(int, x.shape)
    shard_heads = int(weight.shape[0]) // (up * head_dim)
    dense = F.linear(x.view(batch, sequence, heads * head_dim), weight, bias)
    send = dense.view(batch, sequence, up, shard_heads, head_dim).permute(2, 0, 1, 3, 4).contiguous()
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send, group=group)
    return received.permute(1, 0, 2, 3, 4).reshape(batch, up * sequence, shard_heads, head_dim).contiguous()


def port_baseline_pull_gemm(head_x: Tensor, weight: Tensor, bias: Tensor | None, *, up: int, group):
    """``all_to_all_single`` + permute + ``F.linear`` of ``[B,UP*S,H/UP,D]``
    (restates tests/run_distributed_correctness.py:306-336 of the reference)."""

    batch, global_sequence, shard_heads, head_dim = map(int, head_x.shape)
    sequence = global_sequence // up
    heads = shard_heads * up
    send = head_x.view(batch, up, sequence, shard_heads, head_dim).permute(1, 0, 2, 3, 4).contiguous()
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send, group=group)
    materialized = received.permute(1, 2, 0, 3, 4).reshape(batch, sequence, heads, head_dim).contiguous()
    output = F.linear(materialized.view(batch, sequence, heads * head_dim), weight, bias)
    return materialized, output.view(batch, sequence, -1, head_dim)


def reference_baselines() -> tuple[Callable, Callable, str]:
    """``(baseline_peer_write, baseline_pull_gemm, kind)``: the reference's own
    functions (kind ``"reference"``) when its runner is installed under
    ``baseline/_ref``, else the restatements above (kind ``"port"``). The
    runner imports its package at module level only to bind names the baselines
    never call, so a placeholder module stands in for it while the file loads:
    none of the reference's (or this repo's) kernels is imported."""

    if not _RUNNER.exists():
        return port_baseline_peer_write, port_baseline_pull_gemm, "port"
    placeholder = types.ModuleType("mega_up")
    for name in _PACKAGE_NAMES:
        setattr(placeholder, name, None)
    saved = sys.modules.get("mega_up")
    sys.modules["mega_up"] = placeholder
    try:
        spec = importlib.util.spec_from_file_location("_reference_runner", _RUNNER)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return module.baseline_peer_write, module.baseline_pull_gemm, "reference"
    except Exception:  # noqa: BLE001 - an unusable install falls back to the restatement
        return port_baseline_peer_write, port_baseline_pull_gemm, "port"
    finally:
        if saved is None:
            sys.modules.pop("mega_up", None)
        else:
            sys.modules["mega_up"] = saved


class UnfusedRank:
    """One rank's share of the unfused BSHD (B=1) path on the host cores."""

    def __init__(self, rows: int, hidden: int, up: int, seed: int = 0) -> None:
        gen = torch.Generator().manual_seed(seed)
        self.rows, self.hidden, self.up = rows, hidden, up
        shard = hidden // up
        scale = hidden ** -0.5
        self.w_q = (torch.randn(hidden, hidden, generator=gen) * scale).to(torch.bfloat16)
        self.w_o = (torch.randn(hidden, hidden, generator=gen) * scale).to(torch.bfloat16)
        self.b_q = (torch.randn(hidden, generator=gen) * 0.02).to(torch.bfloat16)
        self.b_o = (torch.randn(hidden, generator=gen) * 0.02).to(torch.bfloat16)
        self.x = torch.randn(rows, hidden, generator=gen).to(torch.bfloat16)
        self.head_x = torch.randn(up * rows, shard, generator=gen).to(torch.bfloat16)
        self.recv = torch.empty(up, rows, shard, dtype=torch.bfloat16)

    def peer_write(self) -> Tensor:
        """linear -> [U, rows, shard] send buffer -> exchange -> [U*rows, shard]."""

        dense = F.linear(self.x, self.w_q, self.b_q)
        send = dense.view(self.rows, self.up, -1).permute(1, 0, 2).contiguous()
        self.recv.copy_(send)  # the all-to-all: every block is copied once
        return self.recv.reshape(self.up * self.rows, -1)

    def pull(self) -> Tensor:
        """[U*rows, shard] -> exchange -> dense [rows, hidden] -> linear."""

        send = self.head_x.view(self.up, self.rows, -1)
        self.recv.copy_(send)
        dense = self.recv.permute(1, 0, 2).reshape(self.rows, self.hidden).contiguous()
        return F.linear(dense, self.w_o, self.b_o)

    def step(self) -> None:
        self.peer_write()
        self.pull()

    @property
    def flops_per_step(self) -> float:
        return 2 * 2.0 * self.rows * self.hidden * self.hidden
