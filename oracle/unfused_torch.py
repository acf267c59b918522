"""TEST INFRASTRUCTURE - the reference's unfused CPU path, restated with torch CPU ops
for timing: ``F.linear`` + permute + equal-split all-to-all (the peer-write
baseline) and all-to-all + permute + ``F.linear`` (the pull baseline), as in
tests/run_distributed_correctness.py:236-336 and benchmarks/bench_bshd.py:225-494
of the reference. One process plays one rank; the blocks it would exchange
with its peers are memory copies of the same size (a gloo all_to_all_single
on one host is a set of copies through shared memory as well).

Only the bench's CPU-baseline / reference legs and the tests may import this.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor


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
