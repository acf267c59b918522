"""A host model of how the pull kernel hands tickets to its pull warps (chunks of
eight tickets a stride apart; the first chunk of every warp pre-assigned and
claimed with an atomic maximum of the launch ordinal; later chunks drawn from a
cursor that only grows; unclaimed first chunks taken over once the cursor has
run out). The model restates megaup_b200/csrc/mup_gemm.cuh's pull-worker loop
and the cursor arithmetic of mup_pull_launch; it checks the properties the
kernel relies on under arbitrary warp interleavings, including CTAs that start
late or only after the others have finished: every ticket is copied exactly
once per launch, and consecutive launches agree on the cursor base."""

from __future__ import annotations

import random

import pytest

CHUNK = 8


class Workspace:
    def __init__(self, warps: int) -> None:
        self.cursor = 0
        self.claimed = [0] * warps


def launch(ws: Workspace, launches_before: int, total: int, warps: int, order: list[int], late: set[int], rng):
    """One launch. ``order`` is the order in which warps take a step whenever
    several could; warps in ``late`` only start once every other warp has
    finished. Returns the per-ticket copy counts."""

    block = warps * CHUNK
    chunks = -(-total // block) * warps
    drawn_per_launch = max(chunks - warps, 0)
    epoch1 = launches_before + 1
    cursor_base = launches_before * (drawn_per_launch + warps)
    copied = [0] * total

    def warp_program(me: int):
        before = ws.claimed[me]                       # atomicMax(claimed[me], epoch1)
        ws.claimed[me] = max(before, epoch1)
        copy_it = before < epoch1
        yield
        c, stealing, steal_pos = me, False, 0
        while True:
            drawn = None
            if not stealing:
                drawn = ws.cursor                     # atomicAdd(cursor, 1)
                ws.cursor += 1
            if copy_it:
                t_first = (c // warps) * block + (c % warps)
                for i in range(CHUNK):
                    t = t_first + i * warps
                    if t >= total:
                        break
                    copied[t] += 1
                    yield
            if not stealing:
                c = drawn - cursor_base + warps
                copy_it = True
                if c >= chunks:
                    stealing = True
            if stealing:
                found = False
                while steal_pos < warps and not found:
                    for bit in range(32):
                        idx = steal_pos + bit
                        if idx >= warps:
                            break
                        j = (me + 1 + idx) % warps
                        if ws.claimed[j] < epoch1:
                            yield
                            old = ws.claimed[j]       # atomicMax(claimed[j], epoch1)
                            ws.claimed[j] = max(old, epoch1)
                            if old < epoch1:
                                c, found = j, True
                                break
                    else:
                        steal_pos += 32
                        continue
                    if not found:
                        steal_pos += 32
                if not found:
                    return
                copy_it = True

    running = {w: warp_program(w) for w in order if w not in late}
    waiting = [w for w in order if w in late]
    while running or waiting:
        if not running:
            running = {w: warp_program(w) for w in waiting}
            waiting = []
        w = rng.choice(list(running))
        try:
            next(running[w])
        except StopIteration:
            del running[w]
    return copied, cursor_base + drawn_per_launch + warps


@pytest.mark.parametrize("total,warps", [(8192, 888), (100, 12), (1, 12), (97, 24), (5000, 48), (96, 12)])
@pytest.mark.parametrize("late_fraction", [0.0, 0.1, 0.5])
def test_every_ticket_is_copied_once_and_the_cursor_stays_in_step(total, warps, late_fraction) -> None:
    rng = random.Random(total * 31 + warps)
    ws = Workspace(warps)
    for launches_before in range(3):
        order = list(range(warps))
        rng.shuffle(order)
        late = set(rng.sample(order, int(late_fraction * warps)))
        copied, cursor_after = launch(ws, launches_before, total, warps, order, late, rng)
        assert copied == [1] * total
        # the host predicts where the cursor stands after a launch without reading it back
        assert ws.cursor == cursor_after
        assert all(word == launches_before + 1 for word in ws.claimed)
