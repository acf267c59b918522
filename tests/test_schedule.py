"""The work-item lists the library builds (host arithmetic, no GPU): every list
must tile the output exactly once, respect the widest item a CTA grouping can
run, and start every rank of a peer-write group in a different column block."""

from __future__ import annotations

import ctypes
from collections import defaultdict

import pytest

from megaup_b200 import _native, build

NO_ITEM = 0xFFFFFFFF
UNIT = 64

SHAPES = [
    # rows, n, k, up
    (4096, 5120, 5120, 8),     # Wan2.1-14B projection
    (4096, 5120, 5120, 2),
    (8192, 6144, 4096, 8),     # Llama-3-8B fused QKV
    (16384, 8192, 8192, 8),    # Llama-3-70B O projection
    (512, 2304, 2304, 2),      # odd number of 256-column blocks
    (1024, 2048, 2048, 8),
    (64, 1024, 4096, 8),       # fewer rows than a row tile
    (300, 2304, 2304, 2),      # ragged rows
    (65536, 5120, 5120, 8),
    (129, 256, 64, 2),
]


@pytest.fixture(scope="module", autouse=True)
def _library() -> None:
    build.ensure_built()


def preview(mode: int, rows: int, n: int, k: int, up: int, rank: int, cta_group: int, slots: int):
    count, widest, cycles = ctypes.c_int(), ctypes.c_int(), ctypes.c_double()
    _native.call(
        "mup_schedule_preview", mode, rows, n, k, up, rank, cta_group, slots, None, 0,
        ctypes.byref(count), ctypes.byref(widest), ctypes.byref(cycles),
    )
    buffer = (ctypes.c_uint32 * max(1, count.value))()
    _native.call(
        "mup_schedule_preview", mode, rows, n, k, up, rank, cta_group, slots, buffer, count.value,
        None, None, None,
    )
    return list(buffer[: count.value]), widest.value, cycles.value


def decode(entry: int) -> tuple[int, int, int]:
    return entry & 0x3FFF, (entry >> 14) & 0xFFF, ((entry >> 26) & 0x7) + 1


@pytest.mark.parametrize("rows,n,k,up", SHAPES)
@pytest.mark.parametrize("mode", (0, 1))
@pytest.mark.parametrize("cta_group,slots", ((2, 74), (1, 148), (2, 8)))
def test_items_tile_the_output_exactly_once(rows, n, k, up, mode, cta_group, slots) -> None:
    items, widest, cycles = preview(mode, rows, n, k, up, up - 1, cta_group, slots)
    m_tiles = -(-rows // (128 * cta_group))
    covered: dict[int, list[tuple[int, int]]] = defaultdict(list)
    limit = 512 if cta_group == 2 else 256
    seen_widest = 0
    for entry in items:
        if entry == NO_ITEM:
            continue
        m, n0, w = decode(entry)
        assert 0 <= m < m_tiles
        assert UNIT * w <= limit
        seen_widest = max(seen_widest, UNIT * w)
        covered[m].append((n0, n0 + w))
    assert seen_widest == widest
    assert cycles > 0
    assert sorted(covered) == list(range(m_tiles))
    for m, spans in covered.items():
        spans.sort()
        assert spans[0][0] == 0 and spans[-1][1] == n // UNIT, (m, spans)
        for (_, stop), (start, _) in zip(spans, spans[1:]):
            assert stop == start, (m, spans)
    # the list never ends in a placeholder, and placeholders only pad whole rounds
    assert items[-1] != NO_ITEM
    if NO_ITEM in items:
        assert len(items) > slots


def test_two_accumulator_items_are_chosen_where_they_were_measured_faster() -> None:
    # K = 8192 (16384 x 8192 x 8192 pull: 10 % faster with 512-wide items), not K = 4096 or 5120
    assert preview(1, 16384, 8192, 8192, 8, 0, 2, 74)[1] > 256
    assert preview(0, 4096, 5120, 5120, 8, 0, 2, 74)[1] == 256
    assert preview(0, 8192, 6144, 4096, 8, 0, 2, 74)[1] == 256


def test_headline_shape_balances_the_rounds() -> None:
    items, widest, _ = preview(0, 4096, 5120, 5120, 8, 0, 2, 74)
    per_slot: dict[int, int] = defaultdict(int)
    for index, entry in enumerate(items):
        if entry != NO_ITEM:
            per_slot[index % 74] += decode(entry)[2]
    total = 16 * (5120 // UNIT)
    assert sum(per_slot.values()) == total
    # no CTA pair carries more than 64 columns above an even share
    assert max(per_slot.values()) <= -(-total // 74) + 1


def test_peer_write_ranks_start_in_different_column_blocks() -> None:
    starts = []
    for rank in range(8):
        items, _, _ = preview(0, 4096, 5120, 5120, 8, rank, 2, 74)
        starts.append(decode(items[0])[1] * UNIT)
    assert starts[0] == 0
    assert len(set(starts)) == 8
    assert starts == sorted(starts)
    # pull lists do not rotate: every rank consumes its panels from column 0
    for rank in (0, 5):
        items, _, _ = preview(1, 4096, 5120, 5120, 8, rank, 2, 74)
        assert decode(items[0])[:2] == (0, 0)


def test_pull_lists_consume_row_tiles_in_ascending_order_in_the_first_round() -> None:
    items, _, _ = preview(1, 4096, 5120, 5120, 8, 3, 2, 74)
    first_round = [decode(entry)[0] for entry in items[:74]]
    assert first_round == sorted(first_round)


def test_bad_schedule_arguments_are_rejected() -> None:
    with pytest.raises(_native.NativeError):
        preview(2, 4096, 5120, 5120, 8, 0, 2, 74)
    with pytest.raises(_native.NativeError):
        preview(0, 4096, 5000, 5120, 8, 0, 2, 74)
    with pytest.raises(_native.NativeError):
        preview(0, 4096, 5120, 5120, 8, 8, 2, 74)


def test_long_lists_stay_in_list_order_for_the_item_feed() -> None:
    # 16 rounds or more: the CTA pairs draw the items as they become free, so the
    # list is not dealt round by round (no placeholders; a pull list has its row
    # tiles ascending)
    items, _, _ = preview(1, 65536, 5120, 5120, 8, 0, 2, 74)
    assert len(items) >= 16 * 74
    assert NO_ITEM not in items
    rows = [decode(entry)[0] for entry in items]
    assert rows[: len(rows) - 74] == sorted(rows[: len(rows) - 74])
    assert NO_ITEM not in preview(0, 65536, 5120, 5120, 8, 0, 2, 74)[0]
    # a short pull list is dealt: the headline shape's partly filled last round has placeholders
    items, _, _ = preview(1, 4096, 5120, 5120, 8, 0, 2, 74)
    assert NO_ITEM in items


def test_peer_write_lists_walk_bands_of_row_tiles_and_alternate_destinations() -> None:
    up, shard_units = 8, 5120 // 64 // 8
    items, _, _ = preview(0, 4096, 5120, 5120, up, 3, 2, 74)
    assert NO_ITEM not in items
    decoded = [decode(entry) for entry in items]
    # the first 8 items are one column position of the 8 row tiles of the first band
    assert [d[0] for d in decoded[:8]] == list(range(8))
    assert len({d[1] for d in decoded[:8]}) == 1
    # the rank starts at its own column block, and the next column position goes elsewhere
    assert decoded[0][1] // shard_units == 3
    assert decoded[8][1] // shard_units != 3
    # the second band (row tiles 8..15) follows the first
    first_of_second_band = next(i for i, d in enumerate(decoded) if d[0] >= 8)
    assert all(d[0] < 8 for d in decoded[:first_of_second_band])


def _check_exact_tiling(items, rows, n, cta_group) -> None:
    m_tiles = -(-rows // (128 * cta_group))
    limit = 512 if cta_group == 2 else 256
    covered: dict[int, list[tuple[int, int]]] = defaultdict(list)
    for entry in items:
        if entry == NO_ITEM:
            continue
        m, n0, w = decode(entry)
        assert 0 <= m < m_tiles and UNIT * w <= limit
        covered[m].append((n0, n0 + w))
    assert sorted(covered) == list(range(m_tiles))
    for m, spans in covered.items():
        spans.sort()
        assert spans[0][0] == 0 and spans[-1][1] == n // UNIT, (m, spans)
        for (_, stop), (start, _) in zip(spans, spans[1:]):
            assert stop == start, (m, spans)
    assert items[-1] != NO_ITEM


def test_random_shapes_tile_exactly_once() -> None:
    """Seeded random problems over both modes, both CTA groupings, every UP degree
    and odd grid sizes: whatever list the library chooses (dealt, banded with
    alternating destinations, fed) covers every output element exactly once."""

    import random

    rng = random.Random(20240607)
    for _ in range(300):
        up = rng.choice((2, 4, 8))
        blocks = rng.randint(1, 40)               # exchanged width in 256-column blocks ...
        n = 256 * blocks
        while n % (128 * up):                     # ... with shards that are multiples of 128 columns
            blocks += 1
            n = 256 * blocks
        k = 64 * rng.randint(1, 128) if rng.random() < 0.8 else 8 * rng.randint(8, 1024)
        rows = rng.choice((1, 17, 64, 129, 300, 1000, 4096, rng.randint(1, 70000)))
        mode = rng.choice((0, 1))
        if mode == 1:
            k = n                                   # the pull contracts over the exchanged width
        cta_group = rng.choice((1, 2))
        slots = rng.choice((1, 7, 37, 74)) if cta_group == 2 else rng.choice((1, 13, 148))
        rank = rng.randrange(up)
        items, widest, cycles = preview(mode, rows, n, k, up, rank, cta_group, slots)
        assert cycles > 0 and widest <= (512 if cta_group == 2 else 256)
        _check_exact_tiling(items, rows, n, cta_group)
