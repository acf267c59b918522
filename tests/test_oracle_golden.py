"""Pin the CPU oracle against fixtures produced by running the reference
(tests/golden/make_golden.py) and against its own invariants."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

import make_golden
from oracle import ulysses_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_shape_rule_matches_the_reference_strings() -> None:
    rows = json.loads((GOLDEN / "shape_rule.json").read_text())
    assert len(rows) == len(make_golden.SHAPE_WIDTHS) * len(make_golden.SHAPE_UPS)
    for width, up, reason in rows:
        assert oracle.unsupported_shape_reason(width, up) == reason


def test_rotation_tables() -> None:
    data = json.loads((GOLDEN / "rotation.json").read_text())
    for key, starts in data["starts"].items():
        hidden, up = map(int, key.split(","))
        got = [oracle.peer_n_rotation(r, up, hidden, data["tile_n"]) for r in range(up)]
        assert got == starts
        # property the reference tests (for shards of at least one tile): the
        # first tile overlaps the rank's own shard
        shard = hidden // up
        if shard < 256:
            continue
        for rank, start in enumerate(got):
            assert start * 256 < (rank + 1) * shard and (start + 1) * 256 > rank * shard


def test_thd_layouts() -> None:
    with np.load(GOLDEN / "thd_layouts.npz") as data:
        for i in range(len(make_golden.THD_CASES)):
            cu = tuple(data[f"{i}/cu"].tolist())
            layout = oracle.thd_layout(cu, int(data[f"{i}/up"]))
            assert np.array_equal(layout["to_thd_index"], data[f"{i}/to_thd"])
            assert np.array_equal(layout["to_source_major_index"], data[f"{i}/to_source_major"])
            assert layout["cu_seqlens_out"] == tuple(data[f"{i}/cu_out"].tolist())
            assert layout["fingerprint"] == bytes(data[f"{i}/fingerprint"]).decode()


def test_known_answer_from_the_reference_layout_test() -> None:
    layout = oracle.thd_layout((0, 5, 5, 12, 13), 3)
    assert layout["tokens"] == 13
    assert layout["cu_seqlens_out"] == (0, 15, 15, 36, 39)
    total = 3 * 13
    assert np.array_equal(np.sort(layout["to_thd_index"]), np.arange(total))
    assert np.array_equal(layout["to_thd_index"][layout["to_source_major_index"]], np.arange(total))


def test_layout_helpers() -> None:
    with np.load(GOLDEN / "layout_helpers.npz") as data:
        up, batch, seq, sh, dim = data["meta"].tolist()
        cu = tuple(data["cu"].tolist())
        arena = np.arange(up * batch * seq * sh * dim, dtype=np.float32)
        got = oracle.copy_peer_written(arena, up, batch, seq, sh * dim).reshape(batch, up * seq, sh, dim)
        assert np.array_equal(got, data["source_major_to_bshd"])
        hp = np.arange(batch * up * seq * sh * dim, dtype=np.float32).reshape(batch, up * seq, sh, dim)
        staged = oracle.stage_head_parallel(hp, up).reshape(up, batch * seq, sh * dim)
        assert np.array_equal(staged, data["bshd_to_destination_major"])
        layout = oracle.thd_layout(cu, up)
        arena = np.arange(up * 16 * sh * dim, dtype=np.float32)
        got = oracle.copy_peer_written_indexed(arena, up, 16, sh * dim, layout["to_thd_index"])
        assert np.array_equal(got.reshape(up * 16, sh, dim), data["source_major_to_thd"])
        assert np.array_equal(got, oracle.regroup_thd(arena.reshape(up, 16, sh * dim), cu))
        flat = np.arange(up * 16 * sh * dim, dtype=np.float32).reshape(up * 16, sh * dim)
        staged = oracle.stage_rows_indexed(flat, layout["to_source_major_index"])
        assert np.array_equal(staged.reshape(up, 16, sh * dim), data["thd_to_destination_major"])
        assert np.array_equal(staged.reshape(up, 16, sh * dim), oracle.split_thd(flat, cu, up))


def _oracle_case(name: str):
    g = make_golden.golden_inputs(name)
    layout, cu = g["layout"], g["cu"]
    if layout == "bshd":
        pw = oracle.peer_write_bshd(g["xs"], g["w_pw"], g["b_pw"])
        pull = oracle.pull_bshd(g["head_xs"], g["w_pull"], g["b_pull"])
    elif layout == "sbhd":
        pw = oracle.peer_write_sbhd(g["xs"], g["w_pw"], g["b_pw"])
        pull = oracle.pull_sbhd(g["head_xs"], g["w_pull"], g["b_pull"])
    else:
        pw = oracle.peer_write_thd(g["xs"], g["w_pw"], g["b_pw"], cu)
        pull = oracle.pull_thd(g["head_xs"], g["w_pull"], g["b_pull"], cu)
    return g, pw, pull


@pytest.mark.parametrize("name", [n for n in make_golden.UNFUSED_CASES])
def test_unfused_path_matches_the_reference_run(name: str) -> None:
    """The reference's F.linear + permute + all_to_all_single (gloo, 2 ranks)."""

    g, pw, pull = _oracle_case(name)
    ints = make_golden.UNFUSED_CASES[name][7]
    with np.load(GOLDEN / "unfused_ws2.npz") as data:
        for rank in range(g["up"]):
            got = {"pw": pw[rank], "pull_mat": pull[rank][0], "pull_out": pull[rank][1]}
            for kind, value in got.items():
                key = f"{name}/{kind}/{rank}"
                bits = oracle.bf16_bits(value)
                if name in make_golden.HASH_ONLY:
                    assert tuple(data[key + "/shape"].tolist()) == bits.shape
                    assert hashlib.sha256(bits.tobytes()).hexdigest() == bytes(data[key + "/sha256"]).decode()
                    continue
                want = data[key]
                assert want.shape == bits.shape, key
                if ints or kind == "pull_mat":
                    assert np.array_equal(bits, want), key  # bit-exact
                else:
                    # random values: oneDNN's BF16 dot product is not the FP32
                    # ascending-K sum; the reference's own tolerance is 3e-2
                    ref = oracle.from_bf16_bits(want)
                    assert np.allclose(value, ref, rtol=3e-2, atol=3e-2), key
                    ulp = np.abs(value - ref) / np.maximum(np.abs(ref) * 2.0 ** -7, 1e-30)
                    assert np.mean(bits != want) < 0.02 and ulp.max() <= 2.0, key


@pytest.mark.parametrize("up,batch,seq,n,k", [(2, 1, 24, 512, 256), (4, 2, 9, 1024, 128), (8, 1, 5, 1024, 64), (2, 3, 7, 2304, 64)])
def test_slot_arithmetic_equals_the_all_to_all_path(up, batch, seq, n, k) -> None:
    """Peer routing + dense slot packing + copy-out == linear + permute + all_to_all,
    and staging + pull gather == permute + all_to_all, bit for bit."""

    rng = np.random.default_rng(up * 1000 + n)
    dim = 64
    w = rng.integers(-1, 2, (n, k)).astype(np.float32)
    b = rng.integers(-3, 4, (n,)).astype(np.float32)
    xs = [rng.integers(-4, 5, (batch, seq, k // dim, dim)).astype(np.float32) for _ in range(up)]
    want = oracle.peer_write_bshd(xs, w, b)
    dense = [oracle.linear(x.reshape(batch * seq, k), w, b) for x in xs]
    arenas = oracle.peer_write_fill_arenas(dense, up)
    shard = n // up
    for rank in range(up):
        got = oracle.copy_peer_written(arenas[rank], up, batch, seq, shard)
        assert np.array_equal(got.reshape(want[rank].shape), want[rank])
    # pull direction: exchanged width n on the input side
    heads = [rng.integers(-4, 5, (batch, up * seq, shard // dim, dim)).astype(np.float32) for _ in range(up)]
    w2 = rng.integers(-1, 2, (256, n)).astype(np.float32)
    want_pull = oracle.pull_bshd(heads, w2, None)
    staged = [oracle.stage_head_parallel(h, up) for h in heads]
    for rank in range(up):
        dy = oracle.pull_gather(staged, rank, batch * seq, shard)
        assert np.array_equal(dy.reshape(want_pull[rank][0].shape), want_pull[rank][0])


def test_c_kernel_and_blas_agree_on_exact_cases_and_within_an_ulp_otherwise() -> None:
    rng = np.random.default_rng(7)
    x = rng.integers(-4, 5, (33, 520)).astype(np.float32)
    w = rng.integers(-1, 2, (256, 520)).astype(np.float32)
    b = rng.integers(-3, 4, (256,)).astype(np.float32)
    assert np.array_equal(oracle.linear(x, w, b), oracle.linear(x, w, b, use_c=False))
    x = oracle.bf16_round(rng.standard_normal((64, 1024)).astype(np.float32))
    w = oracle.bf16_round((rng.standard_normal((256, 1024)) / 32).astype(np.float32))
    a, c = oracle.linear(x, w, None), oracle.linear(x, w, None, use_c=False)
    assert np.mean(a != c) < 0.01
    assert np.all(np.abs(a - c) <= np.maximum(np.abs(c), 2.0 ** -126) * 2.0 ** -7)


def test_bf16_rounding_is_nearest_even() -> None:
    # 1 + 2^-8 is a tie -> even (1.0); 1 + 3*2^-8 is a tie -> even (1 + 2^-6)
    values = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 1.005, 0.0], dtype=np.float32)
    got = oracle.bf16_round(values)
    assert got.tolist() == [1.0, 1.0, 1.015625, -1.0, 1.0078125, 0.0]
    assert np.array_equal(oracle.from_bf16_bits(oracle.bf16_bits(got)), got)
