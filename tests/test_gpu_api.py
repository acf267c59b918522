"""The mega_up-compatible host API on one GPU, driven through a single-process
emulated UP group: every layout, prepared and one-shot, against the golden
fixtures produced by the reference's unfused path and against the CPU oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import _gpu_harness as h
import make_golden
import megaup_b200 as mega_up
from megaup_b200 import ops
from oracle import ulysses_oracle as oracle

pytestmark = pytest.mark.gpu
GOLDEN = make_golden.HERE


def _group(up, hidden, max_rows):
    return mega_up.initialize_emulated_group(up, hidden=hidden, max_rows=max_rows, device=h.DEVICE)


def _prepare(kind, direction, weight, runtime, dims, layout, bias, **extra):
    name = f"prepare_{'peer_write' if direction == 'pw' else 'headshard_pull'}_gemm_{kind}"
    kwargs = dict(dims, bias=bias, validate_group=False, **extra)
    if kind == "thd":
        kwargs["layout"] = layout
    return getattr(mega_up, name)(weight, runtime, **kwargs)


def _dims(kind, shape):
    return dict(zip(ops._DIMS[kind], shape))


@pytest.mark.parametrize("name", list(make_golden.UNFUSED_CASES))
def test_api_matches_the_reference_unfused_path(name: str) -> None:
    kind, dims, up, n, k, dim_out, has_bias, ints, cu = make_golden.UNFUSED_CASES[name]
    g = make_golden.golden_inputs(name)
    rows = int(np.prod(dims[:-2]))
    # ---- peer-write: exchanged width n
    runtimes = _group(up, n, rows)
    layouts = [mega_up.prepare_thd_layout(cu, rt) if cu is not None else None for rt in runtimes]
    w, b = h.to_gpu(g["w_pw"]), h.to_gpu(g["b_pw"])
    # heads * head_dim only has to factor K; head_dim is the head size of the
    # exchanged OUTPUT, so the input is viewed with that head size
    pw_shape = tuple(dims[:-2]) + (k // dim_out, dim_out)
    prepared = [
        _prepare(kind, "pw", w, rt, _dims(kind, pw_shape), lay, b) for rt, lay in zip(runtimes, layouts)
    ]
    xs = [h.to_gpu(x).view(pw_shape) for x in g["xs"]]
    outs = mega_up.emulated_peer_write(prepared, xs)
    torch.cuda.synchronize()
    runtimes[0].check_status()
    # ---- pull: exchanged width n on the input side
    w2, b2 = h.to_gpu(g["w_pull"]), h.to_gpu(g["b_pull"])
    heads = n // dim_out
    pull_dims = _dims(kind, dims[:-2] + (heads, dim_out))
    pulls = [_prepare(kind, "pull", w2, rt, pull_dims, lay, b2) for rt, lay in zip(runtimes, layouts)]
    head_xs = [h.to_gpu(x) for x in g["head_xs"]]
    pull_outs = mega_up.emulated_pull(pulls, head_xs)
    torch.cuda.synchronize()
    runtimes[0].check_status()
    with np.load(GOLDEN / "unfused_ws2.npz") as data:
        for rank in range(up):
            got = {
                "pw": outs[rank], "pull_mat": pulls[rank].materialized_input, "pull_out": pull_outs[rank],
            }
            for what, tensor in got.items():
                key = f"{name}/{what}/{rank}"
                bits = tensor.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
                if name in make_golden.HASH_ONLY:
                    import hashlib

                    assert hashlib.sha256(bits.tobytes()).hexdigest() == bytes(data[key + "/sha256"]).decode(), key
                    continue
                want = data[key]
                assert bits.size == want.size, key
                if ints or what == "pull_mat":
                    assert np.array_equal(bits.reshape(want.shape), want), key
                else:
                    # the fixture is the reference's CPU F.linear (oneDNN BF16 dot products);
                    # the reference's own tolerance for GEMM values is rtol = atol = 3e-2
                    ref = torch.from_numpy(oracle.from_bf16_bits(want)).to(h.DEVICE)
                    got32 = tensor.reshape(ref.shape).float()
                    assert torch.allclose(got32, ref, rtol=3e-2, atol=3e-2), key
                    assert float((got32 != ref).float().mean()) < 0.05, key
    # the oracle's restatement of the same path agrees too (checked on CPU
    # against the same fixtures in test_oracle_golden.py)


@pytest.mark.parametrize("up", [2, 4, 8])
def test_wan_q_and_o_projection_bshd(up: int) -> None:
    """Wan2.1-14B-shaped Q/O projection: W[5120,5120] + bias, B=1, S_local=4096, H=40, D=128."""

    seq, heads, dim, hidden = 4096, 40, 128, 5120
    runtimes = _group(up, hidden, seq)
    w = h.seeded((hidden, hidden), 1, ints=True, lo=-1, hi=2)
    b = h.seeded((hidden,), 2, ints=True, lo=-3, hi=4)
    xs = [h.seeded((1, seq, heads, dim), 100 + r, ints=True) for r in range(up)]
    prepared = [
        mega_up.prepare_peer_write_gemm_bshd(w, rt, batch=1, sequence=seq, heads=heads, head_dim=dim, bias=b, validate_group=False)
        for rt in runtimes
    ]
    outs = mega_up.emulated_peer_write(prepared, xs)
    assert outs[0].shape == (1, up * seq, heads // up, dim)
    # exchange + permutation against the unfused path with cuBLAS as the GEMM
    dense = [F.linear(x.view(seq, hidden), w, b) for x in xs]
    shard = hidden // up
    for rank in range(up):
        want = torch.cat([d[:, rank * shard : (rank + 1) * shard] for d in dense], dim=0)
        assert torch.equal(outs[rank].view(up * seq, shard), want)
    # GEMM values against the CPU oracle (exact integers), sampled rows of rank 0's product
    rows = np.r_[0:64, seq - 64 : seq]
    want = oracle.linear(h.to_host(xs[up - 1].view(seq, hidden))[rows], h.to_host(w), h.to_host(b), use_c=False)
    got = h.to_host(outs[0].view(up, seq, shard)[up - 1])[rows]
    assert np.array_equal(got, want[:, :shard])
    # ---- O projection: pull
    head_xs = [h.seeded((1, up * seq, heads // up, dim), 200 + r, ints=True) for r in range(up)]
    pulls = [
        mega_up.prepare_headshard_pull_gemm_bshd(w, rt, batch=1, sequence=seq, heads=heads, head_dim=dim, bias=b, validate_group=False)
        for rt in runtimes
    ]
    results = mega_up.emulated_pull(pulls, head_xs)
    torch.cuda.synchronize()
    runtimes[0].check_status()
    for rank in range(up):
        mat = torch.cat([hx.view(up, seq, shard)[rank] for hx in head_xs], dim=1)
        assert torch.equal(pulls[rank].materialized_input, mat)
        assert torch.equal(results[rank].view(seq, hidden), F.linear(mat, w, b))
        assert results[rank].data_ptr() == pulls[rank].output_2d.data_ptr()  # aliases the reusable buffer
    want = oracle.linear(h.to_host(pulls[0].materialized_input)[rows], h.to_host(w), h.to_host(b), use_c=False)
    assert np.array_equal(h.to_host(results[0].view(seq, hidden))[rows], want)


def test_llama8b_fused_qkv_sbhd_peer_write() -> None:
    """Llama-3-8B-shaped fused QKV at U=8: W[6144,4096], no bias, SBHD, S_local=8192, B=1."""

    up, seq, heads, dim = 8, 8192, 32, 128
    runtimes = _group(up, 6144, seq)
    w = h.seeded((6144, 4096), 3, ints=False, scale=1 / 64)
    xs = [h.seeded((seq, 1, heads, dim), 300 + r, ints=False) for r in range(up)]
    prepared = [
        mega_up.prepare_peer_write_gemm_sbhd(w, rt, sequence=seq, batch=1, heads=heads, head_dim=dim, validate_group=False)
        for rt in runtimes
    ]
    outs = mega_up.emulated_peer_write(prepared, xs)
    assert outs[0].shape == (up * seq, 1, 48 // up, dim)
    shard = 6144 // up
    for rank in (0, 5):
        want = torch.cat([F.linear(x.view(seq, 4096), w)[:, rank * shard : (rank + 1) * shard] for x in xs], dim=0)
        assert torch.equal(outs[rank].view(up * seq, shard), want)


def test_llama70b_o_projection_thd_layout_pull() -> None:
    """Llama-3-70B-shaped O projection: W[8192,8192], U=8, T_local=16384 of seeded
    variable-length samples (512..4096, last truncated), THDLayout row gather."""

    up, tokens, heads, dim = 8, 16384, 64, 128
    gen = torch.Generator().manual_seed(4)
    cu = [0]
    while cu[-1] < tokens:
        cu.append(min(tokens, cu[-1] + int(torch.randint(512, 4097, (1,), generator=gen))))
    runtimes = _group(up, 8192, tokens)
    layouts = [mega_up.prepare_thd_layout(cu, rt) for rt in runtimes]
    assert layouts[0].cu_seqlens_out == tuple(up * v for v in cu)
    w = h.seeded((8192, 8192), 5, ints=True, lo=-1, hi=2)
    head_xs = [h.seeded((up * tokens, heads // up, dim), 400 + r, ints=True) for r in range(up)]
    pulls = [
        mega_up.prepare_headshard_pull_gemm_thd(w, rt, heads=heads, head_dim=dim, layout=lay, validate_group=False)
        for rt, lay in zip(runtimes, layouts)
    ]
    results = mega_up.emulated_pull(pulls, head_xs)
    torch.cuda.synchronize()
    runtimes[0].check_status()
    shard = 8192 // up
    host_layout = oracle.thd_layout(cu, up)
    assert np.array_equal(layouts[0].to_source_major_index.cpu().numpy(), host_layout["to_source_major_index"])
    for rank in (0, 3, 7):
        # slice-by-slice split of every source's packed input, then the gather
        staged = [oracle.split_thd(h.to_host(hx.view(up * tokens, shard)), cu, up)[rank] for hx in head_xs]
        mat = np.concatenate(staged, axis=1)
        assert np.array_equal(h.to_host(pulls[rank].materialized_input), mat)
        rows = np.r_[0:96, tokens - 96 : tokens]
        want = oracle.linear(mat[rows], h.to_host(w), None, use_c=False)
        assert np.array_equal(h.to_host(results[rank].view(tokens, 8192))[rows], want)
        assert torch.equal(results[rank].view(tokens, 8192), F.linear(pulls[rank].materialized_input, w))


def test_shape_edge_sweep() -> None:
    """Edge shapes: (a) 2304 wide, U=2, B=4 strided copies; (b) 2048, D=64,
    U=8; (c) W[1024,4096], U=8, 64 rows (cuBLAS split-K tolerance case)."""

    cases = [
        (2, 4, 128, 2304, 2304, 128), (8, 1, 1024, 2048, 2048, 64), (8, 1, 64, 1024, 4096, 128),
    ]
    for up, batch, seq, n, k, dim in cases:
        runtimes = _group(up, n, batch * seq)
        w = h.seeded((n, k), 6, ints=False, scale=k ** -0.5)
        b = h.seeded((n,), 7, ints=False, scale=0.02)
        xs = [h.seeded((batch, seq, k // dim, dim), 500 + r, ints=False) for r in range(up)]
        prepared = [
            mega_up.prepare_peer_write_gemm_bshd(w, rt, batch=batch, sequence=seq, heads=k // dim, head_dim=dim, bias=b, validate_group=False)
            for rt in runtimes
        ]
        outs = mega_up.emulated_peer_write(prepared, xs)
        host = oracle.peer_write_bshd([h.to_host(x) for x in xs], h.to_host(w), h.to_host(b))
        shard = n // up
        for rank in range(up):
            ref = torch.stack([F.linear(x.view(batch, seq, k), w, b)[..., rank * shard : (rank + 1) * shard] for x in xs], dim=1)
            ref = ref.reshape(batch, up * seq, shard // dim, dim)
            if not torch.equal(outs[rank], ref):
                assert batch * seq < 256 and h.ulp_distance(outs[rank], ref) <= 1
            want = torch.from_numpy(host[rank]).to(h.DEVICE).to(torch.bfloat16)
            assert h.ulp_distance(outs[rank], want) <= 1  # FP32 ascending-K oracle, random values


def test_prepared_calls_reuse_buffers_and_recycle_the_workspace() -> None:
    """Two inputs through one prepared executable, an ``out=`` tensor, three pulls with
    ``workspace_epochs=2`` on alternating streams (forces a workspace recycle)."""

    up, batch, seq, heads, dim = 2, 2, 17, 8, 64
    hidden = heads * dim
    runtimes = _group(up, hidden, 64)
    w = h.seeded((hidden, hidden), 8, ints=True, lo=-1, hi=2)
    prepared = [
        mega_up.prepare_peer_write_gemm_bshd(w, rt, batch=batch, sequence=seq, heads=heads, head_dim=dim, validate_group=False)
        for rt in runtimes
    ]
    for trial in range(2):
        xs = [h.seeded((batch, seq, heads, dim), 600 + 10 * trial + r, ints=True) for r in range(up)]
        outs = [torch.empty(p.output_shape, device=h.DEVICE, dtype=torch.bfloat16) for p in prepared]
        got = mega_up.emulated_peer_write(prepared, xs, outs)
        want = oracle.peer_write_bshd([h.to_host(x) for x in xs], h.to_host(w), None)
        for rank in range(up):
            assert got[rank] is outs[rank]
            assert np.array_equal(h.to_host(got[rank]), want[rank])
    pulls = [
        mega_up.prepare_headshard_pull_gemm_bshd(w, rt, batch=batch, sequence=seq, heads=heads, head_dim=dim, workspace_epochs=2, validate_group=False)
        for rt in runtimes
    ]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for trial in range(3):
        head_xs = [h.seeded((batch, up * seq, heads // up, dim), 700 + 10 * trial + r, ints=True) for r in range(up)]
        torch.cuda.synchronize()
        with torch.cuda.stream(streams[trial % 2]):
            results = mega_up.emulated_pull(pulls, head_xs)
        torch.cuda.synchronize()
        want = oracle.pull_bshd([h.to_host(x) for x in head_xs], h.to_host(w), None)
        for rank in range(up):
            assert np.array_equal(h.to_host(pulls[rank].materialized_input).reshape(want[rank][0].shape), want[rank][0])
            assert np.array_equal(h.to_host(results[rank]), want[rank][1])
        assert pulls[0].compiled.epoch == (trial % 2) + 1  # recycled before the third call
    runtimes[0].check_status()


def test_contract_violations_raise_value_errors() -> None:
    up, hidden = 2, 512
    runtime = _group(up, hidden, 64)[0]
    w = torch.zeros(hidden, hidden, device=h.DEVICE, dtype=torch.bfloat16)
    kw = dict(batch=1, sequence=16, heads=8, head_dim=64, validate_group=False)
    prepared = mega_up.prepare_peer_write_gemm_bshd(w, runtime, **kw)
    assert prepared.output_shape == (1, 32, 4, 64) and (prepared.in_features, prepared.out_features) == (512, 512)
    with pytest.raises(ValueError, match="expects"):
        prepared(torch.zeros(1, 8, 8, 64, device=h.DEVICE, dtype=torch.bfloat16), validate_group=False)
    with pytest.raises(ValueError, match="contiguous BF16"):
        prepared(torch.zeros(1, 16, 8, 64, device=h.DEVICE), validate_group=False)
    with pytest.raises(ValueError, match="out must be"):
        prepared(torch.zeros(1, 16, 8, 64, device=h.DEVICE, dtype=torch.bfloat16), out=torch.zeros(3, device=h.DEVICE), validate_group=False)
    with pytest.raises(ValueError, match="contiguous BF16"):  # transposed rectangular weight
        mega_up.prepare_peer_write_gemm_bshd(torch.zeros(512, 1024, device=h.DEVICE, dtype=torch.bfloat16).t()[:, :512], runtime, **kw)
    with pytest.raises(ValueError, match="bias must have shape"):
        mega_up.prepare_peer_write_gemm_bshd(w, runtime, bias=torch.zeros(4, device=h.DEVICE, dtype=torch.bfloat16), **kw)
    with pytest.raises(ValueError, match="exceed the arena"):
        mega_up.prepare_peer_write_gemm_bshd(w, runtime, **(kw | {"sequence": 65}))
    with pytest.raises(ValueError, match="heads=3 must be divisible"):
        mega_up.prepare_headshard_pull_gemm_bshd(w, runtime, batch=1, sequence=4, heads=3, head_dim=64, validate_group=False)
    with pytest.raises(ValueError, match="workspace_epochs"):
        mega_up.prepare_headshard_pull_gemm_bshd(w, runtime, batch=1, sequence=4, heads=8, head_dim=64, workspace_epochs=0, validate_group=False)
    with pytest.raises(ValueError, match="TypeError: layout must be a THDLayout"):
        mega_up.prepare_peer_write_gemm_thd(w, runtime, heads=8, head_dim=64, layout=object(), validate_group=False)
    with pytest.raises(ValueError, match="tokens is required"):
        mega_up.prepare_peer_write_gemm_thd(w, runtime, heads=8, head_dim=64, validate_group=False)
    # a lease cannot be re-entered
    with runtime.lease():
        with pytest.raises(RuntimeError, match="re-entered"):
            with runtime.lease():
                pass
    with pytest.raises(ValueError, match="hidden"):
        mega_up.initialize_emulated_group(2, hidden=384, max_rows=8)
