"""The kernels behind the Bomipel parts, each alone against its plain statement
(``kernel_references``): the general store kernel with its two rotation layouts and the value
mixing, attention with kept first positions and with values read out of the key rows, the latent
store kernels, the per-head products, the router, dispatch, the routed products, the combine and
the soft cap on logits.
"""
from __future__ import annotations

import pytest
import torch

import kernel_references as ref
from test_gpu_kernels import _attention_case, status, tol

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def close(got, want, dtype):
    torch.testing.assert_close(got, want, **(dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else tol(dtype)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, key, value, pairs, interleaved, mix", [
    (4, 2, 16, 24, 4, True, "source"), (3, 1, 48, 32, 24, True, "blend"), (5, 5, 40, 8, 3, False, None),
    (2, 1, 64, 64, 32, False, "blend"), (1, 1, 200, 72, 50, True, None), (2, 2, 8, 8, 0, True, "source"),
])
def test_store_with_rotation_and_value_mixing(dev, dtype, heads, kv_heads, key, value, pairs, interleaved, mix):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(2)
    tokens, page, pages = 13, 4, 9
    width = (heads + kv_heads) * key + kv_heads * value
    for splits in (1, 3):
        shape = (tokens, width) if splits == 1 else (splits, tokens, width)
        qkv = torch.randn(shape, generator=gen).to(dtype if splits == 1 else torch.float32).to(dev)
        slots = torch.randperm(page * pages, generator=gen)[:tokens].to(torch.int32)
        slots[3] = -1
        slots = slots.to(dev)
        positions = torch.randint(0, 5000, (tokens,), generator=gen).to(torch.int32).to(dev)
        inv_freq = (10000.0 ** (-torch.arange(pairs) / max(pairs, 1))).float().to(dev)
        fraction = torch.tensor([0.3], device=dev)
        results = []
        for fn in (ops.qkv_norm_store, ref.qkv_norm_store):
            q = torch.zeros((tokens, heads, key), dtype=dtype, device=dev)
            k = torch.zeros((pages, kv_heads, page, key), dtype=dtype, device=dev)
            v = torch.zeros((pages, kv_heads, page, value), dtype=dtype, device=dev)
            shared = torch.linspace(-1, 1, tokens * kv_heads * value, device=dev).reshape(tokens, -1).contiguous()
            fn(qkv, None, slots, q, k, v, heads, kv_heads, key, value, None, status(dev), positions=positions,
               inv_freq=inv_freq, interleaved=interleaved, value_mix=mix, shared_values=shared, mix=fraction)
            results.append((q, k, v, shared))
        for got, want in zip(*results):
            if got is results[0][3] and mix == "source":    # the row of the token without a slot is not written
                got, want = got[slots >= 0], want[slots >= 0]
            close(got, want, got.dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, value, page_size, window, keep", [
    (4, 2, 16, 16, 4, 5, 2), (3, 1, 48, 32, 8, 9, 9), (6, 2, 64, 64, 16, 20, 1), (2, 2, 24, 8, 16, 3, 40),
])
def test_attention_with_kept_first_positions(dev, dtype, heads, kv_heads, size, value, page_size, window, keep):
    from einf_b200 import ops

    requests = [(0, 30), (37, 1), (12, 7), (0, 1), (64, 2)]
    (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, window)
    v = v[..., :value].contiguous()
    out = torch.empty((q.shape[0], heads, value), dtype=dtype, device=dev)
    want = torch.empty_like(out)
    st = status(dev)
    ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale, window, st, keep_first=keep)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st, keep_first=keep)
    assert int(st) == 0
    close(out, want, dtype)
    # the kept positions matter: without them the rows far from the start differ
    ops.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st)
    assert (out - want).abs().max() > 1e-2


@pytest.mark.parametrize("size, page_size", [(64, 16), (128, 16), (64, 8), (128, 64), (64, 128)])
@pytest.mark.parametrize("window, keep", [(40, 4), (200, 130), (128, 128), (17, 300), (1, 1), (500, 16), (64, 0)])
def test_tensor_core_attention_with_kept_first_positions(dev, size, page_size, window, keep):
    """The tcgen05 prefill and decode kernels behind ``windowed_attention``: portions that start at 0,
    inside the kept positions, inside the first window and far beyond it, and single tokens at
    every distance, against the plain statement."""
    from einf_b200 import ops

    heads, kv_heads = 6, 2
    portions = [(0, 300), (3, 130), (700, 260), (129, 5), (1500, 128)]
    singles = [(0, 1), (keep, 1), (max(keep - 1, 0), 1), (window + keep, 1), (window + keep + 1, 1), (1000, 1), (2047, 1),
               (127, 1), (128, 1)]
    for requests in (portions, singles, portions[:2] + singles[:5]):
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, torch.bfloat16, heads, kv_heads, size, page_size,
                                                                requests, window)
        tiles, single_tokens, cursor = [], [], 0
        for index, (start, count) in enumerate(requests):
            if count == 1:
                single_tokens.append(cursor)
            else:
                for first in range(0, count, 128):
                    tiles.append([index, cursor + first, min(128, count - first), start + first])
            cursor += count
        q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev).reshape(-1, 4)
        token_list = torch.tensor(single_tokens, dtype=torch.int32, device=dev) if tiles else None
        out = torch.zeros_like(q)
        want = torch.zeros_like(q)
        st = status(dev)
        ops.windowed_attention(q, k, v, table, seq, pos, q_tiles, token_list, out, scale, window, keep, st,
                               max_context=max(s + c for s, c in requests), cached_before=max(s for s, _ in requests))
        ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st, keep_first=keep)
        assert int(st) == 0
        close(out, want, torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, row, rank, page_size", [(3, 32, 24, 4), (16, 80, 64, 16), (5, 576, 512, 16), (1, 10, 8, 8)])
def test_attention_with_values_in_the_key_rows(dev, dtype, heads, row, rank, page_size):
    from einf_b200 import ops

    requests = [(0, 21), (40, 1), (5, 3)]
    (q, k, _, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, 1, row, page_size, requests, None)
    out = torch.empty((q.shape[0], heads, rank), dtype=dtype, device=dev)
    want = torch.empty_like(out)
    st = status(dev)
    ops.paged_attention_generic(q, k, None, table, seq, pos, out, scale, None, st, values_in_keys=rank)
    ref.paged_attention_generic(q, k, None, table, seq, pos, want, scale, None, st, values_in_keys=rank)
    assert int(st) == 0
    close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, row, rank, page_size", [(3, 32, 24, 4), (16, 80, 64, 16), (12, 576, 512, 16), (1, 10, 8, 8),
                                                         (40, 96, 64, 16), (5, 33, 7, 8), (17, 640, 600, 32)])
@pytest.mark.parametrize("splits", [1, 2, 7, 32])
def test_shared_row_decode_attention(dev, dtype, heads, row, rank, page_size, splits):
    from einf_b200 import ops

    requests = [(0, 1), (40, 1), (5, 1), (1000, 1), (31, 1), (32, 1), (255, 1)]
    (q, k, _, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, 1, row, page_size, requests, None)
    out = torch.empty((q.shape[0], heads, rank), dtype=dtype, device=dev)
    want = torch.empty_like(out)
    st = status(dev)
    ops.latent_decode_attention(q, k, table, seq, pos, out, scale, splits, st)
    ref.paged_attention_generic(q, k, None, table, seq, pos, want, scale, None, st, values_in_keys=rank)
    assert int(st) == 0
    close(out, want, dtype)
    table[3, 2] = 10_000                      # a page outside the pool is reported, not read
    ops.latent_decode_attention(q, k, table, seq, pos, out, scale, splits, st)
    assert int(st) == ops.STATUS_BAD_PAGE and torch.isfinite(out).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_rank, kv_rank, rot, interleaved", [(20, 24, 8, False), (96, 64, 32, False), (0, 512, 64, False), (8, 8, 2, True)])
def test_latent_down_store(dev, dtype, q_rank, kv_rank, rot, interleaved):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(3)
    tokens, page, pages = 9, 4, 7
    width = q_rank + kv_rank + rot
    for splits in (1, 2):
        shape = (tokens, width) if splits == 1 else (splits, tokens, width)
        down = torch.randn(shape, generator=gen).to(dtype if splits == 1 else torch.float32).to(dev)
        slots = torch.randperm(page * pages, generator=gen)[:tokens].to(torch.int32)
        slots[2] = -1
        slots = slots.to(dev)
        positions = torch.randint(0, 3000, (tokens,), generator=gen).to(torch.int32).to(dev)
        inv_freq = (5000.0 ** (-torch.arange(rot // 2) / (rot // 2))).float().to(dev)
        wq = (1 + 0.1 * torch.randn(q_rank, generator=gen)).to(dev)
        wk = (1 + 0.1 * torch.randn(kv_rank, generator=gen)).to(dev)
        results = []
        for fn in (ops.latent_down_store, ref.latent_down_store):
            q_latent = torch.zeros((tokens, q_rank), dtype=dtype, device=dev)
            cache = torch.zeros((pages, 1, page, kv_rank + rot), dtype=dtype, device=dev)
            fn(down, q_rank, kv_rank, rot, wq, wk, 1e-5, positions, inv_freq, interleaved, slots, q_latent, cache,
               status(dev))
            results.append((q_latent, cache))
        for got, want in zip(*results):
            close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rot, rank", [(3, 16, 8, 24), (6, 64, 32, 64), (1, 8, 2, 8), (16, 128, 64, 512)])
def test_latent_q_store_and_per_head_products(dev, dtype, heads, dim, rot, rank):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(4)
    tokens = 7
    positions = torch.randint(0, 3000, (tokens,), generator=gen).to(torch.int32).to(dev)
    inv_freq = (5000.0 ** (-torch.arange(rot // 2) / (rot // 2))).float().to(dev)
    weight = (torch.randn((heads, rank, dim), generator=gen) * dim ** -0.5).to(dtype).to(dev)
    for splits in (1, 3):
        shape = (tokens, heads * (dim + rot)) if splits == 1 else (splits, tokens, heads * (dim + rot))
        q = torch.randn(shape, generator=gen).to(dtype if splits == 1 else torch.float32).to(dev)
        results = []
        for module in (ops, ref):
            plain = torch.zeros((tokens, heads, dim), dtype=dtype, device=dev)
            full = torch.zeros((tokens, heads, rank + rot), dtype=dtype, device=dev)
            module.latent_q_store(q, positions, inv_freq, False, plain, full)
            module.per_head_project(plain, weight, full[:, :, :rank])
            results.append((plain, full))
        for got, want in zip(*results):
            close(got, want, dtype)


@pytest.mark.parametrize("experts, top, score, renormalise", [
    (8, 1, "sigmoid", False), (5, 3, "sigmoid", False), (64, 6, "softmax", True), (1, 1, "sigmoid", False),
    (3, 3, "softmax", False), (200, 8, "sigmoid", True),
])
def test_router_topk(dev, experts, top, score, renormalise):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(5)
    logits = (torch.randn((37, experts), generator=gen) * 2).to(dev)
    logits[3, : min(experts, 4)] = 1.5          # ties go to the lower index
    results = []
    for fn in (ops.router_topk, ref.router_topk):
        ids = torch.zeros((37, top), dtype=torch.int32, device=dev)
        weights = torch.zeros((37, top), dtype=torch.float32, device=dev)
        fn(logits, top, score, renormalise, ids, weights)
        results.append((ids, weights))
    assert torch.equal(results[0][0], results[1][0])
    torch.testing.assert_close(results[0][1], results[1][1], rtol=1e-5, atol=1e-6)
    # the same logits as three partial sums
    parts = torch.stack([logits * 0.5, logits * 0.25, logits * 0.25])
    ids = torch.zeros((37, top), dtype=torch.int32, device=dev)
    weights = torch.zeros((37, top), dtype=torch.float32, device=dev)
    ops.router_topk(parts, top, score, renormalise, ids, weights)
    assert torch.equal(ids, results[1][0])
    torch.testing.assert_close(weights, results[1][1], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, hidden, inter, experts, top, on_input", [
    (1, 32, 24, 6, 2, True), (50, 48, 40, 4, 2, True), (300, 64, 96, 8, 1, False), (17, 40, 16, 1, 1, True),
    (64, 128, 72, 16, 4, False), (9, 256, 130, 3, 3, True), (700, 192, 200, 5, 2, True), (2100, 64, 64, 2, 1, True),
])
def test_routed_feed_forward_steps(dev, dtype, tokens, hidden, inter, experts, top, on_input):
    """Dispatch, the two routed products and the combine, against their plain statements; rows of an
    expert may stand in any order, so sorted tensors are compared through ``place``."""
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(6)
    x = torch.randn((tokens, hidden), generator=gen).to(dtype).to(dev)
    ids = torch.stack([torch.randperm(experts, generator=gen)[:top] for _ in range(tokens)]).to(torch.int32).to(dev)
    weights = torch.rand((tokens, top), generator=gen).to(dev)
    w1 = (torch.randn((experts, 2 * inter, hidden), generator=gen) * hidden ** -0.5).to(dtype).to(dev)
    w2 = (torch.randn((experts, hidden, inter), generator=gen) * inter ** -0.5).to(dtype).to(dev)
    addend = torch.randn((3, tokens, hidden), generator=gen).to(dev)
    outs = []
    st = status(dev)                   # with it, bfloat16 products take the tcgen05 kernel
    for module in (ops, ref):
        work = torch.zeros(3 * experts + 1, dtype=torch.int32, device=dev)
        place = torch.zeros((tokens, top), dtype=torch.int32, device=dev)
        sorted_x = torch.zeros((tokens * top, hidden), dtype=dtype, device=dev)
        offsets = module.moe_dispatch(x, ids, weights, experts, on_input, work, place, sorted_x)
        # every pair lies inside its expert's range, and no two share a row
        flat_place, flat_ids = place.reshape(-1).long(), ids.reshape(-1).long()
        assert torch.equal(torch.sort(flat_place).values, torch.arange(tokens * top, device=dev))
        assert bool(((flat_place >= offsets[flat_ids]) & (flat_place < offsets[flat_ids + 1])).all())
        gate_up = torch.zeros((tokens * top, 2 * inter), dtype=dtype, device=dev)
        module.moe_gemm(sorted_x, w1, offsets, gate_up, st)
        hidden_rows = torch.zeros((tokens * top, inter), dtype=dtype, device=dev)
        module.silu_mul(gate_up, hidden_rows)
        y = torch.zeros((tokens * top, hidden), dtype=dtype, device=dev)
        module.moe_gemm(hidden_rows, w2, offsets, y, st)
        out = torch.zeros((tokens, hidden), dtype=torch.float32, device=dev)
        module.moe_combine(y, ids, place, weights, not on_input, addend, out, experts)
        if module is ops and dtype == torch.bfloat16 and inter % 8 == 0:
            # the same with K cut three ways: partial sums that the combine adds up
            cut = ops.gemm_tcgen05_splits(inter, 3)
            parts = torch.zeros((cut, tokens * top, hidden), dtype=torch.float32, device=dev)
            ops.moe_gemm(hidden_rows, w2, offsets, parts, st)
            again = torch.zeros_like(out)
            ops.moe_combine(parts, ids, place, weights, not on_input, addend, again, experts)
            close(again, out, torch.bfloat16)
        outs.append((sorted_x[flat_place], gate_up[flat_place], y[flat_place], out, offsets.clone()))
    assert torch.equal(outs[0][4], outs[1][4]) and int(st) == 0
    for got, want in zip(outs[0][:4], outs[1][:4]):
        close(got, want, got.dtype if got.dtype == torch.bfloat16 else (torch.float32 if dtype == torch.float32 else torch.bfloat16))


def test_softcap(dev):
    from einf_b200 import ops

    values = (torch.randn((5, 1000), generator=torch.Generator().manual_seed(7)) * 30).to(dev)
    want = values.clone()
    ops.softcap(values, 12.5)
    ref.softcap(want, 12.5)
    torch.testing.assert_close(values, want, rtol=1e-5, atol=1e-5)
    assert float(values.abs().max()) <= 12.5
