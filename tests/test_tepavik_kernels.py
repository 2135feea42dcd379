"""The kernels behind the Tepavik mixers, each alone against its plain statement
(``kernel_references``): activations, unit-norm heads with the cache write, the
chunked and soft-capped attention (general kernel and the tcgen05 kernels), the
short convolution with its carried inputs, the recurrence with its state slots,
the gated norm.
"""
from __future__ import annotations

import random

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
@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu", "relu"])
def test_activation(dev, dtype, kind):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(1)
    for shape in ((3, 37), (65, 256), (4, 3, 40)):        # the last: split-K partial sums
        x = (torch.randn(shape, generator=gen) * 2).to(torch.float32 if len(shape) == 3 else dtype).to(dev)
        out = torch.empty(shape[-2:], dtype=dtype, device=dev)
        want = torch.empty_like(out)
        ops.activation(x, out, kind)
        ref.activation(x, want, kind)
        close(out, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, key, value, eps", [
    (4, 2, 16, 24, 1e-5), (3, 1, 64, 64, None), (5, 5, 40, 8, 1e-6), (2, 0, 128, 128, 1e-5), (1, 1, 256, 200, 1e-5),
])
def test_qkv_norm_store(dev, dtype, heads, kv_heads, key, value, eps):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(2)
    tokens, page, pages = 11, 4, 9
    width = (heads + kv_heads) * key + kv_heads * value
    for splits in (1, 3):
        shape = (tokens, width) if splits == 1 else (splits, tokens, width)
        qkv = torch.randn(shape, generator=gen).to(dtype if splits == 1 else torch.float32).to(dev)
        bias = torch.randn(width, generator=gen).to(dev)
        slots = torch.randperm(page * pages, generator=gen)[:tokens].to(torch.int32)
        slots[3] = -1
        slots = slots.to(dev)
        outs = []
        for fn in (ops.qkv_norm_store, ref.qkv_norm_store):
            q = torch.zeros((tokens, heads, key), dtype=dtype, device=dev)
            k = torch.zeros((pages, max(kv_heads, 1), page, key), dtype=dtype, device=dev)
            v = torch.zeros((pages, max(kv_heads, 1), page, value), dtype=dtype, device=dev)
            st = status(dev)
            fn(qkv, bias, slots if kv_heads else None, q, k if kv_heads else None, v if kv_heads else None, heads,
               kv_heads, key, value, eps, st)
            assert int(st) == 0
            outs.append((q, k, v))
        for got, want in zip(*outs):
            close(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, size, value, page_size, chunk, softcap", [
    (4, 2, 16, 24, 4, 7, 5.0), (3, 1, 32, 8, 8, 1, None), (6, 2, 64, 64, 16, 50, 30.0), (2, 2, 20, 36, 16, 16, 2.0),
    (7, 1, 128, 256, 8, 33, None),
])
def test_general_attention_with_chunks_caps_and_value_sizes(dev, dtype, heads, kv_heads, size, value, page_size, chunk,
                                                            softcap):
    from einf_b200 import ops

    requests = [(0, 1), (0, 2 * page_size), (chunk - 1, 3), (3 * chunk - 2, 5), (chunk * 4, 1), (chunk * 4 - 1, 1),
                (70, 1), (0, 37)]
    (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, dtype, heads, kv_heads, size, page_size, requests, None)
    v = torch.randn((k.shape[0], kv_heads, page_size, value), generator=torch.Generator().manual_seed(3)).to(dtype).to(dev)
    out = torch.empty((q.shape[0], heads, value), dtype=dtype, device=dev)
    want = torch.empty_like(out)
    st = status(dev)
    ops.paged_attention_generic(q, k, v, table, seq, pos, out, scale * 3, None, st, chunk=chunk, softcap=softcap)
    ref.paged_attention_generic(q, k, v, table, seq, pos, want, scale * 3, None, st, chunk=chunk, softcap=softcap)
    assert int(st) == 0
    close(out, want, dtype)


@pytest.mark.parametrize("first_case", [0, 12])
def test_tcgen05_attention_with_chunks_and_caps(dev, first_case):
    """Seeded random launches of the tcgen05 prefill and decode kernels with a chunked mask and a
    soft cap: chunk sizes that are no multiple of a page or a tile, portions that start and end
    anywhere (just inside and just outside a chunk's edge among them), single tokens at a chunk's
    first and last position, keys scaled so that the cap bites; against the general kernel."""
    from einf_b200 import ops

    for case in range(first_case, first_case + 12):
        rng = random.Random(1000 + case)
        size, page_size = rng.choice([64, 128]), rng.choice([8, 16, 32, 64, 128])
        kv_heads, group = rng.choice([1, 2, 4]), rng.choice([1, 2, 3, 8])
        chunk = rng.choice([1, 5, 50, 128, 200, 777, 1024, None])
        softcap = rng.choice([None, 2.0, 20.0, 50.0])
        window = rng.choice([None, None, None, 90])
        edge = chunk or 100
        requests = []
        for _ in range(rng.randint(1, 4)):
            start = rng.choice([0, edge - 1, edge, 3 * edge - 2, rng.randrange(1, 200), rng.randrange(200, 2500)])
            requests.append((start, rng.choice([2, 3, edge + 1, rng.randrange(2, 140), rng.randrange(100, 600)])))
        singles = [(rng.choice([edge - 1, edge, 2 * edge + 1, 4 * edge - 1, rng.randrange(1, 3000)]), 1)
                   for _ in range(rng.randint(1, 5))]
        layout = rng.choice(["shuffled", "runs"])
        heads = kv_heads * group
        (q, k, v, table, seq, pos), scale, _ = _attention_case(dev, torch.bfloat16, heads, kv_heads, size, page_size,
                                                               requests + singles, window, seed=case, layout=layout)
        k.mul_(rng.choice([1.0, 3.0, 8.0]))
        tiles, cursor = [], 0
        for r, (start, q_len) in enumerate(requests):
            for first in range(0, q_len, ops.Q_TILE):
                tiles.append((r, cursor + first, min(ops.Q_TILE, q_len - first), start + first))
            cursor += q_len
        q_tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        single_tokens = torch.arange(cursor, cursor + len(singles), dtype=torch.int32, device=dev)
        st = status(dev)
        want = torch.empty_like(q)
        ops.paged_attention_generic(q, k, v, table, seq, pos, want, scale, window, st, chunk=chunk, softcap=softcap)
        out = torch.full_like(q, float("nan"))
        ops.paged_prefill_attention(q, k, v, table, q_tiles, out, scale, window, st, use_tcgen05=True,
                                    prefill_cluster=rng.randrange(0, 5), cached_before=max(s for s, _ in requests),
                                    chunk=chunk, softcap=softcap)
        ops.paged_decode_attention_tcgen05(q, k, v, table, seq, pos, out, scale, window, rng.choice([1, 2, 4, 8]), st,
                                           single_tokens, chunk=chunk, softcap=softcap)
        assert int(st) == 0, case
        torch.testing.assert_close(out, want, **tol(torch.bfloat16), msg=lambda m: f"case {case}: {m}")


def _packed(lengths, dev):
    starts = [0]
    seq = []
    for r, n in enumerate(lengths):
        starts.append(starts[-1] + n)
        seq += [r] * n
    return (torch.tensor(starts, dtype=torch.int32, device=dev), torch.tensor(seq, dtype=torch.int32, device=dev))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channels, taps, heads", [(24, 4, 3), (40, 2, 0), (7, 5, 2), (64, 1, 1), (130, 16, 4)])
def test_conv_silu_carries_its_inputs(dev, dtype, channels, taps, heads):
    """Portions of 1, 2 and many tokens (shorter and longer than the kernel), a request without a
    slot, slots in any order, two steps in a row on the same states."""
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(4)
    slots = torch.tensor([2, -1, 0, 3, 1], dtype=torch.int32, device=dev)
    states = [torch.randn((5, 9 + (taps - 1) * channels), generator=gen).to(dev) for _ in range(1)] * 1
    state_got, state_want = states[0].clone(), states[0].clone()
    for lengths in ((1, 2, 9, 1, taps), (3, 1, 1, 2 * taps + 1, 2)):
        q_start, seq = _packed(lengths, dev)
        tokens = sum(lengths)
        wide = torch.randn((tokens, 5 + channels + heads), generator=gen).to(dtype).to(dev)
        x, dt_raw = wide[:, 5:5 + channels], wide[:, 5 + channels:]
        weight = torch.randn((channels, taps), generator=gen).to(dev)
        bias = torch.randn(channels, generator=gen).to(dev)
        dt_bias, a_log = torch.randn(heads, generator=gen).to(dev), torch.randn(heads, generator=gen).to(dev)
        results = []
        for fn, state in ((ops.conv_silu, state_got), (ref.conv_silu, state_want)):
            out = torch.empty((tokens, channels), dtype=dtype, device=dev)
            dt, decay = torch.empty((tokens, heads), device=dev), torch.empty((tokens, heads), device=dev)
            view = state[:, 9:].view(5, taps - 1, channels)
            if heads:
                fn(x, weight, bias, view, seq, q_start, slots, out, dt_raw, dt_bias, a_log, dt, decay)
            else:
                fn(x, weight, bias, view, seq, q_start, slots, out)
            results.append((out, dt, decay) if heads else (out,))
        for got, want in zip(*results):
            close(got, want, dtype)
        torch.testing.assert_close(state_got, state_want, rtol=0, atol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, groups, dim, vdim, per_token, silu", [
    (3, 3, 24, 16, False, True), (4, 2, 8, 12, True, False), (2, 1, 128, 64, True, False), (1, 1, 40, 8, False, True),
    (6, 3, 20, 8, True, False), (2, 2, 16, 130, False, False), (8, 8, 64, 64, False, True), (2, 1, 300, 20, True, False),
])
@pytest.mark.parametrize("rows, segment_len, columns", [(0, None, 0), (4, 3, 1), (8, None, 1), (16, 16, 2), (0, 5, 0),
                                                        (16, None, 2)])
def test_linear_recurrence_keeps_its_state(dev, dtype, heads, groups, dim, vdim, per_token, silu, rows, segment_len,
                                           columns):
    """Two steps on the same slots (one request without a slot), portions of one token and of many,
    an empty request; inputs as columns of a wider matrix; every number of rows per thread; portions
    cut into segments that run side by side; outputs and states against the plain loop."""
    if rows and 32 * rows < dim:
        pytest.skip("too few rows per thread for this state")
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(5)
    slots = torch.tensor([1, -1, 3, 0], dtype=torch.int32, device=dev)
    base = torch.randn((4, 5 + heads * dim * vdim), generator=gen).to(dev)
    state_got, state_want = base.clone(), base.clone()
    for lengths in ((1, 3, 17, 0), (40, 1, 1, 2), (1, 1, 1, 1)):     # the last: a step of single tokens
        q_start, _ = _packed(lengths, dev)
        tokens = sum(lengths)
        wide = (torch.randn((tokens, 8 + 2 * groups * dim + heads * vdim), generator=gen) * 0.5).to(dtype).to(dev)
        q, k = wide[:, 8:8 + groups * dim], wide[:, 8 + groups * dim:8 + 2 * groups * dim]
        v = wide[:, 8 + 2 * groups * dim:]
        kwargs = dict(silu_inputs=silu)
        if per_token:
            kwargs.update(token_decay=torch.rand((tokens, heads), generator=gen).to(dev),
                          token_scale=torch.rand((tokens, heads), generator=gen).to(dev),
                          skip=torch.randn(heads, generator=gen).to(dev))
        else:
            kwargs.update(head_decay=torch.rand(heads, generator=gen).to(dev))
        ys = []
        for fn, state in ((ops.linear_recurrence, state_got), (ref.linear_recurrence, state_want)):
            y = torch.zeros((tokens, heads * vdim), device=dev)
            fn(q, k, v, state[:, 5:].view(4, heads, dim, vdim), q_start, slots, y, heads, groups, dim, vdim,
               max_q_len=max(lengths), rows=rows, segment_len=segment_len, columns=columns, **kwargs)
            ys.append(y)
        torch.testing.assert_close(ys[0], ys[1], rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(state_got, state_want, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, parts, gate_first, kind", [
    (48, 2, True, "silu"), (64, 1, False, "sigmoid"), (600, 3, True, "silu"), (40, 40, False, "silu"),
])
def test_gated_norm(dev, dtype, width, parts, gate_first, kind):
    from einf_b200 import ops

    gen = torch.Generator().manual_seed(6)
    tokens = 9
    y = torch.randn((tokens, width), generator=gen).to(dev)
    wide = torch.randn((tokens, width + 24), generator=gen).to(dtype).to(dev)
    gate = wide[:, 8:8 + width]
    weight = torch.randn(width, generator=gen).to(dev)
    out, want = (torch.empty((tokens, width), dtype=dtype, device=dev) for _ in range(2))
    ops.gated_norm(y, gate, weight, out, parts, 1e-5, gate_first, kind)
    ref.gated_norm(y, gate, weight, want, parts, 1e-5, gate_first, kind)
    close(out, want, dtype)
