"""The Bomipel decoder stated plainly from its equations: float64, one function per mechanism,
whole sequences with explicit masks, nothing of the package imported.

``forward(config, weights, tokens)`` gives the logits of every position of one sequence (and the
residual stream after every layer); the engine's tests compare against it.

A layer is parallel: ``x <- x + mixer(n) + ff(n)`` with ``n = rms(x) * w`` read by both.  Two
mixers (grouped-query attention with a sliding window that keeps the first tokens, partial
interleaved rotary positions with an optional wavelength-dependent scaling, and values mixed with
those of the first such layer; latent attention with low-rank queries and one cached latent and
rotated key part for all heads) and a routed feed-forward whose weights scale the experts' inputs.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rotary_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with ``scaling`` long wavelengths are stretched by ``factor``,
    short ones kept, and those between blended."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_pairs(x, positions, frequencies, first, second):
    """Rotate the pairs (x[..., first[i]], x[..., second[i]]) by positions * frequencies[i]; x is [T, heads, D]."""
    angles = positions.to(F64)[:, None] * frequencies[None, :]          # [T, pairs]
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    u, v = x[..., first], x[..., second]
    out = x.clone()
    out[..., first] = u * cos - v * sin
    out[..., second] = v * cos + u * sin
    return out


def rotate_interleaved(x, positions, frequencies):
    pairs = frequencies.shape[0]
    index = torch.arange(pairs)
    return rotate_pairs(x, positions, frequencies, 2 * index, 2 * index + 1)


def rotate_halves(x, positions, frequencies):
    pairs = frequencies.shape[0]
    index = torch.arange(pairs)
    return rotate_pairs(x, positions, frequencies, index, index + pairs)


def visible(length, size=None, keep_first=0):
    """[i, j] true where position i sees position j."""
    i = torch.arange(length)[:, None]
    j = torch.arange(length)[None, :]
    mask = j <= i
    if size is not None:
        mask = mask & ((i - j < size) | (j < keep_first))
    return mask


def softmax_attention(q, k, v, mask, scale):
    """q [T, H, D], k [T, H, D], v [T, H, V] -> [T, H, V]"""
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    scores = scores.masked_fill(~mask[None], float("-inf"))
    return torch.einsum("hij,jhv->ihv", torch.softmax(scores, dim=-1), v)


def attention_mixer(h, w, m, positions, shared):
    """``shared`` carries the values of the first value-mixing layer from layer to layer."""
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(tokens, heads, dim)
    k = (h @ w["k"].T).reshape(tokens, kv_heads, dim)
    v = (h @ w["v"].T).reshape(tokens, kv_heads, vdim)
    rot = m.get("rot")
    if rot:
        frequencies = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q = rotate_interleaved(q, positions, frequencies)
        k = rotate_interleaved(k, positions, frequencies)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = w["vmix"].reshape(())
            v = (1 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    group = heads // kv_heads
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    mask_spec = m.get("mask") or {}
    mask = visible(tokens, mask_spec.get("size"), mask_spec.get("keep_first", 0))
    mixed = softmax_attention(q, k, v, mask, m["scale"])
    return mixed.reshape(tokens, heads * vdim) @ w["o"].T


def latent_attention_mixer(h, w, m, positions, eps):
    tokens = h.shape[0]
    heads, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    query_latent = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (query_latent @ w["uq"].T).reshape(tokens, heads, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    down = h @ w["dkv"].T
    latent = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = down[:, rank:].reshape(tokens, 1, rot_dim)
    frequencies = rotary_frequencies(m["rot"]["base"], m["rot"]["dims"], m["rot"].get("scaling"))
    q_rot = rotate_halves(q_rot, positions, frequencies)
    k_rot = rotate_halves(k_rot, positions, frequencies)
    k_plain = (latent @ w["uk"].T).reshape(tokens, heads, dim)
    v = (latent @ w["uv"].T).reshape(tokens, heads, vdim)
    q_full = torch.cat([q_plain, q_rot], dim=-1)
    k_full = torch.cat([k_plain, k_rot.expand(tokens, heads, rot_dim)], dim=-1)
    mixed = softmax_attention(q_full, k_full, v, visible(tokens), m["scale"])
    return mixed.reshape(tokens, heads * vdim) @ w["o"].T


def silu(z):
    return z * torch.sigmoid(z)


def routed_feed_forward(h, w, mlp, margins=None):
    """``margins`` (a list) gets, per token, the gap between the last chosen and the best refused
    router logit: how far the choice is from a close call."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ w["router"].T
    scores = torch.sigmoid(logits)                                      # [T, experts]
    chosen = torch.topk(scores, top, dim=-1).indices
    if margins is not None and top < experts:
        ordered = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            x = scores[t, e] * h[t]
            out[t] += (silu(x @ w[f"e{e}.gate"].T) * (x @ w[f"e{e}.up"].T)) @ w[f"e{e}.down"].T
    return out


def _sub(weights, prefix):
    return {name[len(prefix):]: t.to(F64) for name, t in weights.items() if name.startswith(prefix)}


def forward(config, weights, tokens, start=0, margins=None):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width]."""
    eps = float(config["norm"]["eps"])
    positions = torch.arange(start, start + len(tokens))
    x = weights["embed"].to(F64)[torch.tensor(tokens)]
    shared, streams = {}, []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        n = rms_norm(x, weights[prefix + "norm1"].to(F64), eps)
        w = _sub(weights, prefix + "mix.")
        if layer["type"] == "attention":
            mixed = attention_mixer(n, w, layer["mixer"], positions, shared)
        elif layer["type"] == "latent_attention":
            mixed = latent_attention_mixer(n, w, layer["mixer"], positions, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            mixed = mixed + routed_feed_forward(n, _sub(weights, prefix + "mlp."), layer["mlp"], margins)
        x = x + mixed
        streams.append(x)
    logits = rms_norm(x, weights["final.norm"].to(F64), eps) @ weights["embed"].to(F64).T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams)


def tensor_shapes(config):
    """Name -> shape of every tensor a model folder of this configuration holds."""
    width = config["width"]
    shapes = {"embed": (config["vocab"], width), "final.norm": (width,)}
    for index, layer in enumerate(config["layers"]):
        prefix, m = f"l{index}.", layer["mixer"]
        shapes[prefix + "norm1"] = (width,)
        mix = prefix + "mix."
        if layer["type"] == "attention":
            shapes[mix + "q"] = (m["heads"] * m["dim"], width)
            shapes[mix + "k"] = (m["kv_heads"] * m["dim"], width)
            shapes[mix + "v"] = (m["kv_heads"] * m["vdim"], width)
            shapes[mix + "o"] = (width, m["heads"] * m["vdim"])
            if m.get("v_mix"):
                shapes[mix + "vmix"] = ()
        else:
            shapes[mix + "dq"] = (m["q_rank"], width)
            shapes[mix + "dq.norm"] = (m["q_rank"],)
            shapes[mix + "uq"] = (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
            shapes[mix + "dkv"] = (m["kv_rank"] + m["rot_dim"], width)
            shapes[mix + "dkv.norm"] = (m["kv_rank"],)
            shapes[mix + "uk"] = (m["heads"] * m["dim"], m["kv_rank"])
            shapes[mix + "uv"] = (m["heads"] * m["vdim"], m["kv_rank"])
            shapes[mix + "o"] = (width, m["heads"] * m["vdim"])
        mlp = layer.get("mlp")
        if mlp is not None:
            ff = mlp["expert"]["ff"]
            shapes[prefix + "mlp.router"] = (mlp["router"]["experts"], width)
            for e in range(mlp["router"]["experts"]):
                shapes[prefix + f"mlp.e{e}.gate"] = (ff, width)
                shapes[prefix + f"mlp.e{e}.up"] = (ff, width)
                shapes[prefix + f"mlp.e{e}.down"] = (width, ff)
    return shapes


def random_model(config, seed):
    """Random weights in bfloat16: matrices that keep activations of order one (so that scores and
    router logits spread), norm weights around one, blending weights inside (0, 1)."""
    generator = torch.Generator().manual_seed(seed)
    weights = {}
    for name, shape in sorted(tensor_shapes(config).items()):
        values = torch.randn(shape, generator=generator)
        if name.endswith("norm") or name.endswith("norm1"):
            values = 1.0 + 0.1 * values
        elif name.endswith("vmix"):
            values = 0.2 + 0.6 * torch.sigmoid(values)
        elif name == "embed":
            pass
        elif name.endswith("router"):
            values = values * 2.0 * shape[-1] ** -0.5
        else:
            values = values * shape[-1] ** -0.5
        weights[name] = values.to(torch.bfloat16)
    return weights
