"""A plain, slow statement of the Tepavik decoder, one function per mechanism.

Everything is written token by token or as whole-sequence tensor expressions in
one floating type (float64 by default), from the equations alone; nothing of
``einf_b200`` is imported.  A model is a ``config`` dict with the keys of the
design's ``config.json`` and a dict of tensors by checkpoint name.

Notation: ``T`` tokens of one sequence, positions ``0..T-1``; ``h`` is a mixer's
input ``[T, width]``; matrices are stored ``[out, in]``.
"""
from __future__ import annotations

import math

import torch


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms: the stored weight lies around zero and stands for 1 + w."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x / (1.0 + torch.exp(-x))


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0.0)


def squared_relu_mlp(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    a = torch.clamp(h @ up.T, min=0.0)
    return (a * a) @ down.T


def attention_keys_values(h, w, prefix, m, eps):
    """Keys (unit RMS per head) and values of one attention layer: [T, G, dim], [T, G, vdim]."""
    T = h.shape[0]
    G, dim, vdim = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, dim)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, G, vdim)
    return rms_unit(k, eps), v


def chunked_attention(h, w, prefix, m, eps, keys_values):
    """Softmax attention without positions: unit-RMS queries and keys, a tanh cap on the scores,
    and a mask that lets position i see j <= i of its own block of ``mask.size`` positions."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_unit((h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, dim), eps)
    k, v = keys_values
    size = m["mask"]["size"]
    cap = m["softcap"]
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            first = (i // size) * size
            s = (k[first:i + 1, g] @ q[i, head]) * m["scale"]
            s = cap * torch.tanh(s / cap)
            p = torch.softmax(s, dim=0)
            out[i, head] = p @ v[first:i + 1, g]
    return out.reshape(T, H * vdim) @ w[prefix + "o"].T


def lightning_mixer(h, w, prefix, m, eps):
    """Linear attention with a fixed decay per head, a joint norm over the heads and a sigmoid gate."""
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[prefix + "q"].T).view(T, H, dim)
    k = silu(h @ w[prefix + "k"].T).view(T, H, dim)
    v = silu(h @ w[prefix + "v"].T).view(T, H, vdim)
    out = torch.zeros(T, H, vdim, dtype=h.dtype)
    for head in range(H):
        state = torch.zeros(dim, vdim, dtype=h.dtype)
        decay = float(m["decay"][head])
        for t in range(T):
            state = decay * state + torch.outer(k[t, head], v[t, head])
            out[t, head] = state.T @ q[t, head]
    y = rms_unit(out.reshape(T, H * vdim), eps) * w[prefix + "norm"]
    y = y * torch.sigmoid(h @ w[prefix + "g"].T)
    return y @ w[prefix + "o"].T


def mamba2_mixer(h, w, prefix, m, eps):
    """Selective state space layer in its recurrent form."""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = h @ w[prefix + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    # causal convolution per channel: the last column of the kernel meets the current token
    kernel, bias = w[prefix + "conv"], w[prefix + "conv.b"]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], dim=0)
    conv = torch.zeros_like(xbc)
    for t in range(T):
        conv[t] = (padded[t:t + taps].T * kernel).sum(dim=1) + bias
    conv = silu(conv)
    x = conv[:, :inner].view(T, H, P)
    B = conv[:, inner:inner + G * N].view(T, G, N)
    C = conv[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[prefix + "dt_bias"])
    rate = torch.exp(w[prefix + "A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        state = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            state = math.exp(-float(rate[head]) * float(dt[t, head])) * state \
                + float(dt[t, head]) * torch.outer(B[t, g], x[t, head])
            y[t, head] = state.T @ C[t, g] + w[prefix + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[prefix + "norm"]
    return y @ w[prefix + "o"].T


def forward(config: dict, weights: dict, tokens, dtype=torch.float64):
    """Logits ``[T, vocab]`` of one sequence and the residual stream after every layer."""
    w = {name: t.to(dtype) for name, t in weights.items()}
    eps = float(config["norm"]["eps"])
    x = w["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
    kept = {}
    residuals = []
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        m = layer["mixer"]
        h = offset_norm(x, w[prefix + "norm1"], eps)
        if layer["type"] == "attention":
            source = m.get("kv_from")
            if source is None:
                kept[index] = attention_keys_values(h, w, prefix + "mix.", m, eps)
                source = index
            mixed = chunked_attention(h, w, prefix + "mix.", m, eps, kept[source])
        elif layer["type"] == "lightning":
            mixed = lightning_mixer(h, w, prefix + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            mixed = mamba2_mixer(h, w, prefix + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + mixed
        if layer.get("mlp") is not None:
            h = offset_norm(x, w[prefix + "norm2"], eps)
            x = x + squared_relu_mlp(h, w[prefix + "mlp.up"], w[prefix + "mlp.down"])
        residuals.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(residuals)


# ---------------------------------------------------------------------------
def random_model(config: dict, seed: int, scale: float = 1.0):
    """Random bfloat16 tensors for ``config`` under the design's checkpoint names."""
    gen = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]

    def matrix(rows, cols):
        return (torch.randn(rows, cols, generator=gen) * scale / math.sqrt(cols)).to(torch.bfloat16)

    def vector(n, std=0.1, mean=0.0):
        return (mean + std * torch.randn(n, generator=gen)).to(torch.bfloat16)

    w = {"embed": (torch.randn(vocab, width, generator=gen)).to(torch.bfloat16),
         "final.norm": vector(width), "head": matrix(vocab, width)}
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        w[p + "norm1"] = vector(width)
        if layer["type"] == "attention":
            H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.q.b"] = matrix(H * dim, width), vector(H * dim)
            if m.get("kv_from") is None:
                w[p + "mix.k"], w[p + "mix.k.b"] = matrix(G * dim, width), vector(G * dim)
                w[p + "mix.v"], w[p + "mix.v.b"] = matrix(G * vdim, width), vector(G * vdim)
            w[p + "mix.o"] = matrix(width, H * vdim)
        elif layer["type"] == "lightning":
            H, dim, vdim = m["heads"], m["dim"], m["vdim"]
            w[p + "mix.q"], w[p + "mix.k"] = matrix(H * dim, width), matrix(H * dim, width)
            w[p + "mix.v"], w[p + "mix.g"] = matrix(H * vdim, width), matrix(H * vdim, width)
            w[p + "mix.o"], w[p + "mix.norm"] = matrix(width, H * vdim), vector(H * vdim, 0.1, 1.0)
        else:
            H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, channels = H * P, H * P + 2 * G * N
            w[p + "mix.in"] = matrix(2 * inner + 2 * G * N + H, width)
            w[p + "mix.conv"] = (torch.randn(channels, taps, generator=gen) / math.sqrt(taps)).to(torch.bfloat16)
            w[p + "mix.conv.b"] = vector(channels)
            w[p + "mix.dt_bias"] = vector(H, 0.5, -1.0)
            w[p + "mix.A_log"] = vector(H, 0.5, 0.0)
            w[p + "mix.D"] = vector(H, 0.2, 1.0)
            w[p + "mix.norm"] = vector(inner, 0.1, 1.0)
            w[p + "mix.o"] = matrix(width, inner)
        if layer.get("mlp") is not None:
            w[p + "norm2"] = vector(width)
            w[p + "mlp.up"] = matrix(layer["mlp"]["ff"], width)
            w[p + "mlp.down"] = matrix(width, layer["mlp"]["ff"])
    return w
