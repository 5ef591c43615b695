"""Zetavik, stated plainly: token by token, in float64, one function per mechanism.

This is the tests' oracle.  It shares nothing with the engine: it reads the configuration
document and a dict of tensors and walks a sequence's tokens in order.  Notation: ``h`` is a
layer's normed input ``[T, width]``, ``eps`` the layers' epsilon.

A layer is parallel: ``x <- x + mixer(h) + ff(h)`` with ``h = layer_norm(x)`` (a weight, no
bias).  Mixers: ``mamba2`` (a state-space recurrence behind a short causal convolution),
``latent_attention`` (softmax attention whose keys and values are expanded from a cached
latent, with one rotated key part shared by all heads), ``lightning`` (linear attention with
one fixed decay per head).  Feed-forwards: ``dense`` (squared ReLU) and ``moe`` (softmax
router, group-limited choice, a shared expert).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def _w(tensors, name):
    return tensors[name].to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def layer_norm(x, weight, eps):
    mean = x.mean(-1, keepdim=True)
    dev = x - mean
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * weight


def rms_norm(x, weight, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def rotate_half_split(x, positions, dims, base):
    """Rotates the first ``dims`` entries of every row of ``x[T, D]``: entry ``i`` is paired with
    ``i + dims/2`` and the pair turns by ``position * base^(-2i/dims)``."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    angle = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    u, v = x[:, :half], x[:, half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[:, dims:]], dim=-1)


# --------------------------------------------------------------------------- mixers


def causal_conv(x, taps, bias):
    """``y_t[c] = bias[c] + sum_j taps[c, j] * x_{t - (L-1) + j}[c]`` with zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    padded = torch.cat([torch.zeros((L - 1, C), dtype=F64), x], dim=0)
    y = torch.zeros((T, C), dtype=F64) + bias
    for j in range(L):
        y = y + padded[j : j + T] * taps[:, j]
    return y


def mamba2(tensors, prefix, m, h, eps):
    heads, vdim, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * vdim
    p = h @ _w(tensors, f"{prefix}.in").T
    z, xbc, dt = p[:, :inner], p[:, inner : 2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_conv(xbc, _w(tensors, f"{prefix}.conv"), _w(tensors, f"{prefix}.conv.b")))
    x, B, C = xbc[:, :inner], xbc[:, inner : inner + G * N], xbc[:, inner + G * N :]
    dt = softplus(dt + _w(tensors, f"{prefix}.dt_bias"))
    rate = torch.exp(_w(tensors, f"{prefix}.A_log"))
    skip = _w(tensors, f"{prefix}.D")
    T = h.shape[0]
    y = torch.zeros((T, heads, vdim), dtype=F64)
    for head in range(heads):
        g = head // (heads // G)
        S = torch.zeros((N, vdim), dtype=F64)
        xs = x[:, head * vdim : (head + 1) * vdim]
        for t in range(T):
            S = math.exp(-float(rate[head]) * float(dt[t, head])) * S + dt[t, head] * torch.outer(B[t, g * N : (g + 1) * N], xs[t])
            y[t, head] = S.T @ C[t, g * N : (g + 1) * N] + skip[head] * xs[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * _w(tensors, f"{prefix}.norm")
    return y @ _w(tensors, f"{prefix}.o").T


def latent_attention(tensors, prefix, m, h, eps, positions=None):
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = torch.arange(T) if positions is None else positions
    cq = rms_norm(h @ _w(tensors, f"{prefix}.dq").T, _w(tensors, f"{prefix}.dq.norm"), eps)
    q = (cq @ _w(tensors, f"{prefix}.uq").T).reshape(T, H, dim + rot)
    down = h @ _w(tensors, f"{prefix}.dkv").T
    c = rms_norm(down[:, :rank], _w(tensors, f"{prefix}.dkv.norm"), eps)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    shared = rotate_half_split(down[:, rank:], positions, dims, base)
    k_plain = (c @ _w(tensors, f"{prefix}.uk").T).reshape(T, H, dim)
    v = (c @ _w(tensors, f"{prefix}.uv").T).reshape(T, H, vdim)
    gate = torch.sigmoid(h @ _w(tensors, f"{prefix}.g").T)
    out = torch.zeros((T, H, vdim), dtype=F64)
    visible = positions[None, :] <= positions[:, None]
    for head in range(H):
        q_rot = rotate_half_split(q[:, head, dim:], positions, dims, base)
        scores = (q[:, head, :dim] @ k_plain[:, head].T + q_rot @ shared.T) * m["scale"]
        scores = scores.masked_fill(~visible, -math.inf)
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, head] * gate[:, head : head + 1]
    return out.reshape(T, H * vdim) @ _w(tensors, f"{prefix}.o").T


def lightning(tensors, prefix, m, h, eps):
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ _w(tensors, f"{prefix}.q").T).reshape(T, H, dim)
    k = silu(h @ _w(tensors, f"{prefix}.k").T).reshape(T, H, dim)
    v = silu(h @ _w(tensors, f"{prefix}.v").T).reshape(T, H, vdim)
    out = torch.zeros((T, H, vdim), dtype=F64)
    for head in range(H):
        S = torch.zeros((dim, vdim), dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    o = rms_norm(out.reshape(T, H * vdim), _w(tensors, f"{prefix}.norm"), eps)
    o = o * torch.sigmoid(h @ _w(tensors, f"{prefix}.g").T)
    return o @ _w(tensors, f"{prefix}.o").T


# --------------------------------------------------------------------------- feed-forwards


def dense_ff(tensors, prefix, h):
    mid = torch.relu(h @ _w(tensors, f"{prefix}.up").T)
    return (mid * mid) @ _w(tensors, f"{prefix}.down").T


def gated_expert(tensors, prefix, h):
    return (silu(h @ _w(tensors, f"{prefix}.gate").T) * (h @ _w(tensors, f"{prefix}.up").T)) @ _w(tensors, f"{prefix}.down").T


def route(scores, top, group_count, group_keep):
    """For every row of ``scores[T, E]``: the ``top`` experts with the largest scores among the
    experts of the ``group_keep`` groups (of neighbours) whose largest score is largest.
    Returns a boolean ``[T, E]``."""
    T, E = scores.shape
    per = E // group_count
    best = scores.reshape(T, group_count, per).max(-1).values
    kept = torch.zeros((T, group_count), dtype=torch.bool)
    kept.scatter_(1, best.topk(group_keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(T, group_count, per).reshape(T, E)
    masked = scores.masked_fill(~allowed, -1.0)
    chosen = torch.zeros((T, E), dtype=torch.bool)
    chosen.scatter_(1, masked.topk(top, dim=-1).indices, True)
    return chosen


def route_margin(scores, chosen, group_count):
    """Per row: how far the choice was from falling otherwise, as a share of the score at stake -
    the smaller of (worst chosen score - best score left out) and (worst kept group - best dropped
    group); ``inf`` where nothing was left out."""
    T, E = scores.shape
    inf = torch.full((T,), float("inf"), dtype=F64)
    low = torch.where(chosen, scores, torch.full_like(scores, float("inf"))).min(-1).values
    out = torch.where(~chosen, scores, torch.full_like(scores, -1.0)).max(-1).values
    margin = torch.where(out >= 0, (low - out).abs() / low.clamp_min(1e-30), inf)
    groups = scores.reshape(T, group_count, E // group_count)
    best = groups.max(-1).values
    kept = chosen.reshape(T, group_count, E // group_count).any(-1)
    low_g = torch.where(kept, best, torch.full_like(best, float("inf"))).min(-1).values
    out_g = torch.where(~kept, best, torch.full_like(best, -1.0)).max(-1).values
    return torch.minimum(margin, torch.where(out_g >= 0, (low_g - out_g).abs() / low_g.clamp_min(1e-30), inf))


def moe_ff(tensors, prefix, mlp, h, margins=None):
    r = mlp["router"]
    scores = torch.softmax(h @ _w(tensors, f"{prefix}.router").T, dim=-1)
    chosen = route(scores, r["top"], r["groups"]["count"], r["groups"]["keep"])
    if margins is not None:
        margins.append(route_margin(scores, chosen, r["groups"]["count"]))
    weights = scores * chosen * r["scale"]
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        rows = chosen[:, e].nonzero().flatten()
        if rows.numel():
            out[rows] += weights[rows, e : e + 1] * gated_expert(tensors, f"{prefix}.e{e}", h[rows])
    if mlp.get("shared") is not None:
        out = out + gated_expert(tensors, f"{prefix}.shared", h)
    return out


# --------------------------------------------------------------------------- the model

MIXERS = {"mamba2": mamba2, "latent_attention": latent_attention, "lightning": lightning}


def forward(doc, tensors, tokens, after_layer=None, margins=None):
    """Logits ``[T, vocab]`` (float64) of a whole sequence; ``after_layer(i, x)`` sees the
    residual rows after every layer; a list ``margins`` is given one ``route_margin`` per routed layer."""
    eps = doc["norm"]["eps"]
    table = _w(tensors, "embed")
    x = table[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(doc["layers"]):
        h = layer_norm(x, _w(tensors, f"l{i}.norm1"), eps)
        y = MIXERS[layer["type"]](tensors, f"l{i}.mix", layer["mixer"], h, eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(tensors, f"l{i}.mlp", h) if mlp["kind"] == "dense" else moe_ff(tensors, f"l{i}.mlp", mlp, h, margins))
        x = x + y
        if after_layer is not None:
            after_layer(i, x)
    return layer_norm(x, _w(tensors, "final.norm"), eps) @ table.T
