"""A plain, slow statement of the Filulix design, one function per mechanism.

Everything is evaluated token by token in float64 on the CPU from a configuration document
and a dictionary of tensors; nothing here is shared with the engine.  The tests compare the
engine's logits, and single kernels, with these functions.

Notation: ``T`` tokens of ONE sequence, positions ``0 .. T-1``; ``D`` the model width;
matrices are stored ``[out, in]`` and applied as ``W x``.
"""

from __future__ import annotations

import torch

F64 = torch.float64


def _w(tensors, name):
    return tensors[name].to(F64)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def rms_unit(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def shifted_norm(x, weight, eps):
    """RMS norm whose stored weight lies around zero: ``rms_unit(x) * (1 + weight)``."""
    return rms_unit(x, eps) * (1.0 + weight)


# --------------------------------------------------------------------------- embedding


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous token, token); the
    sequence's first token takes the table's last row (index ``buckets``)."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embedding(doc, tensors, tokens):
    emb = doc.get("embedding", {})
    x = _w(tensors, "embed")[torch.tensor(tokens)] * float(emb.get("scale", 1.0))
    bigram = emb.get("bigram")
    if bigram is not None:
        rows = bigram_rows(tokens, int(bigram["buckets"]), int(bigram["mul_prev"]), int(bigram["mul_cur"]))
        x = x + _w(tensors, "bigram")[torch.tensor(rows)]
    return x


# --------------------------------------------------------------------------- feed-forward


def dense_ff(tensors, prefix, h):
    gate = h @ _w(tensors, f"{prefix}.mlp.gate").T
    up = h @ _w(tensors, f"{prefix}.mlp.up").T
    return (silu(gate) * up) @ _w(tensors, f"{prefix}.mlp.down").T


# --------------------------------------------------------------------------- the wkv mixer


def wkv_mixer(tensors, prefix, spec, h, eps):
    """Time mixing with a decaying matrix state per head.

    ``m_c = h_t + (h_{t-1} - h_t) * mu_c`` for c in r, k, v, g, w (``h_{-1} = 0``);
    ``decay_t = exp(-exp(W2 tanh(W1 m_w) + w0))`` per head and key channel;
    ``o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t``; ``S_t = diag(decay_t) S_{t-1} + k_t v_t^T``;
    each head's ``o_t`` is brought to unit RMS, heads are joined, multiplied by the mixer's norm
    weight and by ``silu(W_g m_g)``, and projected by ``W_o``."""
    T, D = h.shape
    H, d = int(spec["heads"]), int(spec["dim"])
    p = f"{prefix}.mix"
    prev = torch.cat([torch.zeros(1, D, dtype=F64), h[:-1]], dim=0)

    def mixed(c):
        return h + (prev - h) * _w(tensors, f"{p}.mu.{c}")

    r = (mixed("r") @ _w(tensors, f"{p}.r").T).reshape(T, H, d)
    k = (mixed("k") @ _w(tensors, f"{p}.k").T).reshape(T, H, d)
    v = (mixed("v") @ _w(tensors, f"{p}.v").T).reshape(T, H, d)
    gate = silu(mixed("g") @ _w(tensors, f"{p}.g").T)
    z = torch.tanh(mixed("w") @ _w(tensors, f"{p}.w1").T) @ _w(tensors, f"{p}.w2").T + _w(tensors, f"{p}.w0")
    decay = torch.exp(-torch.exp(z)).reshape(T, H, d)
    bonus = _w(tensors, f"{p}.u").reshape(H, d)
    out = torch.zeros(T, H, d, dtype=F64)
    state = torch.zeros(H, d, d, dtype=F64)  # [head, key channel, value channel]
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], state + bonus[:, :, None] * kv)
        state = decay[t][:, :, None] * state + kv
    out = rms_unit(out, eps).reshape(T, H * d) * _w(tensors, f"{p}.norm") * gate
    return out @ _w(tensors, f"{p}.o").T


# --------------------------------------------------------------------------- the parallel mixer


def pooled_window_attention(q, k, v, scale, window, pool):
    """Softmax attention of ``q[T, H, d]`` over ``k[T, G, d]``, ``v[T, G, dv]``.

    Position ``i`` sees the tokens ``j`` with ``0 <= i - j < window`` and, in the same softmax,
    one mean key and mean value for every block ``b`` of ``pool`` consecutive positions that
    ended at or before ``i - window`` (``b * pool + pool - 1 <= i - window``).  Tokens that left
    the window and whose block is not complete behind it are not seen."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        keys, values = [k[lo : i + 1]], [v[lo : i + 1]]
        blocks = 0
        while blocks * pool + pool - 1 <= i - window:
            blocks += 1
        if blocks:
            keys.insert(0, k[: blocks * pool].reshape(blocks, pool, G, d).mean(1))
            values.insert(0, v[: blocks * pool].reshape(blocks, pool, G, -1).mean(1))
        kk, vv = torch.cat(keys), torch.cat(values)
        for h in range(H):
            g = h // (H // G)
            p = torch.softmax((kk[:, g] @ q[i, h]) * scale, dim=0)
            out[i, h] = p @ vv[:, g]
    return out


def rotate_half_split(x, positions, dims, base):
    """Rotates the pairs ``(c, c + dims/2)``, ``c < dims/2``, of the last axis of ``x[T, H, d]``
    by the angle ``position * base^(-2c/dims)``; channels from ``dims`` on pass unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * c / dims) for c in range(half)], dtype=F64)
    angle = torch.tensor(positions, dtype=F64)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def retention(q, k, v, decays):
    """Linear attention with one fixed decay per head: ``S_t = decay * S_{t-1} + k_t v_t^T``,
    ``o_t = S_t^T q_t`` (the current token included, no softmax, no denominator)."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    state = torch.zeros(H, d, v.shape[-1], dtype=F64)
    decay = torch.tensor(list(decays), dtype=F64)[:, None, None]
    for t in range(T):
        state = decay * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", q[t], state)
    return out


def parallel_mixer(tensors, prefix, spec, h, eps, round_cache=None):
    """Windowed attention with pooled blocks (left) beside retention (right) on the same input;
    ``left_scale * left + right_scale * right``.  ``round_cache`` (a dtype) rounds the left keys
    and values to what a cache of that type holds, before they are pooled or read."""
    T = h.shape[0]
    left, right = spec["left"], spec["right"]
    p = f"{prefix}.mix.left"
    H, G, d, dv = int(left["heads"]), int(left["kv_heads"]), int(left["dim"]), int(left["vdim"])
    q = (h @ _w(tensors, f"{p}.q").T).reshape(T, H, d)
    k = (h @ _w(tensors, f"{p}.k").T).reshape(T, G, d)
    v = (h @ _w(tensors, f"{p}.v").T).reshape(T, G, dv)
    if round_cache is not None:
        k, v = k.to(round_cache).to(F64), v.to(round_cache).to(F64)
    mask = left["mask"]
    attn = pooled_window_attention(q, k, v, float(left["scale"]), int(mask["size"]), int(mask["pool"]))
    y_left = attn.reshape(T, H * dv) @ _w(tensors, f"{p}.o").T

    p = f"{prefix}.mix.right"
    H, d, dv = int(right["heads"]), int(right["dim"]), int(right["vdim"])
    q = (h @ _w(tensors, f"{p}.q").T).reshape(T, H, d)
    k = (h @ _w(tensors, f"{p}.k").T).reshape(T, H, d)
    v = (h @ _w(tensors, f"{p}.v").T).reshape(T, H, dv)
    rot = right.get("rot")
    if rot is not None:
        positions = list(range(T))
        q = rotate_half_split(q, positions, int(rot["dims"]), float(rot["base"]))
        k = rotate_half_split(k, positions, int(rot["dims"]), float(rot["base"]))
    k = k * d ** -0.5
    o = rms_unit(retention(q, k, v, right["decay"]), eps).reshape(T, H * dv)
    y_right = (o * silu(h @ _w(tensors, f"{p}.g").T)) @ _w(tensors, f"{p}.o").T
    return float(spec["left_scale"]) * y_left + float(spec["right_scale"]) * y_right


# --------------------------------------------------------------------------- layers and the model


def run_order(doc):
    """Layer indices in the order they run: ``loop.start .. loop.stop - 1`` repeated
    ``loop.times`` times in a row, the other layers once, in place."""
    n = len(doc["layers"])
    loop = doc.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def mixer_of(doc, tensors, i, h, eps, round_cache=None):
    layer = doc["layers"][i]
    if layer["type"] == "wkv":
        return wkv_mixer(tensors, f"l{i}", layer["mixer"], h, eps)
    if layer["type"] == "parallel":
        return parallel_mixer(tensors, f"l{i}", layer["mixer"], h, eps, round_cache)
    raise ValueError(layer["type"])


def hyper_sublayer(tensors, prefix, q, lanes, fn, norm_weight, eps):
    """One sublayer over ``lanes[s, T, D]``: the sublayer reads ``sum_s in[s] lanes[s]``, normed;
    then ``lanes'[t] = sum_s mix[s, t] lanes[s] + out[t] * y`` for all ``t`` at once."""
    w_in = _w(tensors, f"{prefix}.hc{q}.in")
    w_out = _w(tensors, f"{prefix}.hc{q}.out")
    w_mix = _w(tensors, f"{prefix}.hc{q}.mix")
    u = torch.einsum("s,std->td", w_in, lanes)
    y = fn(shifted_norm(u, norm_weight, eps))
    return torch.einsum("sr,std->rtd", w_mix, lanes) + w_out[:, None, None] * y[None]


def forward(doc, tensors, tokens, after_layer=None, round_cache=None):
    """Logits ``[T, vocab]`` (float64) of one sequence.  ``after_layer(run, x)`` is called with
    the residual (the sum of the lanes where there are several) after every layer run."""
    eps = float(doc["norm"]["eps"])
    x = embedding(doc, tensors, tokens)
    streams = doc.get("streams")
    lanes = x[None].repeat(int(streams), 1, 1) if streams else None
    for run, i in enumerate(run_order(doc)):
        prefix = f"l{i}"
        layer = doc["layers"][i]
        mix = lambda h: mixer_of(doc, tensors, i, h, eps, round_cache)  # noqa: E731
        ff = lambda h: dense_ff(tensors, prefix, h)  # noqa: E731
        if lanes is not None:
            lanes = hyper_sublayer(tensors, prefix, 1, lanes, mix, _w(tensors, f"{prefix}.norm1"), eps)
            if layer.get("mlp") is not None:
                lanes = hyper_sublayer(tensors, prefix, 2, lanes, ff, _w(tensors, f"{prefix}.norm2"), eps)
            x = lanes.sum(0)
        else:
            x = x + mix(shifted_norm(x, _w(tensors, f"{prefix}.norm1"), eps))
            if layer.get("mlp") is not None:
                x = x + ff(shifted_norm(x, _w(tensors, f"{prefix}.norm2"), eps))
        if after_layer is not None:
            after_layer(run, x)
    return shifted_norm(x, _w(tensors, "final.norm"), eps) @ _w(tensors, "head").T

