"""Time mixing with a decaying matrix state per head (the RWKV family's wkv recurrence).

With ``h_t`` the mixer's input and ``h_{t-1}`` the previous token's (zeros before a
sequence's first token), each of five projections reads its own blend

    m_c = h_t + (h_{t-1} - h_t) * mu_c,        c in r, k, v, g, w.

``r, k, v = W_r m_r, W_k m_k, W_v m_v`` in heads of ``dim``; ``gate = silu(W_g m_g)``; the
decay of every head and key channel is data-dependent through a low-rank pair,
``decay = exp(-exp(W_2 tanh(W_1 m_w) + w_0))``.  Per head, with a state ``S[key, value]``,

    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t          (the bonus u for the current token only)
    S_t = diag(decay_t) S_{t-1} + k_t v_t^T.

Each head's ``o_t`` is brought to unit RMS, the joined heads are multiplied by a weight
vector and by the gate, and projected.  Per request the mixer keeps ``h`` of the last token
and ``S`` of every head, both float32, zero for a new request.

Kernels: one launch forms the five blends (and a second stores the last row of each
sequence), six products, one launch for ``tanh``, and one launch that walks each sequence's
tokens in order with a head's state in registers and applies decay, bonus, unit RMS, weight
and gate - the decay's two exponentials included, in float32.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import NORMAL, ONES, VECTOR, TensorSpec
from .base import MIXERS, DeferredLinear, FixedState, Mixer

MAX_STATE_DIM = 256  # rows and columns of a head's state the recurrence kernel takes ...
MAX_STATE_SIZE = 32768  # ... and their product: a CTA keeps a head's state in registers

BLENDS = ("r", "k", "v", "g", "w")


@MIXERS.register("wkv_time_mix")
class WkvTimeMix(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``head_dim``, ``eps`` (of the unit RMS), and
    tensor names: ``mu`` (a dict over r, k, v, g, w), ``r_proj``, ``k_proj``, ``v_proj``,
    ``g_proj``, ``decay_down``, ``decay_up``, ``decay_bias``, ``bonus``, ``out_norm``,
    ``out_proj``; optionally ``decay_rank``."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.eps = float(p["eps"])
        if not 0 < self.dim <= MAX_STATE_DIM or self.dim * self.dim > MAX_STATE_SIZE:
            raise UnsupportedShape("head_dim", self.dim, f"the recurrence kernel takes states up to {MAX_STATE_DIM} rows or columns and {MAX_STATE_SIZE} values")
        fits = getattr(env.ops, "recurrence_supported", None)
        if fits is not None and not fits(self.dim, self.dim):
            raise UnsupportedShape("head_dim", self.dim, "the recurrence kernel has no layout for a state of this shape")
        self.names = {k: p[k] for k in ("r_proj", "k_proj", "v_proj", "g_proj", "decay_down", "decay_up", "decay_bias",
                                        "bonus", "out_norm", "out_proj")}
        self.mu_names = dict(p["mu"])
        # the rank of the decay's low-rank pair: the file's, unless the plan names it (random weights need it)
        self.rank = int(p["decay_rank"]) if p.get("decay_rank") else None
        self.mu = self.w = None

    def tensor_specs(self):
        inner = self.heads * self.dim
        n = self.names
        specs = [TensorSpec(self.mu_names[c], (self.hidden,), VECTOR, NORMAL, init_mean=0.4, init_std=0.2) for c in BLENDS]
        specs += [TensorSpec(n[k], (inner, self.hidden)) for k in ("r_proj", "k_proj", "v_proj", "g_proj")]
        specs += [
            TensorSpec(n["decay_down"], (self.rank or -1, self.hidden)),
            TensorSpec(n["decay_up"], (inner, self.rank or -1), init_std=0.1),
            TensorSpec(n["decay_bias"], (inner,), VECTOR, NORMAL, init_mean=-2.0, init_std=1.0),
            TensorSpec(n["bonus"], (self.heads, self.dim), VECTOR, NORMAL, init_mean=0.5, init_std=0.3),
            TensorSpec(n["out_norm"], (inner,), VECTOR, ONES),
            TensorSpec(n["out_proj"], (self.hidden, inner)),
        ]
        return specs

    def bind(self, tensors):
        n = self.names
        self.mu = torch.stack([tensors[self.mu_names[c]].to(torch.float32) for c in BLENDS]).contiguous()
        self.w = {k: tensors[n[k]] for k in n}
        self.rank = self.w["decay_down"].shape[0]
        if self.w["decay_up"].shape[1] != self.rank:
            raise UnsupportedShape("decay rank", tuple(self.w["decay_up"].shape), f"does not fit a pair of rank {self.rank}")

    def cache_spec(self):
        return (FixedState((self.hidden,)), FixedState((self.heads, self.dim, self.dim)))

    def forward(self, x, step, cache):
        ops, dtype, w = self.env.ops, self.env.dtype, self.w
        last_row, state = cache
        blends = ops.token_shift_blend(x, self.mu, last_row.state, step)  # [5, T, hidden]
        r = ops.linear(blends[0], w["r_proj"], dtype)
        k = ops.linear(blends[1], w["k_proj"], dtype)
        v = ops.linear(blends[2], w["v_proj"], dtype)
        g = ops.linear(blends[3], w["g_proj"], dtype)
        low = ops.unary(ops.linear(blends[4], w["decay_down"], torch.float32), "tanh", dtype)
        z = ops.linear(low, w["decay_up"], torch.float32)
        out = torch.empty((x.shape[0], self.heads * self.dim), dtype=dtype, device=x.device)
        ops.decay_recurrence(
            r, k, v, out, state.state, step, self.heads, self.dim, self.dim, self.eps,
            decay_logits=z, decay_bias=w["decay_bias"], bonus=w["bonus"], out_weight=w["out_norm"], gate=g,
        )
        return DeferredLinear(ops, out, w["out_proj"], dtype)
