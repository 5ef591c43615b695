"""Mamba-2: a state-space recurrence with one scalar decay per head and token, behind a short
causal convolution.

With ``inner = heads * vdim``, ``N`` the state size and ``G`` groups, the input projection is
laid out ``[z: inner | x: inner | B: G N | C: G N | dt: heads]``.  ``x``, ``B`` and ``C``
together pass a causal convolution per channel (``taps`` wide, the last tap on the current
token, zeros before a sequence's start, a bias) and ``silu``.  ``dt = softplus(dt + dt_bias)``
without a clamp.  Head ``h`` reads ``B`` and ``C`` of group ``h // (heads / G)``:

    S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T        (S is N x vdim)
    y_t = S_t^T C_t + D_h x_t.

The joined heads are multiplied by ``silu(z)`` first, then brought to unit RMS in
``norm_groups`` equal parts (each by its own root mean square), multiplied by a weight, and
projected.  Per request the mixer keeps the convolution's last ``taps - 1`` inputs and every
head's state, both float32, zero for a new request.

``softplus``, the two exponentials, ``dt`` and the state are float32 inside the recurrence
kernel (``ops.state_recurrence``); the gate and the group norm are a row kernel
(``ops.group_rmsnorm``) on its float32 outputs.
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import NORMAL, ONES, VECTOR, TensorSpec
from .base import MIXERS, DeferredLinear, FixedState, Mixer, project
from .lightning import MAX_STATE_ROWS
from .short_conv import MAX_TAPS


@MIXERS.register("mamba2")
class Mamba2(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``v_head_dim``, ``state``, ``groups``, ``taps``,
    ``norm_groups``, ``eps``, and names ``in_proj``, ``conv``, ``conv_bias``, ``dt_bias``,
    ``a_log``, ``skip``, ``out_norm``, ``out_proj``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.vdim = int(p["v_head_dim"])
        self.state = int(p["state"])
        self.groups = int(p["groups"])
        self.taps = int(p["taps"])
        self.norm_groups = int(p["norm_groups"])
        self.eps = float(p["eps"])
        self.inner = self.heads * self.vdim
        if self.heads % self.groups:
            raise UnsupportedShape("groups", self.groups, f"does not divide {self.heads} heads")
        if self.inner % self.norm_groups:
            raise UnsupportedShape("norm_groups", self.norm_groups, f"does not divide the inner width {self.inner}")
        if not 2 <= self.taps <= MAX_TAPS:
            raise UnsupportedShape("conv taps", self.taps, f"the convolution kernels take 2 to {MAX_TAPS} taps")
        if not 0 < self.state <= MAX_STATE_ROWS:
            raise UnsupportedShape("state", self.state, f"the recurrence kernel takes states of up to {MAX_STATE_ROWS} rows")
        self.names = {k: p[k] for k in ("in_proj", "conv", "conv_bias", "dt_bias", "a_log", "skip", "out_norm", "out_proj")}
        self.w = None

    @property
    def conv_width(self):
        return self.inner + 2 * self.groups * self.state

    def tensor_specs(self):
        n, c = self.names, self.conv_width
        return [
            TensorSpec(n["in_proj"], (self.inner + c + self.heads, self.hidden)),
            TensorSpec(n["conv"], (c, self.taps), VECTOR, NORMAL, alt_shapes=((c, 1, self.taps),), init_std=0.3),
            TensorSpec(n["conv_bias"], (c,), VECTOR, NORMAL, init_std=0.1),
            TensorSpec(n["dt_bias"], (self.heads,), VECTOR, NORMAL, init_mean=-1.0, init_std=0.5),
            TensorSpec(n["a_log"], (self.heads,), VECTOR, NORMAL, init_mean=-1.0, init_std=0.7),
            TensorSpec(n["skip"], (self.heads,), VECTOR, ONES),
            TensorSpec(n["out_norm"], (self.inner,), VECTOR, ONES),
            TensorSpec(n["out_proj"], (self.hidden, self.inner)),
        ]

    def bind(self, tensors):
        self.w = {k: tensors[name] for k, name in self.names.items()}
        if self.w["conv"].dim() == 3:
            self.w["conv"] = self.w["conv"].reshape(self.conv_width, self.taps).contiguous()

    def cache_spec(self):
        return (FixedState((self.taps - 1, self.conv_width)), FixedState((self.heads, self.state, self.vdim)))

    def forward(self, x, step, cache):
        ops, w = self.env.ops, self.w
        window, state = cache
        inner, c, gn = self.inner, self.conv_width, self.groups * self.state
        proj = project(ops, x, w["in_proj"], self.env.dtype)
        xbc = ops.causal_conv(proj[:, inner : inner + c], w["conv"], w["conv_bias"], window.state, step, silu=True)
        raw = ops.state_recurrence(
            xbc[:, inner + gn :], xbc[:, inner : inner + gn], xbc[:, :inner], state.state, step,
            self.heads, self.groups, self.state, self.vdim,
            dt=proj[:, inner + c :], dt_bias=w["dt_bias"], a_log=w["a_log"], skip=w["skip"],
        )
        out = ops.group_rmsnorm(raw, w["out_norm"], self.eps, self.norm_groups, self.env.dtype, gate=proj[:, :inner], gate_mode="silu_before")
        return DeferredLinear(ops, out, w["out_proj"], self.env.dtype)
