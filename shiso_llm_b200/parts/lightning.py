"""Lightning attention: linear attention with one fixed decay per head.

``q = silu(W_q h)`` and ``k = silu(W_k h)`` in heads of ``dim``, ``v = silu(W_v h)`` in heads of
``vdim``.  Per head, with a state ``S[key, value]`` that starts at zero,

    S_t = decay_h * S_{t-1} + k_t v_t^T,        o_t = S_t^T q_t,

with no other scale.  The joined heads are brought to unit RMS together and multiplied by a
weight, then by ``sigmoid(W_g h)``, and projected.  The state is float32 and carried per
request.

The four input projections are one product.  One launch walks each sequence's rows in order
with a head's state in registers (``ops.state_recurrence``, which applies the activations on
load and leaves float32 outputs); a row kernel norms and gates them (``ops.group_rmsnorm``).
"""

from __future__ import annotations

import torch

from ..config.errors import UnsupportedShape
from ..weights.spec import ONES, VECTOR, TensorSpec
from .base import MIXERS, DeferredLinear, FixedState, Mixer, project

MAX_STATE_ROWS = 256  # key rows of a head's state the recurrence kernel takes


@MIXERS.register("lightning_attention")
class LightningAttention(Mixer):
    """``params``: ``hidden_size``, ``num_heads``, ``head_dim``, ``v_head_dim``, ``decay`` (one per
    head), ``eps``, and names ``q_proj``, ``k_proj``, ``v_proj``, ``g_proj``, ``out_norm``,
    ``out_proj``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.vdim = int(p["v_head_dim"])
        self.eps = float(p["eps"])
        decays = [float(d) for d in p["decay"]]
        if len(decays) != self.heads:
            raise UnsupportedShape("decay", decays, f"one decay per head is needed, {self.heads} heads")
        if not 0 < self.dim <= MAX_STATE_ROWS:
            raise UnsupportedShape("head_dim", self.dim, f"the recurrence kernel takes states of up to {MAX_STATE_ROWS} key rows")
        # what the kernel multiplies by: S - (1 - decay) S, with 1 - decay formed in float64
        self.losses = (1.0 - torch.tensor(decays, dtype=torch.float64)).to(torch.float32).to(env.device)
        self.names = {k: p[k] for k in ("q_proj", "k_proj", "v_proj", "g_proj", "out_norm", "out_proj")}
        self.in_matrix = self.out_matrix = self.norm_weight = None

    def tensor_specs(self):
        qk, vg, n = self.heads * self.dim, self.heads * self.vdim, self.names
        return [
            TensorSpec(n["q_proj"], (qk, self.hidden)), TensorSpec(n["k_proj"], (qk, self.hidden)),
            TensorSpec(n["v_proj"], (vg, self.hidden)), TensorSpec(n["g_proj"], (vg, self.hidden)),
            TensorSpec(n["out_norm"], (vg,), VECTOR, ONES), TensorSpec(n["out_proj"], (self.hidden, vg)),
        ]

    def bind(self, tensors):
        n = self.names
        mats = [tensors[n[k]] for k in ("q_proj", "k_proj", "v_proj", "g_proj")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.in_matrix = torch.cat(mats, dim=0).contiguous()
        self.out_matrix = tensors[n["out_proj"]]
        self.norm_weight = tensors[n["out_norm"]]

    def cache_spec(self):
        return FixedState((self.heads, self.dim, self.vdim))

    def forward(self, x, step, cache):
        ops = self.env.ops
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        proj = project(ops, x, self.in_matrix, self.env.dtype)
        raw = ops.state_recurrence(
            proj[:, :qk], proj[:, qk : 2 * qk], proj[:, 2 * qk : 2 * qk + vg], cache.state, step,
            self.heads, self.heads, self.dim, self.vdim, silu_inputs=True, head_loss=self.losses,
        )
        out = ops.group_rmsnorm(raw, self.norm_weight, self.eps, 1, self.env.dtype, gate=proj[:, 2 * qk + vg :], gate_mode="sigmoid_after")
        return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
