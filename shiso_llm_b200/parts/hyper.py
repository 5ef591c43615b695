"""Hyper-connections: a layer arrangement that keeps several copies of the residual stream.

Instead of one stream ``x`` there are ``n`` copies ``x_1 .. x_n`` (all equal to the embedding
output at the start).  A sublayer (the mixer, then the feed-forward) reads a weighted sum of
the copies and writes into all of them:

    u      = sum_s  a[s] * x_s
    y      = sublayer(norm(u))
    x_t'   = sum_s  M[s, t] * x_s  +  b[t] * y        (all ``t`` from the old copies)

with a read vector ``a``, a write vector ``b`` and a mixing matrix ``M`` (indexed
``[from, to]``) per sublayer.  After the last layer the stream is the sum of the copies.

The copies live on the ``Stream`` (``lanes``, float32 ``[n, T, hidden]``).  A sublayer's
write is left waiting (``lane_update``) and done by the kernel that makes the next read, so
a sublayer costs one pass over the copies: ``hyper_mix_read`` writes the waiting update,
forms ``u`` and normalises it in one launch; ``hyper_mix_sum`` closes the last layer.
The first read takes the single stream for every copy (no copies are made before the
first write).
"""

from __future__ import annotations

from ..weights.spec import IDENTITY, NORMAL, ONES, VECTOR, TensorSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, DeferredLinear

MAX_COPIES = 8  # what the kernel keeps of one element in registers


def _tensor(value):
    return value.materialize() if isinstance(value, DeferredLinear) else value


@BLOCKS.register("hyper_pre_norm")
class HyperPreNormBlock(Block):
    """``params``: ``copies``; ``mixer_io`` and ``ff_io``: the names of the read vector, write
    vector and mixing matrix of each sublayer (``{"read": .., "write": .., "mix": ..}``)."""

    def __init__(self, spec, env, layer):
        super().__init__(spec, env)
        self.name = layer.name
        self.copies = int(spec.params["copies"])
        if not 1 <= self.copies <= MAX_COPIES:
            raise ValueError(f"{self.copies} copies of the stream: the kernel takes 1 to {MAX_COPIES}")
        self.mixer_norm = NORMS.build(layer.mixer_norm, env)
        self.mixer = MIXERS.build(layer.mixer, env)
        self.feed_forward = None
        self.ff_norm = None
        self.io_names = [dict(spec.params["mixer_io"])]
        if layer.feed_forward is not None:
            self.feed_forward = FEED_FORWARDS.build(layer.feed_forward, env)
            self.ff_norm = NORMS.build(layer.feed_forward_norm, env)
            self.io_names.append(dict(spec.params["ff_io"]))
        for norm in (self.mixer_norm, self.ff_norm):
            if norm is not None and not hasattr(norm, "rms_params"):
                raise ValueError("the read of the copies normalises with an RMS norm")
        self.io = []

    def sub_parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward) if p is not None]

    def tensor_specs(self):
        n = self.copies
        specs = []
        for part in self.sub_parts():
            specs += part.tensor_specs()
        for names in self.io_names:
            specs += [
                TensorSpec(names["read"], (n,), VECTOR, NORMAL, init_mean=1.0 / n, init_std=0.1),
                TensorSpec(names["write"], (n,), VECTOR, ONES),
                TensorSpec(names["mix"], (n, n), VECTOR, IDENTITY),
            ]
        return specs

    def bind(self, tensors):
        for part in self.sub_parts():
            part.bind(tensors)
        self.io = [(tensors[n["read"]], tensors[n["write"]], tensors[n["mix"]]) for n in self.io_names]

    def mixer_part(self):
        return self.mixer

    def _read(self, stream, read, norm):
        """Writes the waiting update, then the normed weighted sum of the copies."""
        ops = self.env.ops
        weight, eps = norm.rms_params()
        if stream.pending is not None:
            raise RuntimeError("a block output is waiting to be added to a single stream; copies cannot take it")
        source = stream.lanes if stream.lanes is not None else stream.residual
        update = stream.lane_update
        stream.lane_update = None
        if update is None:
            lanes, x = ops.hyper_mix_read(source, None, None, None, self.copies, read, weight, eps, self.env.dtype)
        else:
            y, mix, write = update
            lanes, x = ops.hyper_mix_read(source, y, mix, write, self.copies, read, weight, eps, self.env.dtype)
        if lanes is not None:
            stream.lanes = lanes
        return x

    def _leave(self, stream, y, write, mix):
        stream.lane_update = (_tensor(y), mix, write)
        if stream.observer is not None:
            stream.observer(stream)

    def forward(self, stream, step, cache):
        read, write, mix = self.io[0]
        x = self._read(stream, read, self.mixer_norm)
        self._leave(stream, self.mixer.forward(x, step, cache), write, mix)
        if self.feed_forward is not None:
            read, write, mix = self.io[1]
            x = self._read(stream, read, self.ff_norm)
            self._leave(stream, self.feed_forward.forward(x, step), write, mix)
