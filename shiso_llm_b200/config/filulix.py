"""Filulix: typed configuration and model plan.

A decoder whose layers keep several copies of the residual stream (hyper-connections) and
mix tokens in one of two ways: ``wkv`` - time mixing with a data-dependent decaying state -
or ``parallel`` - windowed softmax attention that also sees pooled blocks of old tokens,
beside retention, on the same input.  Token rows are scaled and joined by a row of a hashed
table of (previous token, token) pairs; norm weights are stored around zero and applied as
``1 + w``; a run of layers may be repeated with the same weights, each pass with a cache of
its own.

config.json keys: ``architecture``, ``vocab``, ``width``, ``streams``, ``norm.eps``,
``embedding.scale``, ``embedding.bigram.{buckets, mul_prev, mul_cur}``, ``loop.{start, stop,
times}`` and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with, for ``wkv``,
``mixer.{heads, dim}``, for ``parallel``, ``mixer.{left_scale, right_scale}``,
``mixer.left.{heads, kv_heads, dim, vdim, scale, mask.{size, pool}}`` and
``mixer.right.{heads, dim, vdim, decay, rot.{dims, base}}``, and ``mlp.{kind, ff}`` or null.
Tensor names: ``embed``, ``bigram``, ``final.norm``, ``head`` and, for layer ``i``,
``l<i>.norm1/2``, ``l<i>.hc1/2.{in, out, mix}``, ``l<i>.mix.*``, ``l<i>.mlp.{gate, up, down}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping, Optional

from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .errors import ConfigMissing, InvalidValue
from .registry import register_architecture

ARCHITECTURE = "Filulix"
WKV = "wkv"
PARALLEL = "parallel"
DENSE = "dense"


def _get(document: Mapping[str, Any], path: str):
    at = document
    for key in path.split("."):
        if not isinstance(at, Mapping) or key not in at or at[key] is None:
            raise ConfigMissing(path)
        at = at[key]
    return at


def _int(document, path: str, least: int = 1) -> int:
    value = _get(document, path)
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise InvalidValue(path, value, f"expected an integer of at least {least}")
    return value


def _num(document, path: str) -> float:
    value = _get(document, path)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise InvalidValue(path, value, "expected a number")
    return float(value)


@dataclass(frozen=True)
class FilulixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple  # the documents of the layers, checked
    streams: Optional[int] = None  # copies of the residual stream; None: one plain stream
    embedding_scale: float = 1.0
    bigram: Optional[tuple] = None  # (buckets, mul_prev, mul_cur)
    loop: Optional[tuple] = None  # (start, stop, times)

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "FilulixConfig":
        if document.get("architecture") != ARCHITECTURE:
            raise InvalidValue("architecture", document.get("architecture"), f"expected {ARCHITECTURE!r}")
        vocab, width = _int(document, "vocab"), _int(document, "width")
        eps = _num(document, "norm.eps")
        if not 0.0 < eps < 1.0:
            raise InvalidValue("norm.eps", eps, "expected a small positive number")
        streams = document.get("streams")
        if streams is not None:
            streams = _int(document, "streams")
        embedding = document.get("embedding") or {}
        scale = _num(document, "embedding.scale") if embedding.get("scale") is not None else 1.0
        bigram = None
        if embedding.get("bigram") is not None:
            bigram = (_int(document, "embedding.bigram.buckets"), _int(document, "embedding.bigram.mul_prev", 0),
                      _int(document, "embedding.bigram.mul_cur", 0))
        layers = _get(document, "layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidValue("layers", layers, "expected a non-empty list of layers")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer)
        loop = None
        if document.get("loop") is not None:
            loop = (_int(document, "loop.start", 0), _int(document, "loop.stop", 0), _int(document, "loop.times", 1))
            if not loop[0] <= loop[1] <= len(layers):
                raise InvalidValue("loop", document["loop"], f"start <= stop <= {len(layers)} layers is needed")
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(copy.deepcopy(layers)), streams=streams,
                   embedding_scale=scale, bigram=bigram, loop=loop)

    @staticmethod
    def _check_layer(i: int, layer) -> None:
        at = f"layers[{i}]"
        if not isinstance(layer, Mapping):
            raise InvalidValue(at, layer, "expected an object")
        kind = layer.get("type")
        if kind == WKV:
            _int(layer, "mixer.heads"), _int(layer, "mixer.dim")
        elif kind == PARALLEL:
            for key in ("left.heads", "left.kv_heads", "left.dim", "left.vdim", "left.mask.size", "left.mask.pool",
                        "right.heads", "right.dim", "right.vdim"):
                _int(layer, f"mixer.{key}")
            for key in ("left.scale", "left_scale", "right_scale"):
                _num(layer, f"mixer.{key}")
            left, right = layer["mixer"]["left"], layer["mixer"]["right"]
            if left["heads"] % left["kv_heads"]:
                raise InvalidValue(f"{at}.mixer.left.kv_heads", left["kv_heads"], f"does not divide {left['heads']} query heads")
            decay = _get(layer, "mixer.right.decay")
            if not isinstance(decay, list) or len(decay) != right["heads"] or not all(isinstance(d, (int, float)) for d in decay):
                raise InvalidValue(f"{at}.mixer.right.decay", decay, f"expected one number per head, {right['heads']} heads")
            if right.get("rot") is not None:
                dims = _int(layer, "mixer.right.rot.dims", 2)
                if dims % 2 or dims > right["dim"]:
                    raise InvalidValue(f"{at}.mixer.right.rot.dims", dims, f"must be even and at most the head size {right['dim']}")
                if _num(layer, "mixer.right.rot.base") <= 0:
                    raise InvalidValue(f"{at}.mixer.right.rot.base", right["rot"]["base"], "expected a positive base")
        else:
            raise InvalidValue(f"{at}.type", kind, f"expected {WKV!r} or {PARALLEL!r}")
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp.get("kind") != DENSE:
                raise InvalidValue(f"{at}.mlp.kind", mlp.get("kind"), f"expected {DENSE!r}")
            _int(layer, "mlp.ff")

    def to_dict(self) -> dict:
        document = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                    "layers": copy.deepcopy(list(self.layers))}
        if self.streams is not None:
            document["streams"] = self.streams
        embedding = {"scale": self.embedding_scale}
        if self.bigram is not None:
            embedding["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        document["embedding"] = embedding
        if self.loop is not None:
            document["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return document

    def run_order(self) -> list:
        """Layer indices in the order they run: the looped run ``times`` times in a row."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def build_plan(config: FilulixConfig) -> ModelPlan:
    width, eps = config.width, config.eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"tensor": name, "size": width, "eps": eps, "offset": 1.0})

    layers, unused = [], []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}"
        m = layer["mixer"]
        if layer["type"] == WKV:
            p = f"{prefix}.mix"
            mixer = PartSpec("wkv_time_mix", {
                "hidden_size": width, "num_heads": m["heads"], "head_dim": m["dim"], "eps": eps, "decay_rank": m.get("rank"),
                "mu": {c: f"{p}.mu.{c}" for c in ("r", "k", "v", "g", "w")},
                "r_proj": f"{p}.r", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "g_proj": f"{p}.g",
                "decay_down": f"{p}.w1", "decay_up": f"{p}.w2", "decay_bias": f"{p}.w0",
                "bonus": f"{p}.u", "out_norm": f"{p}.norm", "out_proj": f"{p}.o",
            })
        else:
            left, right = m["left"], m["right"]
            p = f"{prefix}.mix.left"
            attention = PartSpec("pooled_window_attention", {
                "hidden_size": width, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
                "v_head_dim": left["vdim"], "scale": left["scale"], "window": left["mask"]["size"], "pool": left["mask"]["pool"],
                "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "out_proj": f"{p}.o",
            })
            p = f"{prefix}.mix.right"
            rot = right.get("rot")
            position = PartSpec("rope_half_split", {"theta": rot["base"], "rotary_dim": rot["dims"]}) if rot else PartSpec("none")
            retention = PartSpec("retention", {
                "hidden_size": width, "num_heads": right["heads"], "head_dim": right["dim"], "v_head_dim": right["vdim"],
                "decay": tuple(right["decay"]), "eps": eps, "position": position,
                "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "g_proj": f"{p}.g", "out_proj": f"{p}.o",
            })
            mixer = PartSpec("parallel_mixer", {"branches": ((attention, m["left_scale"]), (retention, m["right_scale"]))})
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            feed_forward = PartSpec("swiglu", {
                "hidden_size": width, "intermediate_size": mlp["ff"],
                "gate": f"{prefix}.mlp.gate", "up": f"{prefix}.mlp.up", "down": f"{prefix}.mlp.down",
            })
        else:
            unused += [f"{prefix}.norm2"] + [f"{prefix}.hc2.{k}" for k in ("in", "out", "mix")]
        if config.streams is not None:
            io = lambda q: {"read": f"{prefix}.hc{q}.in", "write": f"{prefix}.hc{q}.out", "mix": f"{prefix}.hc{q}.mix"}  # noqa: E731
            block = PartSpec("hyper_pre_norm", {"copies": config.streams, "mixer_io": io(1), "ff_io": io(2)})
        else:
            block = PartSpec("pre_norm")
        layers.append(LayerSpec(
            name=prefix, block=block, mixer=mixer, mixer_norm=norm(f"{prefix}.norm1"),
            feed_forward=feed_forward, feed_forward_norm=norm(f"{prefix}.norm2") if feed_forward is not None else None,
        ))

    if config.bigram is not None:
        buckets, mul_prev, mul_cur = config.bigram
        embedding = PartSpec("hashed_pair_embedding", {
            "tensor": "embed", "pair_tensor": "bigram", "vocab_size": config.vocab, "hidden_size": width,
            "scale": config.embedding_scale, "buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur,
        })
    else:
        embedding = PartSpec("token_embedding", {"tensor": "embed", "vocab_size": config.vocab, "hidden_size": width,
                                                 "scale": config.embedding_scale})
    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        embedding=embedding,
        layers=tuple(layers),
        order=tuple(RunEntry(layer=i) for i in config.run_order()),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tied_to": None, "tensor": "head"}),
        unused_tensors=tuple(unused),
    )


register_architecture(ARCHITECTURE, FilulixConfig, build_plan)
