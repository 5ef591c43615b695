"""Zetavik: typed configuration and model plan.

A decoder of parallel layers: one layer norm (a weight, no bias) per layer, whose output
both the mixer and the feed-forward read, and both outputs are added to the residual stream.
A layer's mixer is one of ``latent_attention`` (softmax attention over a cached latent and one
rotated key part shared by the heads, queries through a latent of their own, a sigmoid gate per
head), ``lightning`` (linear attention with one fixed decay per head) or ``mamba2`` (a
state-space recurrence behind a short causal convolution); its feed-forward is ``dense``
(squared ReLU), ``moe`` (softmax router, group-limited choice of ``top`` experts, optionally a
shared expert) or absent.  The head is the embedding table.

config.json keys: ``architecture``, ``vocab``, ``width``, ``norm.eps`` and ``layers``: a list of
``{"type", "mixer", "mlp"}`` with, for ``latent_attention``, ``mixer.{heads, dim, rot_dim, vdim,
q_rank, kv_rank, scale, rot.{dims, base}}``; for ``lightning``, ``mixer.{heads, dim, vdim,
decay}``; for ``mamba2``, ``mixer.{heads, vdim, state, groups, conv, norm_groups}``; and
``mlp.{kind, ff}`` or ``mlp.{kind, expert.ff, router.{experts, top, scale, groups.{count, keep}},
shared.ff}`` or null.
Tensor names: ``embed``, ``final.norm`` and, for layer ``i``, ``l<i>.norm1``, ``l<i>.mix.*``
(``dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o`` / ``q, k, v, g, norm, o`` / ``in, conv, conv.b,
dt_bias, A_log, D, norm, o``), ``l<i>.mlp.{up, down}`` or ``l<i>.mlp.{router, e<j>.{gate, up,
down}, shared.{gate, up, down}}``.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Mapping

from ..parts.plan import LayerSpec, ModelPlan, PartSpec, RunEntry
from .errors import ConfigMissing, InvalidValue
from .registry import register_architecture

ARCHITECTURE = "Zetavik"
LATENT = "latent_attention"
LIGHTNING = "lightning"
MAMBA2 = "mamba2"
DENSE = "dense"
MOE = "moe"


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
class ZetavikConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple  # the documents of the layers, checked

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "ZetavikConfig":
        if document.get("architecture") != ARCHITECTURE:
            raise InvalidValue("architecture", document.get("architecture"), f"expected {ARCHITECTURE!r}")
        vocab, width = _int(document, "vocab"), _int(document, "width")
        eps = _num(document, "norm.eps")
        if not 0.0 < eps < 1.0:
            raise InvalidValue("norm.eps", eps, "expected a small positive number")
        layers = _get(document, "layers")
        if not isinstance(layers, list) or not layers:
            raise InvalidValue("layers", layers, "expected a non-empty list of layers")
        for i, layer in enumerate(layers):
            cls._check_layer(i, layer)
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(copy.deepcopy(layers)))

    @staticmethod
    def _check_layer(i: int, layer) -> None:
        at = f"layers[{i}]"
        if not isinstance(layer, Mapping):
            raise InvalidValue(at, layer, "expected an object")
        kind = layer.get("type")
        if kind == LATENT:
            for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "rot.dims"):
                _int(layer, f"mixer.{key}")
            _num(layer, "mixer.scale")
            m = layer["mixer"]
            if _num(layer, "mixer.rot.base") <= 0:
                raise InvalidValue(f"{at}.mixer.rot.base", m["rot"]["base"], "expected a positive base")
            if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
                raise InvalidValue(f"{at}.mixer.rot.dims", m["rot"]["dims"], f"must be even and at most rot_dim = {m['rot_dim']}")
        elif kind == LIGHTNING:
            for key in ("heads", "dim", "vdim"):
                _int(layer, f"mixer.{key}")
            decay = _get(layer, "mixer.decay")
            heads = layer["mixer"]["heads"]
            if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                raise InvalidValue(f"{at}.mixer.decay", decay, f"expected one number per head, {heads} heads")
        elif kind == MAMBA2:
            for key in ("heads", "vdim", "state", "groups", "norm_groups"):
                _int(layer, f"mixer.{key}")
            _int(layer, "mixer.conv", 2)
            m = layer["mixer"]
            if m["heads"] % m["groups"]:
                raise InvalidValue(f"{at}.mixer.groups", m["groups"], f"does not divide {m['heads']} heads")
            if (m["heads"] * m["vdim"]) % m["norm_groups"]:
                raise InvalidValue(f"{at}.mixer.norm_groups", m["norm_groups"], f"does not divide the inner width {m['heads'] * m['vdim']}")
        else:
            raise InvalidValue(f"{at}.type", kind, f"expected {LATENT!r}, {LIGHTNING!r} or {MAMBA2!r}")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if mlp.get("kind") == DENSE:
            _int(layer, "mlp.ff")
        elif mlp.get("kind") == MOE:
            experts, top = _int(layer, "mlp.router.experts"), _int(layer, "mlp.router.top")
            _int(layer, "mlp.expert.ff"), _num(layer, "mlp.router.scale")
            if top > experts:
                raise InvalidValue(f"{at}.mlp.router.top", top, f"more than the {experts} experts")
            groups = mlp["router"].get("groups")
            if groups is not None:
                count, keep = _int(layer, "mlp.router.groups.count"), _int(layer, "mlp.router.groups.keep")
                if experts % count or keep > count:
                    raise InvalidValue(f"{at}.mlp.router.groups", groups, f"count must divide {experts} experts and keep be at most count")
                if keep * (experts // count) < top:
                    raise InvalidValue(f"{at}.mlp.router.groups", groups, f"{keep} groups hold fewer than top = {top} experts")
            if mlp.get("shared") is not None:
                _int(layer, "mlp.shared.ff")
        else:
            raise InvalidValue(f"{at}.mlp.kind", mlp.get("kind"), f"expected {DENSE!r} or {MOE!r}")

    def to_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "layers": copy.deepcopy(list(self.layers))}


def _mixer_spec(kind: str, m: Mapping[str, Any], p: str, width: int, eps: float) -> PartSpec:
    if kind == LATENT:
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
            "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": eps,
            "position": PartSpec("rope_half_split", {"theta": m["rot"]["base"], "rotary_dim": m["rot"]["dims"]}),
            "q_down": f"{p}.dq", "q_norm": f"{p}.dq.norm", "q_up": f"{p}.uq", "kv_down": f"{p}.dkv", "kv_norm": f"{p}.dkv.norm",
            "k_up": f"{p}.uk", "v_up": f"{p}.uv", "gate": f"{p}.g", "out_proj": f"{p}.o",
        })
    if kind == LIGHTNING:
        return PartSpec("lightning_attention", {
            "hidden_size": width, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "decay": tuple(m["decay"]), "eps": eps,
            "q_proj": f"{p}.q", "k_proj": f"{p}.k", "v_proj": f"{p}.v", "g_proj": f"{p}.g", "out_norm": f"{p}.norm", "out_proj": f"{p}.o",
        })
    return PartSpec("mamba2", {
        "hidden_size": width, "num_heads": m["heads"], "v_head_dim": m["vdim"], "state": m["state"], "groups": m["groups"],
        "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": eps,
        "in_proj": f"{p}.in", "conv": f"{p}.conv", "conv_bias": f"{p}.conv.b", "dt_bias": f"{p}.dt_bias", "a_log": f"{p}.A_log",
        "skip": f"{p}.D", "out_norm": f"{p}.norm", "out_proj": f"{p}.o",
    })


def _expert_names(p: str) -> dict:
    return {"gate": f"{p}.gate", "up": f"{p}.up", "down": f"{p}.down"}


def _ff_spec(mlp: Mapping[str, Any], p: str, width: int) -> PartSpec:
    if mlp["kind"] == DENSE:
        return PartSpec("relu2_ff", {"hidden_size": width, "intermediate_size": mlp["ff"], "up": f"{p}.up", "down": f"{p}.down"})
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    shared = None
    if mlp.get("shared") is not None:
        shared = PartSpec("swiglu", {"hidden_size": width, "intermediate_size": mlp["shared"]["ff"], **_expert_names(f"{p}.shared")})
    return PartSpec("routed_experts", {
        "hidden_size": width, "intermediate_size": mlp["expert"]["ff"], "experts": r["experts"], "top": r["top"],
        "group_count": groups["count"], "group_keep": groups["keep"], "scale": r["scale"], "scores": "softmax", "renormalize": False,
        "router": f"{p}.router", "expert_names": tuple(_expert_names(f"{p}.e{e}") for e in range(r["experts"])), "shared": shared,
    })


def build_plan(config: ZetavikConfig) -> ModelPlan:
    width, eps = config.width, config.eps
    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}"
        mlp = layer.get("mlp")
        layers.append(LayerSpec(
            name=prefix,
            block=PartSpec("parallel_pre_norm"),
            mixer=_mixer_spec(layer["type"], layer["mixer"], f"{prefix}.mix", width, eps),
            mixer_norm=PartSpec("layernorm", {"tensor": f"{prefix}.norm1", "size": width, "eps": eps}),
            feed_forward=_ff_spec(mlp, f"{prefix}.mlp", width) if mlp is not None else None,
        ))
    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=width,
        vocab_size=config.vocab,
        embedding=PartSpec("token_embedding", {"tensor": "embed", "vocab_size": config.vocab, "hidden_size": width}),
        layers=tuple(layers),
        order=tuple(RunEntry(layer=i) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", {"tensor": "final.norm", "size": width, "eps": eps}),
        head=PartSpec("linear_head", {"vocab_size": config.vocab, "hidden_size": width, "tied_to": "embed", "tensor": None}),
    )


register_architecture(ARCHITECTURE, ZetavikConfig, build_plan)
