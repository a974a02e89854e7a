"""Typed configuration of the Pilutar decoder, read from config.json's own keys.

    architecture    "Pilutar"
    vocab, width
    norm.eps
    embedding.scale the embedding output's factor (absent: 1)
    logit_scale     the logits' factor (absent: 1)
    layers[]        type: which mixer the layer has; mixer: its sizes; mlp: its feed-forward, or null for none
      "latent_attention"  mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims} (absent: nothing turns),
                                 mask {size} (absent: every earlier key is seen)}
      "parallel"          mixer {left {heads, kv_heads, dim, vdim, scale, softcap (absent: none), rot, mask},
                                 right {heads, dim, vdim, tau, rank (absent: whatever the stored tensors have)},
                                 left_scale, right_scale}
      mlp {kind "dense", ff}
      mlp {kind "moe", expert {ff}, router {experts, top, identity (absent: 0), groups {count, keep} (absent: none)},
           shared {ff} (absent: no shared expert)}

Every size and constant is a parameter.  The design has no table of positions and no limit of its own on a request's
length.  `initializer_range` (absent: 0.02) only serves the random-weights mode, which also needs `right.rank`."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .model_config import ConfigError
from .nafevik_config import _number, _positive_int, _section

MIXER_TYPES = ("latent_attention", "parallel")
MLP_KINDS = ("dense", "moe")


def _rot(mixer: dict, limit: int, where: str) -> None:
    if mixer.get("rot") is None:                 # absent: nothing is rotated
        return
    rot = _section(mixer, "rot", where)
    dims = _positive_int(rot.get("dims"), f"{where}.rot.dims")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}")
    _number(rot.get("base"), f"{where}.rot.base")


def _mask(mixer: dict, where: str) -> None:
    if mixer.get("mask") is not None:
        _positive_int(_section(mixer, "mask", where).get("size"), f"{where}.mask.size")


def _mlp(mlp, where: str) -> None:
    if mlp is None:
        return
    if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind is not known; known: {MLP_KINDS}")
    if mlp["kind"] == "dense":
        _positive_int(mlp.get("ff"), f"{where}.ff")
        return
    _positive_int(_section(mlp, "expert", where).get("ff"), f"{where}.expert.ff")
    router = _section(mlp, "router", where)
    experts = _positive_int(router.get("experts"), f"{where}.router.experts")
    top = _positive_int(router.get("top"), f"{where}.router.top")
    identity = router.get("identity", 0)
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(f"config.json: {where}.router.identity must be a non-negative integer")
    outputs = experts + identity
    if top > outputs:
        raise ConfigError(f"config.json: {where}.router.top exceeds the number of router outputs")
    if router.get("groups") is not None:
        groups = _section(router, "groups", f"{where}.router")
        count = _positive_int(groups.get("count"), f"{where}.router.groups.count")
        keep = _positive_int(groups.get("keep"), f"{where}.router.groups.keep")
        if outputs % count or keep > count or keep * (outputs // count) < top:
            raise ConfigError(f"config.json: {where}.router.groups: count must divide the router's outputs, keep be at most "
                              "count, and the kept groups hold at least `top` outputs")
    if mlp.get("shared") is not None:
        _positive_int(_section(mlp, "shared", where).get("ff"), f"{where}.shared.ff")


@dataclass(frozen=True)
class PilutarConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: tuple                      # of dicts as in config.json (validated)
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    initializer_range: float = 0.02
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "PilutarConfig":
        width = _positive_int(raw.get("width"), "width")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not known; known: {MIXER_TYPES}")
            where = f"layers[{i}].mixer"
            mixer = _section(layer, "mixer", f"layers[{i}]")
            if kind == "latent_attention":
                for key in ("heads", "dim", "vdim", "rot_dim", "kv_rank"):
                    _positive_int(mixer.get(key), f"{where}.{key}")
                _number(mixer.get("scale"), f"{where}.scale")
                _rot(mixer, mixer["rot_dim"], where)
                _mask(mixer, where)
            else:
                left, right = _section(mixer, "left", where), _section(mixer, "right", where)
                for key in ("heads", "kv_heads", "dim", "vdim"):
                    _positive_int(left.get(key), f"{where}.left.{key}")
                if left["heads"] % left["kv_heads"]:
                    raise ConfigError(f"config.json: {where}.left.heads must be a multiple of kv_heads")
                _number(left.get("scale"), f"{where}.left.scale")
                if left.get("softcap") is not None:
                    _number(left.get("softcap"), f"{where}.left.softcap")
                _rot(left, left["dim"], f"{where}.left")
                _mask(left, f"{where}.left")
                for key in ("heads", "dim", "vdim"):
                    _positive_int(right.get(key), f"{where}.right.{key}")
                _number(right.get("tau"), f"{where}.right.tau")
                if right.get("rank") is not None:
                    _positive_int(right.get("rank"), f"{where}.right.rank")
                for key in ("left_scale", "right_scale"):
                    _number(mixer.get(key, 1.0), f"{where}.{key}", positive=False)
            _mlp(layer.get("mlp"), f"layers[{i}].mlp")
            checked.append(copy.deepcopy(layer))
        embedding = raw.get("embedding") or {}
        known = {"architecture", "vocab", "width", "norm", "layers", "embedding", "logit_scale", "initializer_range"}
        return cls(width=width, vocab=_positive_int(raw.get("vocab"), "vocab"),
                   norm_eps=_number(_section(raw, "norm", "the model").get("eps"), "norm.eps"),
                   layers=tuple(checked),
                   embedding_scale=_number(embedding.get("scale", 1.0), "embedding.scale", positive=False),
                   logit_scale=_number(raw.get("logit_scale", 1.0), "logit_scale", positive=False),
                   initializer_range=float(raw.get("initializer_range", 0.02)),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": "Pilutar", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
               "layers": copy.deepcopy(list(self.layers))}
        if self.initializer_range != 0.02:
            out["initializer_range"] = self.initializer_range
        out.update(self.extra)
        return out
