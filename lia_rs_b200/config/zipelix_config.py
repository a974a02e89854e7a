"""Typed configuration of the Zipelix decoder, read from config.json's own keys.

    architecture    "Zipelix"
    vocab, width
    norm.eps
    streams         copies of the residual stream (hyper-connections); absent: one stream and plain residual sums
    logit_softcap   cap of the logits, cap * tanh(logits / cap); absent: none
    layers[]        type: which mixer the layer has; mixer: its sizes; mlp: its feed-forward, or null for none
      "latent_attention"  mixer {heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims} (absent: nothing turns),
                                 kv_from (absent: the layer has a cache of its own; j: it reads layer j's)}
      "retention"         mixer {heads, dim, vdim, decay [one per head], rot {base, dims} (absent: nothing turns)}
      mlp {kind "dense", ff}
      mlp {kind "moe", expert {ff}, router {experts, top, scale}, shared {ff} (absent: no shared expert)}

Every size and constant is a parameter.  The design has no table of positions and no limit of its own on a request's
length; the output head is the embedding table.  `initializer_range` (absent: 0.02) only serves the random-weights mode."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Optional

from .model_config import ConfigError
from .nafevik_config import _number, _positive_int, _section

MIXER_TYPES = ("latent_attention", "retention")
MLP_KINDS = ("dense", "moe")


def _rot(mixer: dict, limit: int, where: str) -> None:
    if mixer.get("rot") is None:                 # absent: nothing is rotated
        return
    rot = _section(mixer, "rot", where)
    dims = _positive_int(rot.get("dims"), f"{where}.rot.dims")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}")
    if not _number(rot.get("base"), f"{where}.rot.base") > 0:
        raise ConfigError(f"config.json: {where}.rot.base must be positive")


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
    if top > experts:
        raise ConfigError(f"config.json: {where}.router.top exceeds the number of experts")
    _number(router.get("scale"), f"{where}.router.scale")
    if mlp.get("shared") is not None:
        _positive_int(_section(mlp, "shared", where).get("ff"), f"{where}.shared.ff")


@dataclass(frozen=True)
class ZipelixConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: tuple                      # of dicts as in config.json (validated)
    streams: Optional[int] = None
    logit_softcap: Optional[float] = None
    initializer_range: float = 0.02
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "ZipelixConfig":
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
            heads = _positive_int(mixer.get("heads"), f"{where}.heads")
            dim = _positive_int(mixer.get("dim"), f"{where}.dim")
            _positive_int(mixer.get("vdim"), f"{where}.vdim")
            if kind == "latent_attention":
                for key in ("rot_dim", "kv_rank"):
                    _positive_int(mixer.get(key), f"{where}.{key}")
                _number(mixer.get("scale"), f"{where}.scale")
                _rot(mixer, mixer["rot_dim"], where)
                source = mixer.get("kv_from")
                if source is not None:
                    if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
                        raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer")
                    other = checked[source]
                    if other["type"] != "latent_attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.kv_from must name a latent-attention layer with a cache of its own")
                    if any(other["mixer"].get(key) != mixer.get(key) for key in ("kv_rank", "rot_dim", "rot")):
                        raise ConfigError(f"config.json: {where}: kv_rank, rot_dim and rot must equal those of layer {source}")
            else:
                decay = mixer.get("decay")
                if not isinstance(decay, list) or len(decay) != heads:
                    raise ConfigError(f"config.json: {where}.decay must list one number per head")
                for j, a in enumerate(decay):
                    if not 0.0 < _number(a, f"{where}.decay[{j}]") <= 1.0:
                        raise ConfigError(f"config.json: {where}.decay[{j}] must lie in (0, 1]")
                _rot(mixer, dim, where)
            _mlp(layer.get("mlp"), f"layers[{i}].mlp")
            checked.append(copy.deepcopy(layer))
        streams = raw.get("streams")
        if streams is not None:
            streams = _positive_int(streams, "streams")
        cap = raw.get("logit_softcap")
        if cap is not None and not _number(cap, "logit_softcap") > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        known = {"architecture", "vocab", "width", "norm", "layers", "streams", "logit_softcap", "initializer_range"}
        return cls(width=width, vocab=_positive_int(raw.get("vocab"), "vocab"),
                   norm_eps=_number(_section(raw, "norm", "the model").get("eps"), "norm.eps"),
                   layers=tuple(checked), streams=streams, logit_softcap=None if cap is None else float(cap),
                   initializer_range=float(raw.get("initializer_range", 0.02)),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": "Zipelix", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(list(self.layers))}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.initializer_range != 0.02:
            out["initializer_range"] = self.initializer_range
        out.update(self.extra)
        return out
