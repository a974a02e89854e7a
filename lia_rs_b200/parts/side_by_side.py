"""Several mixers side by side: all read the same input, and the result is the weighted sum of theirs,

    mixer(x) = sum_i scale_i * mixer_i(x).

Each member is a registered mixer with its own parameters and checkpoint prefix; every member adds its share into the
residual stream itself (a mixer's `forward` does `residual += scale * f(x)`, so the weights ride on the members' last
products and no sum is formed anywhere else).  At most one member may ask for a paged cache and at most one for
per-request state: the layer's cache and state are handed to those.

Parameters: `members`: a list of {"kind", "params", "prefix", "scale"}."""
from __future__ import annotations

from .base import MIXERS, Mixer, lookup, register_mixer


@register_mixer("side_by_side")
class SideBySide(Mixer):
    can_store = False

    @staticmethod
    def _members(params):
        return [(lookup(MIXERS, m["kind"], "mixer"), m["params"], m.get("prefix", ""), float(m.get("scale", 1.0)))
                for m in params["members"]]

    @staticmethod
    def check_params(params):
        members = SideBySide._members(params)
        if not members:
            raise ValueError("mixers side by side: at least one member")
        for cls, member_params, _, _ in members:
            cls.check_params(member_params)
        if sum(cls.cache_request(p) is not None for cls, p, _, _ in members) > 1 or \
                sum(cls.state_request(p) is not None for cls, p, _, _ in members) > 1:
            raise ValueError("mixers side by side: at most one member with a paged cache and one with per-request state")

    @staticmethod
    def tensor_specs(params, prefix):
        return [spec for cls, p, member_prefix, _ in SideBySide._members(params) for spec in cls.tensor_specs(p, prefix + member_prefix)]

    @staticmethod
    def cache_request(params):
        for cls, p, _, _ in SideBySide._members(params):
            if cls.cache_request(p) is not None:
                return cls.cache_request(p)
        return None

    @staticmethod
    def state_request(params):
        for cls, p, _, _ in SideBySide._members(params):
            if cls.state_request(p) is not None:
                return cls.state_request(p)
        return None

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.members = []
        for cls, p, member_prefix, scale in self._members(params):
            part = cls(p, tensors, prefix + member_prefix, runtime)
            if part.output_bias is not None:
                raise ValueError("mixers side by side: a member's output bias is not added")
            self.members.append((part, scale, cls.cache_request(p) is not None, cls.state_request(p) is not None))
        self.graph_safe = all(part.graph_safe for part, _, _, _ in self.members)
        self.takes_deferred_norm = all(part.takes_deferred_norm for part, _, _, _ in self.members)

    def graph_key(self, ctx) -> tuple:
        key = ()
        for part, _, _, _ in self.members:
            key += part.graph_key(ctx)
        return key

    def forward(self, ctx, x, residual, scale, kv=None, state=None):
        for part, weight, wants_cache, wants_state in self.members:
            part.forward(ctx, x, residual, scale * weight, kv=kv if wants_cache else None, state=state if wants_state else None)
