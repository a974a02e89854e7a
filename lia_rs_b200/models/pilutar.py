"""Pilutar: a decoder of parallel layers, x <- x + mixer(h) + feed_forward(h) with one layer norm (weight and bias)
h = LN(x) that both sublayers read.  The mixer is, layer by layer, attention through a latent (queries straight from the
input, interleaved rotary pairs on a rotated part that all heads share, a window, one sigmoid gate per head), or two
mixers side by side whose outputs are added with fixed weights: windowed grouped-query softmax attention (biases on q, k
and v, one RMS norm over the whole q projection and one over the whole k projection, rotation in halves, a tanh cap on the
scores) and gated linear attention (a linear recurrence with a decay per token and key channel, a norm per head and a SiLU
gate).  The feed-forward is a dense one with a ReLU gate, a mixture of ungated squared-ReLU experts (a correction of the
scores for the choice, groups of outputs, identity outputs, renormalised weights, a gated shared expert), or absent.  The
embedding output and the logits have fixed factors; the output head is a matrix of its own.  This file only translates a
`PilutarConfig` into a `ModelSpec`: every mechanism is a registered part.

Checkpoint names: embed, head, final.norm, final.norm.b, l<i>.norm1, l<i>.norm1.b, l<i>.mix.* (l<i>.mix.left.*,
l<i>.mix.right.*), l<i>.mlp.*."""
from __future__ import annotations

from ..config import PilutarConfig, register_architecture
from ..parts import LayerSpec, PartSpec
from .decoder import ModelSpec


def _window(mixer: dict):
    return int(mixer["mask"]["size"]) if mixer.get("mask") else None


def build_pilutar(config: PilutarConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = PartSpec("layernorm", {"hidden": width, "eps": eps, "tensor": "", "bias_tensor": ".b"})
    layers = []
    for layer in config.layers:
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden": width, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": None, "scale": m["scale"], "window": _window(m), "norm_eps": eps,
                "rot": m.get("rot"), "rot_pairs": True, "gate": "sigmoid_head"})
        else:
            left, right = m["left"], m["right"]
            attention = {
                "hidden": width, "heads": left["heads"], "kv_heads": left["kv_heads"], "head_dim": left["dim"],
                "v_head_dim": left["vdim"], "scale": left["scale"], "softcap": left.get("softcap"), "window": _window(left),
                "rot": left.get("rot"), "biases": "qkv", "qk_norm": "whole", "norm_eps": eps}
            recurrence = {
                "hidden": width, "heads": right["heads"], "head_dim": right["dim"], "v_head_dim": right["vdim"],
                "tau": right["tau"], "norm_eps": eps, "decay_rank": right.get("rank")}
            mixer = PartSpec("side_by_side", {"members": [
                {"kind": "sink_attention", "params": attention, "prefix": "left.", "scale": m.get("left_scale", 1.0)},
                {"kind": "gated_linear_attention", "params": recurrence, "prefix": "right.", "scale": m.get("right_scale", 1.0)}]})
        mlp = layer.get("mlp")
        if mlp is None:
            feed_forward = None
        elif mlp["kind"] == "dense":
            feed_forward = PartSpec("swiglu", {"hidden": width, "intermediate": mlp["ff"], "gate_activation": "relu",
                                               "names": {"gate": "gate", "up": "up", "down": "down"}})
        else:
            router, shared = mlp["router"], mlp.get("shared")
            feed_forward = PartSpec("expert_mixture", {
                "hidden": width, "experts": router["experts"], "top": router["top"], "router_scale": 1.0,
                "intermediate": mlp["expert"]["ff"], "expert_form": "relu_squared", "identity": router.get("identity", 0),
                "correction": True, "groups": router.get("groups"), "renormalise": True,
                "shared": {"intermediate": shared["ff"]} if shared else None})
        layers.append(LayerSpec(mixer=mixer, feed_forward=feed_forward, norm=norm, arrangement="parallel",
                                names={"norm1": "norm1", "mixer": "mix.", "feed_forward": "mlp."}))
    return ModelSpec(hidden_size=width, vocab_size=config.vocab, max_positions=None, layers=layers, final_norm=norm,
                     embedding_scale=config.embedding_scale, logit_scale=config.logit_scale, embedding_name="embed",
                     head_name="head", layer_prefix="l{}.", final_norm_prefix="final.norm")


register_architecture(("Pilutar",), PilutarConfig, build_pilutar)
