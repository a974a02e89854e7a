"""Zipelix: a pre-norm decoder over several copies of the residual stream (hyper-connections: every sublayer reads a
weighted sum of the copies and writes back through a mixing matrix), whose mixer is, layer by layer, attention through
a latent (queries straight from the input, interleaved rotary pairs, a sigmoid output gate; a layer may read the
latents that an earlier layer cached instead of making its own) or retention (a decayed linear recurrence per head with
rotate-half encoding, a norm per head and a SiLU gate); the feed-forward is a gated dense one, a mixture of such
experts with a gated shared expert, or absent.  RMS norms with plain weights, no position table, the embedding table as
the output head, and a tanh cap on the logits.  This file only translates a `ZipelixConfig` into a `ModelSpec`: every
mechanism is a registered part.

Checkpoint names: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, l<i>.hc1.{in,out,mix}, l<i>.hc2.{in,out,mix},
final.norm."""
from __future__ import annotations

from ..config import ZipelixConfig, register_architecture
from ..parts import LayerSpec, PartSpec
from .decoder import ModelSpec, ScheduleEntry


def build_zipelix(config: ZipelixConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = PartSpec("rmsnorm", {"hidden": width, "eps": eps, "tensor": ""})
    streams = config.streams or 1
    layers, schedule = [], []
    for i, layer in enumerate(config.layers):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            source = m.get("kv_from")
            mixer = PartSpec("latent_attention", {
                "hidden": width, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": None, "scale": m["scale"], "window": None, "norm_eps": eps, "rot": m.get("rot"),
                "rot_pairs": True, "gate": "sigmoid", "shared_cache": source is not None})
            # a layer that reads another layer's latents uses that layer's cache and appends nothing
            schedule.append(ScheduleEntry(i, cache=i if source is None else int(source), writes=source is None))
        else:
            mixer = PartSpec("retention", {
                "hidden": width, "heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"], "decay": list(m["decay"]),
                "rot": m.get("rot"), "norm_eps": eps})
            schedule.append(ScheduleEntry(i, cache=None))
        mlp = layer.get("mlp")
        if mlp is None:
            feed_forward = None
        elif mlp["kind"] == "dense":
            feed_forward = PartSpec("swiglu", {"hidden": width, "intermediate": mlp["ff"],
                                               "names": {"gate": "gate", "up": "up", "down": "down"}})
        else:
            shared = mlp.get("shared")
            feed_forward = PartSpec("expert_mixture", {
                "hidden": width, "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                "router_scale": mlp["router"]["scale"], "intermediate": mlp["expert"]["ff"],
                "shared": {"intermediate": shared["ff"]} if shared else None})
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=feed_forward, norm=norm, arrangement="hyper",
            options={"streams": streams, "learned": config.streams is not None},
            names={"norm1": "norm1", "norm2": "norm2", "mixer": "mix.", "feed_forward": "mlp.", "hc1": "hc1.", "hc2": "hc2."}))
    return ModelSpec(hidden_size=width, vocab_size=config.vocab, max_positions=None, layers=layers, final_norm=norm,
                     schedule=schedule, embedding_name="embed", head_name=None, layer_prefix="l{}.",
                     final_norm_prefix="final.norm", streams=streams, logit_softcap=config.logit_softcap)


register_architecture(("Zipelix",), ZipelixConfig, build_zipelix)
