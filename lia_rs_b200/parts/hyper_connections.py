"""`hyper`: a pre-norm layer over several copies of the residual stream (hyper-connections).

A token's residual is `streams` vectors x_1..x_s that lie side by side in one 32-bit row [streams * hidden].  Sublayer q
(the mixer, then the feed-forward if the layer has one) with its coefficients in_q [s], mix_q [s, s] (indexed [from, to])
and out_q [s]:

    u = sum_s in_q[s] x_s;   y = sublayer_q(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   (all t from the old x)

One kernel (csrc/hyper_connections.cu) does a sublayer's write-back together with the read and the norm of the next
sublayer, in one pass over the token's row; a layer's last write-back is left to the layer behind it (`ctx.owed`), which
does it in the pass of its first read, so a layer costs two passes over the streams and the model one more (`settle`).  The sublayers
store their output into a 32-bit buffer of the arrangement.  The norms must be RMS norms (`rms_record`).

`options`: {"streams": s, "learned": bool (default True)}.  Without learned coefficients (in = out = 1, mix = the
identity; only with one stream) the layer is the plain pre-norm layer x <- x + sublayer(norm(x)).  Checkpoint names:
`names["norm1"]`, `["mixer"]`, `["norm2"]`, `["feed_forward"]`, and `["hc1"]`, `["hc2"]` (defaults "hc1.", "hc2.") ahead of
"in", "out" and "mix"."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import FEED_FORWARDS, MIXERS, NORMS, Arrangement, lookup, register_arrangement


@register_arrangement("hyper")
class HyperConnectionBlock(Arrangement):
    @staticmethod
    def streams(spec) -> int:
        return int(spec.options.get("streams", 1))

    @staticmethod
    def _classes(spec):
        """[(class, params, place)] of the parts that exist."""
        out = [(lookup(NORMS, spec.norm_at("norm1").kind, "norm"), spec.norm_at("norm1").params, "norm1"),
               (lookup(MIXERS, spec.mixer.kind, "mixer"), spec.mixer.params, "mixer")]
        if spec.feed_forward is not None:
            out += [(lookup(NORMS, spec.norm_at("norm2").kind, "norm"), spec.norm_at("norm2").params, "norm2"),
                    (lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward"), spec.feed_forward.params, "feed_forward")]
        return out

    @staticmethod
    def _coefficient_places(spec):
        if not spec.options.get("learned", True):
            return []
        return [spec.names.get("hc1", "hc1.")] + ([spec.names.get("hc2", "hc2.")] if spec.feed_forward is not None else [])

    @staticmethod
    def check(spec) -> None:
        for cls, params, _ in HyperConnectionBlock._classes(spec):
            cls.check_params(params)
        streams = HyperConnectionBlock.streams(spec)
        if not 1 <= streams <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"hyper-connections: {streams} streams; the kernel takes 1..{ops.HYPER_MAX_STREAMS}")
        if not spec.options.get("learned", True) and streams != 1:
            raise ValueError("hyper-connections: several streams need learned coefficients")
        if float(spec.residual_scale) != 1.0:
            raise ValueError("the hyper-connection arrangement takes no residual scale (the out coefficients are it)")

    @staticmethod
    def tensor_specs(spec, prefix: str) -> list:
        specs = [t for cls, params, place in HyperConnectionBlock._classes(spec)
                 for t in cls.tensor_specs(params, prefix + spec.names[place])]
        s = HyperConnectionBlock.streams(spec)
        for place in HyperConnectionBlock._coefficient_places(spec):
            specs += [TensorSpec(prefix + place + "in", (s,), kind="norm"), TensorSpec(prefix + place + "out", (s,), kind="norm"),
                      TensorSpec(prefix + place + "mix", (s, s), kind="identity")]
        return specs

    def __init__(self, spec, tensors: dict, prefix: str, runtime):
        self.runtime = runtime
        self.n_streams = self.streams(spec)
        parts = {place: cls(params, tensors, prefix + spec.names[place], runtime) for cls, params, place in self._classes(spec)}
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.norms = []
        for place in ("norm1", "norm2"):
            if place in parts:
                record = parts[place].rms_record()
                if record is None:
                    raise ValueError("the hyper-connection arrangement needs RMS norms")
                self.norms.append((record[0].to(torch.float32).contiguous(), float(record[1])))
        if self.mixer.output_bias is not None:
            raise ValueError("the hyper-connection arrangement does not add a mixer's output bias")
        s, device = self.n_streams, runtime.device
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.coefficients = []                       # per sublayer (in [s], mix [s, s], out [s]), 32-bit
        places = self._coefficient_places(spec)
        for q in range(2 if self.feed_forward is not None else 1):
            if places:
                p = prefix + places[q]
                self.coefficients.append((f32(tensors[p + "in"]), f32(tensors[p + "mix"]), f32(tensors[p + "out"])))
            else:
                self.coefficients.append((None, torch.eye(s, dtype=torch.float32, device=device),
                                          torch.ones(s, dtype=torch.float32, device=device)))
        self._parts = list(parts.values())
        self.graph_safe = all(part.graph_safe for part in self._parts)

    def graph_key(self, ctx) -> tuple:
        key = ()
        for part in self._parts:
            key += part.graph_key(ctx)
        return key

    def _sublayer(self, ctx, part, x, y, **more):
        if part.can_store:
            part.forward(ctx, x, y, 1.0, store=True, **more)
        else:
            y.zero_()
            part.forward(ctx, x, y, 1.0, **more)

    def forward(self, ctx, residual, kv=None, state=None):
        s, n = self.n_streams, residual.shape[0]
        hidden = residual.shape[1] // s
        dtype = self.runtime.compute_dtype
        u = ctx.buffer("hyper.u", (n, hidden), torch.float32)
        y = ctx.buffer("block.sublayer", (n, hidden), torch.float32)
        x1 = ctx.buffer("block.x", (n, hidden), dtype)
        (in1, mix1, out1), (w1, eps1) = self.coefficients[0], self.norms[0]
        owed = getattr(ctx, "owed", None)
        if owed is not None:
            # the layer ahead left its last write-back: it is done in the pass of this layer's first read
            ctx.owed = None
            ops.hyper_step(residual, s, y=owed[1], mix=owed[2], out_weights=owed[3], in_weights=in1, u=u, norm_weight=w1,
                           normed=x1, eps=eps1)
        else:
            ops.hyper_step(residual, s, in_weights=in1, u=u, norm_weight=w1, normed=x1, eps=eps1)
        self._sublayer(ctx, self.mixer, x1, y, kv=kv, state=state)
        if self.feed_forward is None:
            ctx.owed = (self, y, mix1, out1)
            return None
        (in2, mix2, out2), (w2, eps2) = self.coefficients[1], self.norms[1]
        x2 = ctx.buffer("block.x2", (n, hidden), dtype)
        ops.hyper_step(residual, s, y=y, mix=mix1, out_weights=out1, in_weights=in2, u=u, norm_weight=w2, normed=x2, eps=eps2)
        self._sublayer(ctx, self.feed_forward, x2, y)
        ctx.owed = (self, y, mix2, out2)
        return None

    def settle(self, ctx, residual) -> None:
        owed = getattr(ctx, "owed", None)
        if owed is not None and owed[0] is self:
            ctx.owed = None
            ops.hyper_step(residual, self.n_streams, y=owed[1], mix=owed[2], out_weights=owed[3])
