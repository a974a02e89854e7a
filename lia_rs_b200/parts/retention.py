"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

    q = W_q x, k = W_k x  (heads x head_dim),  v = W_v x  (heads x v_head_dim),  g = W_g x  (heads x v_head_dim)
    q, k rotated in halves over the first rot.dims elements of a head (element i with i + dims / 2, angle
        position * base^(-2i / dims));  k <- k * head_dim^(-1/2) after the rotation
    S_t = decay_h S_(t-1) + k_t v_t^T,   S before a request's first token = 0       (per head, [head_dim, v_head_dim])
    o_t = S_t^T q_t;   out = W_o concat_h( o_t,h / sqrt(mean(o_t,h^2) + eps) * silu(g_t,h) )

What a request carries from token to token is one 32-bit state [heads, head_dim, v_head_dim] per slot.  The four input
products are one product against [W_q; W_k; W_v; W_g] with 32-bit output; rotation, scaling, decays, the state, the sums
over it, the heads' norms and the gate are 32-bit (csrc/retention.cu).  Single tokens update the state in place; prompt
portions are cut into chunks that run side by side and continue from the slot's state, so a portion cut anywhere gives
what token-by-token steps give, up to the order of the additions.

Parameters: hidden, heads, head_dim, v_head_dim, decay (one number per head, each in (0, 1]), rot {base, dims} or None,
norm_eps, and optionally `names`."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, StateRequest, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight
from .softmax_attention import _check_rot, _frequencies


@register_mixer("retention")
class Retention(Mixer):
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o"}

    def graph_key(self, ctx) -> tuple:
        return ()            # the chunks' number follows from the step's numbers of tokens, single tokens and portions

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**Retention.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        heads, d, dv = (int(params[k]) for k in ("heads", "head_dim", "v_head_dim"))
        if heads <= 0 or not 0 < d <= ops.RETENTION_MAX_HEAD or not 0 < dv <= ops.RETENTION_MAX_HEAD:
            raise ValueError(f"retention: heads positive, head_dim and v_head_dim within 1..{ops.RETENTION_MAX_HEAD} "
                             "(what the kernel takes)")
        decay = list(params["decay"])
        if len(decay) != heads or not all(0.0 < float(a) <= 1.0 for a in decay):
            raise ValueError("retention: decay lists one number in (0, 1] per head")
        rot = params.get("rot")
        if rot and rot.get("scaling"):
            raise ValueError("retention: plain rotary frequencies only")
        _check_rot(rot, d, "retention")

    @staticmethod
    def tensor_specs(params, prefix):
        h, heads, d, dv = (int(params[k]) for k in ("hidden", "heads", "head_dim", "v_head_dim"))
        n = Retention._names(params, prefix)
        return [TensorSpec(n["q"], (heads * d, h)), TensorSpec(n["k"], (heads * d, h)), TensorSpec(n["v"], (heads * dv, h)),
                TensorSpec(n["gate"], (heads * dv, h)), TensorSpec(n["o"], (h, heads * dv))]

    @staticmethod
    def state_request(params):
        return StateRequest((int(params["heads"]), int(params["head_dim"]), int(params["v_head_dim"])), torch.float32)

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.heads = int(params["hidden"]), int(params["heads"])
        self.d, self.dv = int(params["head_dim"]), int(params["v_head_dim"])
        self.eps = float(params.get("norm_eps", 1e-6))
        n = self._names(params, prefix)
        used = 2 * self.heads * (self.d + self.dv)
        self.width = (used + 7) // 8 * 8
        blocks = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        if self.width > used:
            blocks.append(torch.zeros((self.width - used, self.hidden), dtype=blocks[0].dtype, device=blocks[0].device))
        self.w_in = prepare_weight(torch.cat(blocks, dim=0), runtime)
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        self.decay = torch.tensor([float(a) for a in params["decay"]], dtype=torch.float32, device=runtime.device)
        self.rot_dims, self.freq = _frequencies(params.get("rot"), runtime.device)
        self.k_scale = float(self.d) ** -0.5

    def forward(self, ctx, x, residual, scale, kv=None, state=None, store=False):
        rt, n = self.runtime, x.shape[0]
        heads, d, dv = self.heads, self.d, self.dv
        flag = ctx.error_flag
        rows = ctx.buffer("retention.in", (n, self.width), torch.float32)
        linear(rt, STORE, x, self.w_in, rows, error_flag=flag, name="qkvg")
        ops.retention_encode(rows, self.freq, self.rot_dims, ctx.positions, ctx.slots, heads, d, self.k_scale)
        portions = ctx.n_prefill_segments
        chunks = ops.retention_chunks(n - ctx.n_single, portions) if portions else 0
        scratch = ctx.runtime.scratch("retention.chunks", ops.retention_scratch_floats(chunks, heads, d, dv),
                                      torch.float32) if chunks else None
        o = ctx.buffer("retention.o", (n, heads * dv), rt.compute_dtype)
        ops.retention(rows, self.decay, state, ctx.prefill_segments, portions, chunks, ctx.decode_rows, ctx.slots, o,
                      heads, d, dv, self.eps, scratch=scratch)
        linear(rt, STORE if store else ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
