"""Gated linear attention: a linear recurrence per head whose decay is computed for every token and key channel.

    q = W_q x * head_dim^(-1/2), k = W_k x  (heads x head_dim),  v = W_v x, g = W_g x  (heads x v_head_dim)
    alpha = sigmoid(W_a2 (W_a1 x) + b_a2)^(1/tau)                 (heads x head_dim, a low-rank product; in (0, 1))
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   S before a request's first token = 0       (per head, [head_dim, v_head_dim])
    o_t = S_t^T q_t;   out = W_o concat_h( o_t,h / sqrt(mean(o_t,h^2) + eps) * w * silu(g_t,h) ),  w [v_head_dim] for all heads

What a request carries from token to token is one 32-bit state [heads, head_dim, v_head_dim] per slot.  The five input
products are one product against [W_q; W_k; W_v; W_g; W_a1] with 32-bit output; the second decay product, the decays
with their logarithms and powers, the state, the sums over it, the heads' norm and the gate are 32-bit
(csrc/gated_linear_attention.cu).  Single tokens update the state in place; prompt portions are cut into chunks that run
side by side and continue from the slot's state, so a portion cut anywhere gives what token-by-token steps give, up to
the order of the additions.

Parameters: hidden, heads, head_dim, v_head_dim, tau, norm_eps, decay_rank (the rank of the decay's product; None: it is
whatever the stored W_a1 has), and optionally `names`."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, StateRequest, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", "decay_down": "a1", "decay_up": "a2",
             "decay_bias": "a2.b"}

    def graph_key(self, ctx) -> tuple:
        return ()            # the chunks' number follows from the step's numbers of tokens, single tokens and portions

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**GatedLinearAttention.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        heads, d, dv = (int(params[k]) for k in ("heads", "head_dim", "v_head_dim"))
        if heads <= 0 or not 0 < d <= ops.GLA_MAX_HEAD or not 0 < dv <= ops.GLA_MAX_HEAD:
            raise ValueError(f"gated linear attention: heads positive, head_dim and v_head_dim within 1..{ops.GLA_MAX_HEAD} "
                             "(what the kernel takes)")
        if not float(params["tau"]) > 0:
            raise ValueError("gated linear attention: tau must be positive")
        if params.get("decay_rank") is not None and int(params["decay_rank"]) <= 0:
            raise ValueError("gated linear attention: decay_rank must be positive, or None for the stored tensor's")

    @staticmethod
    def tensor_specs(params, prefix):
        h, heads, d, dv = (int(params[k]) for k in ("hidden", "heads", "head_dim", "v_head_dim"))
        rank = None if params.get("decay_rank") is None else int(params["decay_rank"])
        n = GatedLinearAttention._names(params, prefix)
        return [TensorSpec(n["q"], (heads * d, h)), TensorSpec(n["k"], (heads * d, h)), TensorSpec(n["v"], (heads * dv, h)),
                TensorSpec(n["gate"], (heads * dv, h)), TensorSpec(n["o"], (h, heads * dv)),
                TensorSpec(n["norm"], (dv,), kind="norm"), TensorSpec(n["decay_down"], (rank, h)),
                TensorSpec(n["decay_up"], (heads * d, rank)), TensorSpec(n["decay_bias"], (heads * d,))]

    @staticmethod
    def state_request(params):
        return StateRequest((int(params["heads"]), int(params["head_dim"]), int(params["v_head_dim"])), torch.float32)

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.heads = int(params["hidden"]), int(params["heads"])
        self.d, self.dv = int(params["head_dim"]), int(params["v_head_dim"])
        self.eps, self.tau = float(params.get("norm_eps", 1e-6)), float(params["tau"])
        n = self._names(params, prefix)
        self.rank = int(tensors[n["decay_down"]].shape[0])
        if tuple(tensors[n["decay_up"]].shape) != (self.heads * self.d, self.rank):
            raise ValueError("gated linear attention: the two matrices of the decay's product disagree in their rank")
        used = 2 * self.heads * (self.d + self.dv) + self.rank
        self.width = (used + 7) // 8 * 8
        blocks = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]], tensors[n["decay_down"]]]
        if self.width > used:
            blocks.append(torch.zeros((self.width - used, self.hidden), dtype=blocks[0].dtype, device=blocks[0].device))
        self.w_in = prepare_weight(torch.cat(blocks, dim=0), runtime)
        self.w_decay_up = prepare_weight(tensors[n["decay_up"]], runtime)
        self.decay_bias = tensors[n["decay_bias"]].to(torch.float32).contiguous()
        self.norm_weight = tensors[n["norm"]].to(torch.float32).contiguous()
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        self.q_scale = float(self.d) ** -0.5

    def forward(self, ctx, x, residual, scale, kv=None, state=None, store=False):
        rt, n = self.runtime, x.shape[0]
        heads, d, dv = self.heads, self.d, self.dv
        flag = ctx.error_flag
        rows = ctx.buffer("gla.in", (n, self.width), torch.float32)
        linear(rt, STORE, x, self.w_in, rows, error_flag=flag, name="qkvga")
        portions = ctx.n_prefill_segments
        o = ctx.buffer("gla.o", (n, heads * dv), rt.compute_dtype)
        if not portions:
            # single tokens alone: the recurrence's kernel encodes each token's head itself
            ops.gla(rows, None, state, ctx.prefill_segments, 0, 0, ctx.decode_rows, ctx.slots, self.norm_weight, o, heads, d, dv,
                    self.eps, encode=(self.w_decay_up, self.decay_bias, self.q_scale, self.tau))
            linear(rt, STORE if store else ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
            return
        log_decay = ctx.buffer("gla.decay", (n, heads * d), torch.float32)
        ops.gla_encode(rows, self.w_decay_up, self.decay_bias, log_decay, ctx.slots, heads, d, dv, self.q_scale, self.tau)
        chunks = ops.retention_chunks(n - ctx.n_single, portions) if portions else 0
        scratch = ctx.runtime.scratch("gla.chunks", ops.gla_scratch_floats(chunks, heads, d, dv), torch.float32) if chunks else None
        ops.gla(rows, log_decay, state, ctx.prefill_segments, portions, chunks, ctx.decode_rows, ctx.slots, self.norm_weight, o,
                heads, d, dv, self.eps, scratch=scratch)
        linear(rt, STORE if store else ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
