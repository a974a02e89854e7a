"""A mixture of gated feed-forward experts.

    z = W_router x  (32-bit),  s = softmax(z) over all experts
    the `top` experts with the largest s are chosen (the lower index wins a tie); weight_e = s_e * router_scale,
        not renormalised over the chosen
    expert_e(x) = W_down,e (silu(W_gate,e x) * (W_up,e x))
    f(x) = sum over the chosen e of weight_e expert_e(x)  [+ sigmoid(w_sg . x) * shared(x)]

`shared` (optional) is one more expert of a size of its own that every token uses, times a gate of one number per token.
The router's product, the softmax, the choice and the weights are 32-bit; the (token, choice) pairs are grouped by expert
on the device, each expert's rows go through its two products in tiles (bfloat16: the grouped product on the tensor
cores, csrc/gemm_tc.cu, over rows padded to whole tiles per expert; 32-bit, and sizes that TMA cannot address: the
product on the 32-bit pipes), and one kernel adds a token's weighted rows, in the order of its choices, into the
residual stream (csrc/moe.cu).  Nothing is decided on the host, so a step's launches
depend on its number of tokens alone, and a token's result does not depend on what else is in the batch.

Options (each absent by default):
  * `expert_form` "relu_squared": the experts (and the shared expert) are ungated, expert_e(x) = W_down,e relu(W_up,e x)^2,
    and have no gate matrix;
  * `identity` n: the router has n more outputs behind the experts'; an identity output that is chosen contributes
    weight * x itself (its pair belongs to no row of the products);
  * `correction`: a stored vector over the router's outputs that is added to the scores for the choice only (the weights
    use the scores without it);
  * `groups` {"count", "keep"}: the router's outputs form `count` equal groups of neighbours, a group's score is its
    largest choice score, and only outputs of the `keep` best groups can be chosen;
  * `renormalise`: weight_e = s_e / (sum of the chosen s + 1e-20) * router_scale.

Parameters: hidden, experts, top, intermediate, router_scale, shared ({"intermediate": n} or None), and optionally
`names`.  Checkpoint names behind the part's prefix: router, correction, e<i>.gate, e<i>.up, e<i>.down, shared.gate,
shared.up, shared.down, shared.sg."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import STORE, SWIGLU, linear, prepare_weight


@register_feed_forward("expert_mixture")
class ExpertMixture(FeedForward):
    graph_safe = True
    can_store = True
    NAMES = {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "shared": "shared.",
             "shared_gate": "shared.sg", "correction": "correction"}

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def _names(params, prefix):
        return {key: name for key, name in {**ExpertMixture.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        experts, top = int(params["experts"]), int(params["top"])
        if not 0 < experts <= ops.MOE_MAX_EXPERTS or not 0 < top <= min(experts + int(params.get("identity") or 0), ops.MOE_MAX_TOP):
            raise ValueError(f"expert mixture: 1..{ops.MOE_MAX_EXPERTS} experts, of which 1..{ops.MOE_MAX_TOP} (at most all) "
                             "are chosen")
        if int(params["intermediate"]) <= 0 or (params.get("shared") and int(params["shared"]["intermediate"]) <= 0):
            raise ValueError("expert mixture: the experts' sizes must be positive")
        if params.get("expert_form", "gated_silu") not in ("gated_silu", "relu_squared"):
            raise ValueError("expert mixture: expert_form is 'gated_silu' or 'relu_squared'")
        outputs = experts + int(params.get("identity") or 0)
        if int(params.get("identity") or 0) < 0 or outputs > ops.MOE_MAX_EXPERTS or top > outputs:
            raise ValueError(f"expert mixture: identity outputs are not negative, the router has at most {ops.MOE_MAX_EXPERTS} "
                             "outputs and no more are chosen than there are")
        groups = params.get("groups")
        if groups:
            count, keep = int(groups["count"]), int(groups["keep"])
            if count <= 0 or outputs % count or not 1 <= keep <= count or keep * (outputs // count) < top:
                raise ValueError("expert mixture: groups.count divides the router's outputs, 1 <= groups.keep <= count, and "
                                 "the kept groups hold at least `top` outputs")

    @staticmethod
    def tensor_specs(params, prefix):
        h, experts, ff = int(params["hidden"]), int(params["experts"]), int(params["intermediate"])
        n = ExpertMixture._names(params, prefix)
        gated = params.get("expert_form", "gated_silu") == "gated_silu"
        outputs = experts + int(params.get("identity") or 0)
        specs = []
        for e in range(experts):
            p = prefix + n["expert"].format(e)
            specs += ([TensorSpec(p + n["gate"], (ff, h))] if gated else []) + \
                [TensorSpec(p + n["up"], (ff, h)), TensorSpec(p + n["down"], (h, ff))]
        specs.append(TensorSpec(prefix + n["router"], (outputs, h)))
        if params.get("correction"):
            specs.append(TensorSpec(prefix + n["correction"], (outputs,)))
        if params.get("shared"):
            ffs, p = int(params["shared"]["intermediate"]), prefix + n["shared"]
            specs += ([TensorSpec(p + n["gate"], (ffs, h))] if gated else []) + \
                [TensorSpec(p + n["up"], (ffs, h)), TensorSpec(p + n["down"], (h, ffs)), TensorSpec(prefix + n["shared_gate"], (1, h))]
        return specs

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.experts, self.top = int(params["hidden"]), int(params["experts"]), int(params["top"])
        self.ff, self.router_scale = int(params["intermediate"]), float(params.get("router_scale", 1.0))
        self.gated = params.get("expert_form", "gated_silu") == "gated_silu"
        self.identity = int(params.get("identity") or 0)
        self.renormalise = bool(params.get("renormalise"))
        groups = params.get("groups")
        self.groups, self.keep = (int(groups["count"]), int(groups["keep"])) if groups else (0, 0)
        n = self._names(params, prefix)
        expert = lambda e, key: tensors[prefix + n["expert"].format(e) + n[key]]
        first = (lambda e: torch.cat([expert(e, "gate"), expert(e, "up")], dim=0)) if self.gated else (lambda e: expert(e, "up"))
        self.w_gate_up = prepare_weight(torch.stack([first(e) for e in range(self.experts)]), runtime)  # [E, 2 ff or ff, hidden]
        self.w_down = prepare_weight(torch.stack([expert(e, "down") for e in range(self.experts)]), runtime)   # [E, hidden, ff]
        router = [tensors[prefix + n["router"]]]
        self.shared = bool(params.get("shared"))
        if self.shared:
            self.ffs, p = int(params["shared"]["intermediate"]), prefix + n["shared"]
            router.append(tensors[prefix + n["shared_gate"]].view(1, self.hidden))        # the gate's row rides on the router's product
            first = torch.cat([tensors[p + n["gate"]], tensors[p + n["up"]]], dim=0) if self.gated else tensors[p + n["up"]]
            self.w_shared_gate_up = prepare_weight(first, runtime)
            self.w_shared_down = prepare_weight(tensors[p + n["down"]], runtime)
        self.router = torch.cat(router, dim=0).to(torch.float32).contiguous()
        self.correction = tensors[prefix + n["correction"]].to(torch.float32).contiguous() if params.get("correction") else None
        self.grouped = None          # whether the tensor-core product takes the experts' matrices: known at the first step

    def forward(self, ctx, x, residual, scale, store=False):
        rt, n = self.runtime, x.shape[0]
        top, experts, dtype = self.top, self.experts, rt.compute_dtype
        pairs = n * top
        scratch = ctx.runtime.scratch
        ids = scratch("moe.ids", pairs, torch.int32).view(n, top)
        weights = scratch("moe.weights", pairs, torch.float32).view(n, top)
        shared_gate = scratch("moe.shared_gate", n, torch.float32) if self.shared else None
        ops.moe_route(x, self.router, top, self.router_scale, ids, weights, shared_gate, correction=self.correction,
                      groups=self.groups, keep=self.keep, renormalise=self.renormalise)
        if self.grouped is None:
            self.grouped = ops.moe_grouped_accepts(x, self.w_gate_up, self.w_down)
        if self.grouped:
            # the tensor cores: every expert's rows begin at a multiple of the tile, the rows' inputs are laid side by side
            tile_rows = ops.moe_grouped_tile_rows(pairs, experts)
            max_tiles = ops.moe_max_tiles(pairs, experts, tile_rows)
            rows = max_tiles * tile_rows
        else:
            tile_rows, max_tiles, rows = 0, ops.moe_max_tiles(pairs, experts), pairs
        lists = scratch("moe.lists", experts + 2 + rows + pairs + 3 * max_tiles, torch.int32)
        offsets, n_tiles = lists[:experts + 1], lists[experts + 1:experts + 2]
        order, inverse = lists[experts + 2:experts + 2 + rows], lists[experts + 2 + rows:experts + 2 + rows + pairs]
        tiles = lists[experts + 2 + rows + pairs:]
        # (pairs whose output names no expert, the identity outputs, get no row: `inverse` is negative there)
        ops.moe_plan(ids.view(-1), experts, offsets, order, inverse, tiles, n_tiles, tile_rows, pad=self.grouped)
        act = scratch("moe.act", rows * self.ff, dtype).view(rows, self.ff)
        y = scratch("moe.y", rows * self.hidden, torch.float32).view(rows, self.hidden)
        if self.grouped:
            sorted_x = scratch("moe.x", rows * self.hidden, dtype).view(rows, self.hidden)
            ops.moe_gather(x, order, top, sorted_x)
            if self.gated:
                ops.gemm_tc_grouped(SWIGLU, sorted_x, self.w_gate_up, act, tile_rows, tiles, n_tiles, max_tiles, pairs,
                                    error_flag=ctx.error_flag, label="gate_up")
            else:
                ops.gemm_tc_grouped(STORE, sorted_x, self.w_gate_up, act, tile_rows, tiles, n_tiles, max_tiles, pairs,
                                    error_flag=ctx.error_flag, label="up", act=ops.ACT_RELU_SQUARED)
            ops.gemm_tc_grouped(STORE, act, self.w_down, y, tile_rows, tiles, n_tiles, max_tiles, pairs,
                                error_flag=ctx.error_flag, label="down")
        else:
            ops.moe_gemm(1 if self.gated else 2, x, order, top, self.w_gate_up, act, tiles, n_tiles, max_tiles,
                         label="gate_up" if self.gated else "up")
            ops.moe_gemm(0, act, None, top, self.w_down, y, tiles, n_tiles, max_tiles, label="down")
        shared_y = None
        if self.shared:
            shared_act = ctx.buffer("moe.shared_act", (n, self.ffs), dtype)
            if self.gated:
                linear(rt, SWIGLU, x, self.w_shared_gate_up, shared_act, error_flag=ctx.error_flag, name="shared_gate_up")
            else:
                shared_up = ctx.buffer("moe.shared_up", (n, self.ffs), torch.float32)
                if not linear(rt, STORE, x, self.w_shared_gate_up, shared_act, error_flag=ctx.error_flag, name="shared_up",
                              activation=ops.ACT_RELU_SQUARED, unactivated=shared_up):
                    ops.activation_rows(shared_up, shared_act, ops.ACT_RELU_SQUARED)
            shared_y = ctx.buffer("moe.shared_y", (n, self.hidden), torch.float32)
            linear(rt, STORE, shared_act, self.w_shared_down, shared_y, error_flag=ctx.error_flag, name="shared_down")
        ops.moe_combine(residual, y, inverse, weights, shared_y, shared_gate, top, scale, store,
                        x=x if self.identity else None)
