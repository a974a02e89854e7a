"""Dense SwiGLU feed-forward: act = up * gate / (1 + exp(-gate)), f = act Wd^T, no biases
(src/inference/moe.rs:31-61, src/gpu/kernels/basic.rs:150-157).  Gate and up are one product
against [Wg; Wu] whose epilogue applies the activation (the reference's gated kernel does the
same with two matrices: src/gpu/kernels/llama_gated.rs:181-222); the down product adds into the
residual stream.  Parameters: hidden, intermediate, and optionally `names`: the checkpoint names of the gate, up
and down matrices behind the part's prefix, and `gate_activation`: "silu" (default) or "relu", act = up * relu(gate), in
the same epilogues."""
from __future__ import annotations

import torch

from ..weights import TensorSpec
from .base import FeedForward, register_feed_forward
from .linear import ACCUM, STORE, SWIGLU, linear, prepare_weight


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # rows in, rows out: only the number of tokens matters
    takes_deferred_norm = True
    can_store = True

    NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    @staticmethod
    def _names(params, prefix):
        names = {**SwiGLU.NAMES, **params.get("names", {})}
        return prefix + names["gate"], prefix + names["up"], prefix + names["down"]

    @staticmethod
    def tensor_specs(params, prefix):
        h, i = params["hidden"], params["intermediate"]
        gate, up, down = SwiGLU._names(params, prefix)
        return [TensorSpec(gate, (i, h)), TensorSpec(up, (i, h)), TensorSpec(down, (h, i))]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        gate, up, down = self._names(params, prefix)
        self.w_gate_up = prepare_weight(torch.cat([tensors[gate], tensors[up]], dim=0), runtime)
        self.w_down = prepare_weight(tensors[down], runtime)
        self.relu = params.get("gate_activation", "silu") == "relu"

    @staticmethod
    def check_params(params):
        if params.get("gate_activation", "silu") not in ("silu", "relu"):
            raise ValueError("gated feed-forward: gate_activation is 'silu' or 'relu'")

    def forward(self, ctx, x, residual, scale, store=False):
        rt, n = self.runtime, x.shape[0]
        act = ctx.buffer("ffn.act", (n, self.intermediate), rt.compute_dtype)
        linear(rt, SWIGLU, x, self.w_gate_up, act, error_flag=ctx.error_flag, name="gate_up",
               gate_activation=rt.ops.ACT_RELU if self.relu else 0)
        linear(rt, STORE if store else ACCUM, act, self.w_down, residual, scale, error_flag=ctx.error_flag, name="down")


@register_feed_forward("dense_act")
class DenseActivation(FeedForward):
    """Dense feed-forward without a gate: f = Wd act(Wu x), no biases.  `activation`: "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))), "silu", "relu_squared" (relu(z)^2), "relu" or "none".  The activation is taken of the up product's
    32-bit result and rounded once to the compute element type: in the product's epilogue where the kernel can (the
    few-token persistent product), else by a kernel of its own on the product's 32-bit rows; the down product adds into
    the residual stream.  Parameters: hidden, intermediate, activation, and optionally `names`: the checkpoint names of the up and
    down matrices behind the part's prefix."""
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    NAMES = {"up": "up_proj.weight", "down": "down_proj.weight"}
    ACTIVATIONS = {"none": 0, "gelu_tanh": 1, "silu": 2, "relu_squared": 3, "relu": 4}

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def _names(params, prefix):
        names = {**DenseActivation.NAMES, **params.get("names", {})}
        return prefix + names["up"], prefix + names["down"]

    @staticmethod
    def check_params(params):
        if params.get("activation", "gelu_tanh") not in DenseActivation.ACTIVATIONS:
            raise ValueError(f"dense feed-forward: activation {params.get('activation')!r} is not one of "
                             f"{sorted(DenseActivation.ACTIVATIONS)}")

    @staticmethod
    def tensor_specs(params, prefix):
        h, i = params["hidden"], params["intermediate"]
        up, down = DenseActivation._names(params, prefix)
        return [TensorSpec(up, (i, h)), TensorSpec(down, (h, i))]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.intermediate = int(params["hidden"]), int(params["intermediate"])
        self.activation = self.ACTIVATIONS[params.get("activation", "gelu_tanh")]
        up, down = self._names(params, prefix)
        self.w_up = prepare_weight(tensors[up], runtime)
        self.w_down = prepare_weight(tensors[down], runtime)

    def forward(self, ctx, x, residual, scale, store=False):
        rt, n = self.runtime, x.shape[0]
        up = ctx.buffer("ffn.up", (n, self.intermediate), torch.float32)
        act = ctx.buffer("ffn.act", (n, self.intermediate), rt.compute_dtype)
        if self.activation == 0:
            linear(rt, STORE, x, self.w_up, act, error_flag=ctx.error_flag, name="up")
        elif not linear(rt, STORE, x, self.w_up, act, error_flag=ctx.error_flag, name="up", activation=self.activation,
                        unactivated=up):
            rt.ops.activation_rows(up, act, self.activation)
        linear(rt, STORE if store else ACCUM, act, self.w_down, residual, scale, error_flag=ctx.error_flag, name="down")
