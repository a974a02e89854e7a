"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, the weight used as stored
(src/gpu/kernels/normalization.rs:46-112).  Parameters: hidden, eps, and optionally `tensor`: what follows the
norm's prefix in the weight's checkpoint name (default "weight"), and `one_plus`: the stored weight w lies around zero and
the norm multiplies by 1 + w (the sum is taken once, at load, in 32-bit, and kept so)."""
from __future__ import annotations

import torch

from ..weights import TensorSpec
from .base import Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # rows in, rows out: only the number of tokens matters

    @staticmethod
    def tensor_specs(params, prefix):
        kind = "matrix" if params.get("one_plus") else "norm"          # random weights: around zero, or ones
        return [TensorSpec(prefix + params.get("tensor", "weight"), (params["hidden"],), kind=kind)]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden = int(params["hidden"])
        self.eps = float(params["eps"])
        self.weight = tensors[prefix + params.get("tensor", "weight")]     # bfloat16 or, if stored so, float32
        if params.get("one_plus"):
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def forward(self, ctx, x, out, rows_index=None, out_scale=1.0):
        self.runtime.ops.rmsnorm(x, self.weight, out, self.eps, out_scale, rows_index)

    def rms_record(self):
        return self.weight, self.eps


@register_norm("layernorm")
class LayerNorm(Norm):
    """Layer norm: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, mean and variance over the row in 32-bit
    (csrc/elementwise.cu).  Parameters: hidden, eps, and optionally `tensor` and `bias_tensor`: what follows the norm's
    prefix in the checkpoint names of weight and bias (defaults "weight" and "bias"); `bias_tensor` None: no bias.  It is
    not an RMS norm, so no product kernel applies it (`rms_record` answers None) and it always runs its own kernel."""
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def _names(params, prefix):
        bias = params.get("bias_tensor", "bias")
        return prefix + params.get("tensor", "weight"), None if bias is None else prefix + bias

    @staticmethod
    def tensor_specs(params, prefix):
        weight, bias = LayerNorm._names(params, prefix)
        specs = [TensorSpec(weight, (params["hidden"],), kind="norm")]
        if bias is not None:
            specs.append(TensorSpec(bias, (params["hidden"],)))
        return specs

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden, self.eps = int(params["hidden"]), float(params["eps"])
        weight, bias = self._names(params, prefix)
        self.weight = tensors[weight].to(torch.float32).contiguous()
        self.bias = None if bias is None else tensors[bias].to(torch.float32).contiguous()

    def forward(self, ctx, x, out, rows_index=None, out_scale=1.0):
        if out_scale != 1.0:
            raise ValueError("layer norm: no output scale")
        self.runtime.ops.layernorm(x, self.weight, self.bias, out, self.eps, rows_index)
