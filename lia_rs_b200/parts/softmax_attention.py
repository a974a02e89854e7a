"""Two softmax attentions over the paged cache whose queries, keys and values are more than one product's output.

`sink_attention`: grouped-query attention, q = Wq x + bq, k = Wk x + bk, v = Wv x + bv (biases optional), with
  * an RMS norm of every q head and every k head over the head's elements, with one weight of the head's size for all
    q heads and one for all k heads (optional; `qk_norm` "whole": one RMS norm over all of q's elements at once and one
    over all of k's, with weights of those sizes), ahead of the rotation;
  * rotate-half encoding over the first `rot.dims` elements of a head, frequencies plain or scaled by wavelength bands
    (`rotary.band_scaled_frequencies`);
  * values of a head size of their own;
  * value mixing (optional): the first such layer of a model leaves its values of the step's tokens in a step buffer
    (`value_mix` "source"), later ones ("mixed") use v <- (1 - lambda) v + lambda v_first, lambda a stored scalar; the
    mixed values are what the pages hold;
  * a sink (optional): one is added to the softmax's denominator, p_j = exp(s_j) / (1 + sum exp(s_j)), the weight of
    a key of score 0 that has no value;
  * a cap on the scores (optional, `softcap`): s <- cap * tanh(s / cap) ahead of the softmax;
  * all keys j <= i, or the last `window` of them;
  * an output projection whose bias (optional; `biases` "qkv": the three input projections have biases and the output
    projection none) is the mixer's `output_bias`.

`latent_attention`: queries and keys go through latents.  c_q = rms(W_dq x) w; q = W_uq c_q, per head `head_dim`
unrotated and `rot_dim` rotated elements.  W_dkv x gives `kv_rank` elements whose RMS norm (with a weight) is the latent
c, and `rot_dim` more that are one rotated key part for all heads.  Head h's key is [W_uk,h c | rotated part], its value
W_uv,h c.  The pages hold c and the rotated part only (the cache's "keys" are the latents, its "values" the rotated
parts), so attention runs in the latent's space: the unrotated query is taken through W_uk,h^T once per token,
q~_h = W_uk,h^T q_h, the score is scale (q~_h . c_j + q_rot,h . r_j), the weighted sum of the latents is taken through
W_uv,h afterwards, and the heads side by side through W_o.  A window as above; no sink.  Options: `q_rank` None: the
queries come straight from the input, q = W_q x; `rot_pairs`: the rotation pairs element 2i with 2i + 1 instead of i with
i + dims / 2; `gate` "sigmoid": the heads side by side are multiplied by sigmoid(W_g x) ahead of W_o ("sigmoid_head": W_g
has one row a head, and a head's output is multiplied by that one number); `shared_cache`: the
layer has no W_dkv and reads the latents and rotated parts that another layer of the same sizes and rotation put into the
pages (the model's schedule names that layer's cache), with W_uk, W_uv and queries of its own.

Scores, softmax, norms and angles are 32-bit in both.  Which kernel serves which rows: the kernel for every size and
element type (csrc/attention_generic.cu, `attention_general`); `sink_attention` in bfloat16 with equal key and value
head sizes that the tensor-core kernels take uses those (`PagedAttention` with its `sink`)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import DeferredNorm, KVCacheRequest, Mixer, NORMS, lookup, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight
from .paged_attention import PagedAttention
from .rotary import band_scaled_frequencies


def _frequencies(rot, device):
    """(rot_dims, 32-bit frequencies on the device) of a `rot` record {base, dims, scaling} (None: no encoding)."""
    if not rot or not int(rot["dims"]):
        return 0, None
    dims = int(rot["dims"])
    freq = band_scaled_frequencies(float(rot["base"]), dims, rot.get("scaling"))
    return dims, freq.to(torch.float32).to(device)


def _check_rot(rot, limit, what):
    if rot is None:
        return
    dims = int(rot["dims"])
    if dims < 0 or dims % 2 or dims > limit or (dims and not float(rot["base"]) > 0):
        raise ValueError(f"{what}: rot.dims must be even and at most {limit}, rot.base positive")
    scaling = rot.get("scaling")
    if scaling and not (float(scaling["high"]) != float(scaling["low"]) and float(scaling["factor"]) > 0
                        and float(scaling["original"]) > 0 and float(scaling["low"]) > 0 and float(scaling["high"]) > 0):
        raise ValueError(f"{what}: rot.scaling needs positive factor, original, low and high, low and high apart")


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
             "q_norm": "q.norm", "k_norm": "k.norm", "mix": "vmix"}

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**SinkAttention.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        nq, nkv, d, dv = (int(params[k]) for k in ("heads", "kv_heads", "head_dim", "v_head_dim"))
        if nq <= 0 or nkv <= 0 or nq % nkv:
            raise ValueError("attention: heads must be a positive multiple of kv_heads")
        if not 0 < d <= 1024 or not 0 < dv <= 512:
            raise ValueError("attention: head_dim must be within 1..1024 and v_head_dim within 1..512 (what the kernel takes)")
        _check_rot(params.get("rot"), d, "attention")
        if params.get("value_mix") not in (None, "source", "mixed"):
            raise ValueError("attention: value_mix is None, 'source' or 'mixed'")
        if params.get("window") is not None and int(params["window"]) <= 0:
            raise ValueError("attention: window must be positive or None")
        if params.get("softcap") is not None and not float(params["softcap"]) > 0:
            raise ValueError("attention: softcap must be positive or None")
        if params.get("biases") not in (None, False, True, "qkv") or params.get("qk_norm") not in (None, False, True, "whole"):
            raise ValueError("attention: biases is absent, True or 'qkv'; qk_norm is absent, True or 'whole'")
        if params.get("softcap") is not None and params.get("sink"):
            raise ValueError("attention: a sink and a cap on the scores together are not built")

    @staticmethod
    def tensor_specs(params, prefix):
        h, nq, nkv, d, dv = (int(params[k]) for k in ("hidden", "heads", "kv_heads", "head_dim", "v_head_dim"))
        n = SinkAttention._names(params, prefix)
        specs = [TensorSpec(n["q"], (nq * d, h)), TensorSpec(n["k"], (nkv * d, h)), TensorSpec(n["v"], (nkv * dv, h)),
                 TensorSpec(n["o"], (h, nq * dv))]
        if params.get("biases"):
            specs += [TensorSpec(n["q_bias"], (nq * d,)), TensorSpec(n["k_bias"], (nkv * d,)),
                      TensorSpec(n["v_bias"], (nkv * dv,))]
            if params["biases"] != "qkv":
                specs.append(TensorSpec(n["o_bias"], (h,)))
        if params.get("qk_norm") == "whole":
            specs += [TensorSpec(n["q_norm"], (nq * d,), kind="norm"), TensorSpec(n["k_norm"], (nkv * d,), kind="norm")]
        elif params.get("qk_norm"):
            specs += [TensorSpec(n["q_norm"], (d,), kind="norm"), TensorSpec(n["k_norm"], (d,), kind="norm")]
        if params.get("value_mix"):
            specs.append(TensorSpec(n["mix"], ()))          # the first such layer stores one too and does not use it
        return specs

    @staticmethod
    def cache_request(params):
        return KVCacheRequest(int(params["kv_heads"]), int(params["head_dim"]), params.get("window"),
                              v_head_dim=int(params["v_head_dim"]))

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden = int(params["hidden"])
        self.nq, self.nkv = int(params["heads"]), int(params["kv_heads"])
        self.d, self.dv = int(params["head_dim"]), int(params["v_head_dim"])
        self.scale, self.window, self.sink = float(params["scale"]), params.get("window"), bool(params.get("sink"))
        self.eps = float(params.get("norm_eps", 1e-6))
        n = self._names(params, prefix)
        device = runtime.device
        used = (self.nq + self.nkv) * self.d + self.nkv * self.dv
        self.width = (used + 7) // 8 * 8
        parts = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        if self.width > used:
            parts.append(torch.zeros((self.width - used, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = prepare_weight(torch.cat(parts, dim=0), runtime)
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.bias_in, self.output_bias = None, None
        if params.get("biases"):
            self.bias_in = f32(torch.cat([tensors[n["q_bias"]], tensors[n["k_bias"]], tensors[n["v_bias"]]]))
            self.output_bias = f32(tensors[n["o_bias"]]) if params["biases"] != "qkv" else None
        self.norm_whole = params.get("qk_norm") == "whole"
        self.softcap = None if params.get("softcap") is None else float(params["softcap"])
        self.q_norm = f32(tensors[n["q_norm"]]) if params.get("qk_norm") else None
        self.k_norm = f32(tensors[n["k_norm"]]) if params.get("qk_norm") else None
        self.rot_dims, self.freq = _frequencies(params.get("rot"), device)
        self.mix_mode = {None: 0, "source": 1, "mixed": 2}[params.get("value_mix")]
        self.mix_lambda = float(tensors[n["mix"]].to(torch.float32)) if self.mix_mode == 2 else 0.0
        # bfloat16 with keys and values of one head size that the tensor-core kernels take: those kernels; else the
        # kernel for every size
        self.paged = None
        if runtime.compute_dtype == torch.bfloat16 and self.d == self.dv and self.d in ops.DECODE_HEAD_DIMS and \
                self.nq // self.nkv <= 64:
            self.paged = PagedAttention(runtime.compute_dtype, self.nq, self.nkv, self.d, self.window, self.scale, sink=self.sink,
                                        softcap=self.softcap)

    def graph_key(self, ctx) -> tuple:
        return self.paged.graph_key(ctx) if self.paged is not None else ()

    def forward(self, ctx, x, residual, scale, kv=None, state=None, store=False):
        rt, n = self.runtime, x.shape[0]
        nq, nkv, d, dv = self.nq, self.nkv, self.d, self.dv
        flag = ctx.error_flag
        projected = ctx.buffer("sinkattn.in", (n, self.width), torch.float32)
        linear(rt, STORE, x, self.w_in, projected, error_flag=flag, name="qkv")
        q = ctx.buffer("sinkattn.q", (n, nq * d), rt.compute_dtype)
        v_first = ctx.buffer("sinkattn.v_first", (n, nkv * dv), torch.float32) if self.mix_mode else None
        ops.qkv_prepare(projected, self.bias_in, self.q_norm, self.k_norm, self.eps, self.freq, self.rot_dims,
                        self.mix_mode, self.mix_lambda, v_first, ctx.positions, ctx.slots, kv.block_table, q, kv.k_pages,
                        kv.v_pages, nq, nkv, d, dv, write_kv=kv.writes, error_flag=flag, norm_whole=self.norm_whole)
        o = ctx.buffer("sinkattn.o", (n, nq * dv), rt.compute_dtype)
        if self.paged is not None:
            self.paged.forward(ctx, q, kv, o)
        else:
            ops.attention_general(q, (nq * d, d), None, None, kv.k_pages, None, kv.v_pages, dv, dv, ctx.positions, ctx.slots,
                                  kv.block_table, o, (nq * dv, dv), n, nq, nkv, self.window, self.scale, sink=self.sink,
                                  error_flag=flag, softcap=self.softcap)
        linear(rt, STORE if store else ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    NAMES = {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "q": "q", "kv_down": "dkv", "kv_norm": "dkv.norm",
             "k_up": "uk", "v_up": "uv", "gate": "g", "o": "o"}

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**LatentAttention.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        for key in ("heads", "head_dim", "rot_dim", "v_head_dim", "kv_rank"):
            if int(params[key]) <= 0:
                raise ValueError(f"latent attention: {key} must be positive")
        if params.get("q_rank") is not None and int(params["q_rank"]) <= 0:
            raise ValueError("latent attention: q_rank must be positive, or None for queries straight from the input")
        if int(params["kv_rank"]) + int(params["rot_dim"]) > 1024 or int(params["kv_rank"]) > 512:
            raise ValueError("latent attention: kv_rank at most 512 and kv_rank + rot_dim at most 1024 (what the kernel takes)")
        _check_rot(params.get("rot"), int(params["rot_dim"]), "latent attention")
        if params.get("window") is not None and int(params["window"]) <= 0:
            raise ValueError("latent attention: window must be positive or None")
        if params.get("gate") not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError("latent attention: gate is None, 'sigmoid' or 'sigmoid_head'")

    @staticmethod
    def tensor_specs(params, prefix):
        h, H, d, dr, dv, rank = (int(params[k]) for k in ("hidden", "heads", "head_dim", "rot_dim", "v_head_dim", "kv_rank"))
        n = LatentAttention._names(params, prefix)
        if params.get("q_rank") is None:
            specs = [TensorSpec(n["q"], (H * (d + dr), h))]
        else:
            q_rank = int(params["q_rank"])
            specs = [TensorSpec(n["q_down"], (q_rank, h)), TensorSpec(n["q_norm"], (q_rank,), kind="norm"),
                     TensorSpec(n["q_up"], (H * (d + dr), q_rank))]
        if not params.get("shared_cache"):
            specs += [TensorSpec(n["kv_down"], (rank + dr, h)), TensorSpec(n["kv_norm"], (rank,), kind="norm")]
        specs += [TensorSpec(n["k_up"], (H * d, rank)), TensorSpec(n["v_up"], (H * dv, rank))]
        if params.get("gate"):
            specs.append(TensorSpec(n["gate"], (H if params["gate"] == "sigmoid_head" else H * dv, h)))
        return specs + [TensorSpec(n["o"], (h, H * dv))]

    @staticmethod
    def cache_request(params):
        # the pages' "keys" are the latents, their "values" the shared rotated key parts: one record a token for all heads
        return KVCacheRequest(1, int(params["kv_rank"]), params.get("window"), v_head_dim=int(params["rot_dim"]))

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.heads = int(params["hidden"]), int(params["heads"])
        self.d, self.dr, self.dv = int(params["head_dim"]), int(params["rot_dim"]), int(params["v_head_dim"])
        self.rank = int(params["kv_rank"])
        self.q_rank = None if params.get("q_rank") is None else int(params["q_rank"])
        self.scale, self.window = float(params["scale"]), params.get("window")
        self.eps = float(params.get("norm_eps", 1e-6))
        self.pairs, self.gated, self.own_cache = bool(params.get("rot_pairs")), bool(params.get("gate")), not params.get("shared_cache")
        self.gate_span = int(params["v_head_dim"]) if params.get("gate") == "sigmoid_head" else 1
        n = self._names(params, prefix)
        H, d, dv, rank = self.heads, self.d, self.dv, self.rank
        # One product for everything that is read from the input beside a query latent: [W_q (queries straight from the
        # input) | W_dkv (a cache of the layer's own) | W_g (a gate)], padded with zero rows to a multiple of 8 columns.
        blocks, at, self.columns = [], 0, {}
        for key, present, rows in (("q", self.q_rank is None, H * (d + self.dr)), ("kv_down", self.own_cache, rank + self.dr),
                                   ("gate", self.gated, H * dv // self.gate_span)):
            if present:
                blocks.append(tensors[n[key]])
                self.columns[key] = (at, at + rows)
                at += rows
        self.in_width = (at + 7) // 8 * 8
        if self.in_width > at:
            blocks.append(torch.zeros((self.in_width - at, self.hidden), dtype=blocks[0].dtype, device=blocks[0].device))
        self.w_in = prepare_weight(torch.cat(blocks, dim=0), runtime) if at else None
        if self.q_rank is not None:
            self.w_q_down = prepare_weight(tensors[n["q_down"]], runtime)
            self.w_q_up = prepare_weight(tensors[n["q_up"]], runtime)
            norm_params = {"hidden": self.q_rank, "eps": self.eps, "tensor": ""}
            self.q_norm = lookup(NORMS, "rmsnorm", "norm")(norm_params, {n["q_norm"]: tensors[n["q_norm"]]}, n["q_norm"], runtime)
        # head h's share of the key expansion, transposed: the product that takes a query into the latent's space
        self.w_k_up_t = prepare_weight(tensors[n["k_up"]].view(H, d, rank).transpose(1, 2), runtime)       # [H, rank, d]
        self.w_v_up = prepare_weight(tensors[n["v_up"]].view(H, dv, rank), runtime)                         # [H, dv, rank]
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        self.kv_norm = tensors[n["kv_norm"]].to(torch.float32).contiguous() if self.own_cache else None
        self.rot_dims, self.freq = _frequencies(params.get("rot"), runtime.device)
        self.tensor_cores = runtime.compute_dtype == torch.bfloat16 and ops.latent_attention_accepts(self.rank, self.dr)

    def _splits(self, ctx, n: int) -> int:
        """Into how many ranges the tensor-core kernel cuts each token's keys: as many as give every SM two CTAs, none
        shorter than four tiles of 32 keys at the step's context bucket and window, at most 16.  It depends on the number
        of rows and the context bucket alone, as a captured step needs."""
        longest = min(ctx.context_bucket, self.window or ctx.context_bucket)
        ctas = max(1, n * ((self.heads + 15) // 16))
        return max(1, min(2 * ctx.runtime.sm_count // ctas, 16, longest // 128))

    def _work(self, ctx):
        """(cache bytes the single tokens read, flops of the prompt portions), for the profile only."""
        if ops._profiler is None:
            return 0, 0
        seen = lambda p: min(p + 1, self.window or p + 1)
        keys = sum(seen(start) for _, start, count, _ in ctx.segments if count == 1)
        pairs = sum(seen(start + i) for _, start, count, _ in ctx.segments if count > 1 for i in range(count))
        return keys * (self.rank + self.dr) * 2, 2 * self.heads * (2 * self.rank + self.dr) * pairs

    TENSOR_CORES_FROM = 1             # tokens from which the heads' products go to the tensor cores (bfloat16)

    def _head_products(self, ctx, a, w, out, name):
        """out[h] = a[h] @ w[h]^T for every head (3-D tensors, a head a plane), all heads in one launch: in
        bfloat16 on the tensor cores (csrc/gemm_mma_batched.cu) where that kernel takes the sizes (8 tokens of 16 heads:
        5 us against 29 on the 32-bit pipes), else, and on the 32-bit path, on the 32-bit pipes."""
        if a.dtype == torch.bfloat16 and a.shape[1] >= self.TENSOR_CORES_FROM and ops.gemm_mma_batched_accepts(a, w, out):
            ops.gemm_mma_batched(a, w, out, label=name)
        else:
            ops.gemm_simt_batched(STORE, a, w, out, label=name)

    def forward(self, ctx, x, residual, scale, kv=None, state=None, store=False):
        rt, n = self.runtime, x.shape[0]
        H, d, dr, dv, rank = self.heads, self.d, self.dr, self.dv, self.rank
        flag, dtype = ctx.error_flag, rt.compute_dtype
        shared = gate = None
        if self.w_in is not None:
            rows = ctx.buffer("latent.in", (n, self.in_width), torch.float32)
            linear(rt, STORE, x, self.w_in, rows, error_flag=flag, name="latent_in")
            part = lambda key: rows[:, self.columns[key][0]:self.columns[key][1]] if key in self.columns else None
            shared, gate = part("kv_down"), part("gate")
        if self.q_rank is None:
            q_rows = part("q")
        else:
            q_latent = ctx.buffer("latent.cq", (n, self.q_rank), torch.float32)
            linear(rt, STORE, x, self.w_q_down, q_latent, error_flag=flag, name="q_down")
            q_rows = ctx.buffer("latent.q", (n, H * (d + dr)), torch.float32)
            linear(rt, STORE, DeferredNorm(ctx, self.q_norm, q_latent, buffer_name="latent.cq_normed"), self.w_q_up, q_rows,
                   error_flag=flag, name="q_up")
        scratch = ctx.runtime.scratch
        q_plain = scratch("latent.q_plain", H * n * d, dtype).view(H, n, d)
        q_rotated = ctx.buffer("latent.q_rot", (n, H * dr), dtype)
        ops.latent_prepare(q_rows, shared, self.kv_norm, self.eps, self.freq, self.rot_dims, ctx.positions, ctx.slots,
                           kv.block_table, q_plain, q_rotated, kv.k_pages, kv.v_pages, H, d, dr, rank,
                           write_kv=kv.writes and self.own_cache, error_flag=flag, pairs=self.pairs)
        q_absorbed = scratch("latent.q_absorbed", H * n * rank, dtype).view(H, n, rank)
        self._head_products(ctx, q_plain, self.w_k_up_t, q_absorbed, "k_up")
        mixed = scratch("latent.mixed", H * n * rank, dtype).view(H, n, rank)
        if self.tensor_cores:
            splits = self._splits(ctx, n)
            partial = scratch("latent.partial", splits * H * n * (rank + 2), torch.float32) if splits > 1 else None
            work_bytes, work_flops = self._work(ctx)
            ops.latent_attention(q_absorbed, q_rotated, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table,
                                 mixed, H, self.window, self.scale, splits=splits, partial=partial, error_flag=flag,
                                 work_bytes=work_bytes, work_flops=work_flops)
        else:
            ops.attention_general(q_absorbed, (rank, n * rank), q_rotated, (H * dr, dr), kv.k_pages, kv.v_pages, kv.k_pages,
                                  rank, rank, ctx.positions, ctx.slots, kv.block_table, mixed, (rank, n * rank), n, H, 1,
                                  self.window, self.scale, sink=False, error_flag=flag)
        o = ctx.buffer("latent.o", (n, H * dv), dtype)
        self._head_products(ctx, mixed, self.w_v_up, o.view(n, H, dv).transpose(0, 1), "v_up")
        if gate is not None:
            ops.gate_rows(o, gate, ops.GATE_SIGMOID, span=self.gate_span)
        linear(rt, STORE if store else ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
