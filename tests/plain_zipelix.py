"""A plain, slow implementation of the Zipelix decoder in dense 64-bit torch operations over whole sequences: one
function per mechanism, each written from the mechanism's equations (stated in its docstring) and sharing no code
with the package.

The design: x = embed[token], kept as `streams` copies x_1..x_s.  Every layer has a mixer and, optionally, a
feed-forward; sublayer q reads u = sum_s in_q[s] x_s through an RMS norm and the streams become
x_t <- sum_s mix_q[s, t] x_s + out_q[t] y.  The mixer is attention through a latent (`latent_attention`, optionally on
the latents that an earlier layer cached) or a decayed linear recurrence (`retention`); the feed-forward is a gated
dense one or a mixture of such experts.  logits = cap tanh(embed N(sum_s x_s) / cap)."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x, w, eps):
    """rms(x) * w."""
    return rms(x, eps) * w.to(F64)


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(base, dims):
    """f_i = base^(-2i/dims), i < dims/2."""
    return torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def rotate_interleaved(x, positions, base, dims):
    """x [T, ..., d]: for i < dims/2 the pair (u, v) = (x[2i], x[2i+1]) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i; elements from dims on pass unchanged."""
    out = x.clone()
    f = frequencies(base, dims)
    angle = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(x, positions, base, dims):
    """As above with the pair (x[i], x[i + dims/2])."""
    out = x.clone()
    half = dims // 2
    f = frequencies(base, dims)
    angle = positions.to(F64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_cache(h, positions, w_dkv, w_norm, m, eps):
    """What a latent-attention layer caches for its tokens: c = norm(first kv_rank rows of W_dkv h), and the last
    rot_dim rows, rotated in interleaved pairs: one key part for all heads."""
    rank, dr = m["kv_rank"], m["rot_dim"]
    both = h @ w_dkv.to(F64).T
    c = norm(both[:, :rank], w_norm, eps)
    shared = both[:, rank:rank + dr]
    if m.get("rot"):
        shared = rotate_interleaved(shared, positions, m["rot"]["base"], m["rot"]["dims"])
    return c, shared


def latent_attention(h, positions, w, m, cache):
    """h [T, width].  q = W_q h, per head [dim unrotated | rot_dim rotated]; head keys [W_uk c | shared part], values
    W_uv c; causal softmax of scale * (q . k); heads side by side, times sigmoid(W_g h), through W_o.
    `cache` = (c, shared) of all T positions."""
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    c, shared = cache
    q = (h @ w["q"].to(F64).T).view(T, H, d + dr)
    q_plain = q[:, :, :d]
    q_rot = q[:, :, d:].contiguous()
    if m.get("rot"):
        q_rot = rotate_interleaved(q_rot, positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w["uk"].to(F64).T).view(T, H, d)
    v = (c @ w["uv"].to(F64).T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, shared)) * float(m["scale"])
    visible = positions[:, None] >= positions[None, :]
    scores = scores.masked_fill(~visible[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].to(F64).T)
    return o @ w["o"].to(F64).T


def retention(h, positions, w, m, eps, fragile=None):
    """q = W_q h, k = W_k h [T, H, dim], v = W_v h [T, H, vdim]; q and k rotated in halves over the first rot.dims
    elements; k times dim^(-1/2); per head S_t = decay_h S_(t-1) + k_t v_t^T (S before the first token is zero),
    o_t = S_t^T q_t; each head's o over its root mean square; heads side by side times silu(W_g h), through W_o."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].to(F64).T).view(T, H, d)
    k = (h @ w["k"].to(F64).T).view(T, H, d)
    v = (h @ w["v"].to(F64).T).view(T, H, dv)
    if m.get("rot"):
        q = rotate_halves(q, positions, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_halves(k, positions, m["rot"]["base"], m["rot"]["dims"])
    k = k * d ** -0.5
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        decay = float(m["decay"][head])
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    if fragile is not None:
        fragile |= retention_is_fragile(q, k, v, out, m)
    out = rms(out, eps).reshape(T, H * dv)
    out = out * silu(h @ w["g"].to(F64).T)
    return out @ w["o"].to(F64).T


def retention_is_fragile(q, k, v, out, m):
    """Rows whose output direction rests on a cancellation, so that 16-bit rounding of q and k may turn it.  A head's
    o_t = sum_j decay^(t-j) (q_t . k_j) v_j is divided by its own size afterwards; rounding moves each q_t . k_j by about
    r |q_t| |k_j| / sqrt(dim), so o_t moves by about r n_t / sqrt(dim), n_t^2 = sum_j (decay^(t-j) |q_t| |k_j| |v_j|)^2.
    The first token is the plain case: its output is sign(q_0 . k_0) v_0 / |v_0|.  Fragile: n_t / sqrt(dim) > 8 |o_t|."""
    T, H, d = q.shape
    flags = torch.zeros(T, dtype=torch.bool)
    for head in range(H):
        decay = float(m["decay"][head])
        kv = (k[:, head].norm(dim=-1) * v[:, head].norm(dim=-1)) ** 2
        carried = torch.zeros((), dtype=F64)
        for t in range(T):
            carried = decay * decay * carried + kv[t]
            n = q[t, head].norm() * carried.sqrt()
            flags[t] |= bool(n / d ** 0.5 > 8.0 * out[t, head].norm())
    return flags


def gated_mlp(h, gate, up, down):
    """down (silu(gate h) * (up h))."""
    return (silu(h @ gate.to(F64).T) * (h @ up.to(F64).T)) @ down.to(F64).T


def expert_mixture(h, w, mlp, fragile=None):
    """s = softmax(W_router h) over all experts; the `top` largest are chosen; output = sum over the chosen of
    s_e * router.scale * expert_e(h) (not renormalised), plus sigmoid(W_sg h) * shared(h) if there is a shared expert."""
    router = mlp["router"]
    z = h @ w["router"].to(F64).T
    scores = torch.softmax(z, dim=-1)
    top = torch.topk(scores, int(router["top"]), dim=-1)
    if fragile is not None and int(router["top"]) < z.shape[1]:
        # a close call between the last expert chosen and the first one left out: rounding may turn it
        ranked = torch.sort(z, dim=-1, descending=True).values
        margin = ranked[:, int(router["top"]) - 1] - ranked[:, int(router["top"])]
        fragile |= margin < 0.04 * z.abs().max(dim=-1).values + 0.05
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for weight, e in zip(top.values[t], top.indices[t]):
            e = int(e)
            out[t] += weight * float(router["scale"]) * gated_mlp(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        shared = gated_mlp(h, w["shared.gate"], w["shared.up"], w["shared.down"])
        out = out + torch.sigmoid(h @ w["shared.sg"].to(F64).T) * shared
    return out


def hyper_step(streams, hc, prefix, sublayer, norm_weight, eps):
    """streams [s, T, width]: u = sum_s in[s] x_s; y = sublayer(norm(u)); x_t <- sum_s mix[s, t] x_s + out[t] y."""
    u = torch.einsum("s,stw->tw", hc[prefix + "in"].to(F64), streams)
    y = sublayer(norm(u, norm_weight, eps))
    return torch.einsum("sr,stw->rtw", hc[prefix + "mix"].to(F64), streams) + hc[prefix + "out"].to(F64)[:, None, None] * y[None]


def forward(config: dict, tensors: dict, tokens, layer_outputs=None, fragile=None):
    """Logits [T, vocab] (64-bit) of one sequence from position 0.  `layer_outputs`: a list that receives the sum of
    the streams after every layer.  `fragile`: a boolean tensor [T] in which the rows are marked whose result rests on
    a close call that 16-bit rounding may turn (a router's choice, a retention head's cancellation)."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    embed = tensors["embed"].to(F64)
    x = embed[torch.tensor(list(tokens), dtype=torch.long)]
    n_streams = int(config.get("streams", 0))
    streams = x[None].repeat(max(n_streams, 1), 1, 1)
    caches = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        w = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mix.")}

        def mixer(h, i=i, layer=layer, m=m, w=w):
            if layer["type"] == "latent_attention":
                if m.get("kv_from") is None:
                    caches[i] = latent_cache(h, positions, w["dkv"], w["dkv.norm"], m, eps)
                    cache = caches[i]
                else:
                    cache = caches[int(m["kv_from"])]
                return latent_attention(h, positions, w, m, cache)
            return retention(h, positions, w, m, eps, fragile)

        def feed_forward(h, layer=layer, p=p):
            mlp = layer["mlp"]
            w = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mlp.")}
            if mlp["kind"] == "dense":
                return gated_mlp(h, w["gate"], w["up"], w["down"])
            return expert_mixture(h, w, mlp, fragile)

        sublayers = [("1", mixer)] + ([("2", feed_forward)] if layer.get("mlp") else [])
        for q, sublayer in sublayers:
            if n_streams:
                hc = {k[len(p):]: v for k, v in tensors.items() if k.startswith(p + "hc" + q)}
                streams = hyper_step(streams, hc, f"hc{q}.", sublayer, tensors[p + "norm" + q], eps)
            else:
                streams = streams + sublayer(norm(streams[0], tensors[p + "norm" + q], eps))[None]
        if layer_outputs is not None:
            layer_outputs.append(streams.sum(dim=0).clone())
    x = norm(streams.sum(dim=0), tensors["final.norm"], eps)
    logits = x @ embed.T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


def greedy(config, weights, prompt, count):
    """`count` tokens after `prompt`, each the largest logit's id (the largest id among equals)."""
    tokens, out = list(prompt), []
    for _ in range(count):
        row = forward(config, weights, tokens)[-1]
        best = row.max()
        token = max(i for i in range(len(row)) if row[i] == best)
        out.append(token)
        tokens.append(token)
    return out
