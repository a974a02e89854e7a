"""A plain, slow implementation of the Pilutar decoder in dense 64-bit torch operations over whole sequences: one
function per mechanism, each written from the mechanism's equations (stated in its docstring) and sharing no code
with the package.

The design: x = embed[token] * embedding.scale.  Every layer computes h = LN(x) once (a layer norm with weight and
bias) and adds mixer(h) + feed_forward(h) to x.  The mixer is attention through a latent with a window and one
sigmoid gate per head (`latent_attention`), or two mixers side by side (`parallel`): windowed grouped-query softmax
attention with biases, a norm over the whole q and k projections, rotation in halves and a tanh cap on the scores,
beside gated linear attention (a linear recurrence whose decay is computed per token and key channel).  The
feed-forward is a gated dense one with a ReLU gate, a mixture of ungated squared-ReLU experts (score correction,
groups, identity experts, a gated shared expert), or absent.  logits = head LN(x) * logit_scale."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b over the last axis."""
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * w.to(F64) + b.to(F64)


def frequencies(base, dims):
    """f_i = base^(-2i/dims), i < dims/2."""
    return torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def _angles(x, positions, base, dims):
    angle = positions.to(F64)[:, None] * frequencies(base, dims)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    return torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)


def rotate_interleaved(x, positions, base, dims):
    """x [T, ..., d]: for i < dims/2 the pair (u, v) = (x[2i], x[2i+1]) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i; elements from dims on pass unchanged."""
    out = x.clone()
    c, s = _angles(x, positions, base, dims)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(x, positions, base, dims):
    """As above with the pair (x[i], x[i + dims/2])."""
    out = x.clone()
    half = dims // 2
    c, s = _angles(x, positions, base, dims)
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def window_mask(positions, size):
    """[T, T] True where key j is visible to query i: 0 <= p_i - p_j < size (size None: every j <= i)."""
    delta = positions[:, None] - positions[None, :]
    visible = delta >= 0
    if size is not None:
        visible &= delta < int(size)
    return visible


def latent_attention(h, positions, w, m, eps):
    """q = W_q h, per head [dim unrotated | rot_dim rotated].  W_dkv h: the first kv_rank rows, RMS-normed with a
    weight, are the latent c; the last rot_dim are one key part for all heads.  The rotated parts of q and of the key
    turn in interleaved pairs.  Head keys [W_uk c | shared part], values W_uv c; softmax of scale * (q . k) over the
    window; head h's output times sigmoid(W_g h)_h; heads side by side through W_o."""
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    both = h @ w["dkv"].to(F64).T
    c = rms(both[:, :rank], eps) * w["dkv.norm"].to(F64)
    shared = both[:, rank:rank + dr]
    q = (h @ w["q"].to(F64).T).view(T, H, d + dr)
    q_plain, q_rot = q[:, :, :d], q[:, :, d:].contiguous()
    if m.get("rot"):
        shared = rotate_interleaved(shared, positions, m["rot"]["base"], m["rot"]["dims"])
        q_rot = rotate_interleaved(q_rot, positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w["uk"].to(F64).T).view(T, H, d)
    v = (c @ w["uv"].to(F64).T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, shared)) * float(m["scale"])
    scores = scores.masked_fill(~window_mask(positions, (m.get("mask") or {}).get("size"))[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v)
    o = o * torch.sigmoid(h @ w["g"].to(F64).T)[:, :, None]
    return o.reshape(T, H * dv) @ w["o"].to(F64).T


def capped_attention(h, positions, w, m, eps):
    """q = W_q h + b_q, k = W_k h + b_k, v = W_v h + b_v.  q and k are each RMS-normed over their whole row (all heads
    at once) with a weight of that size, then split into heads and rotated in halves over the first rot.dims elements.
    Query head a reads key/value head a // (H / G).  s = scale * (q . k); s <- cap * tanh(s / cap); softmax over the
    window; heads side by side through W_o."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = h @ w["q"].to(F64).T + w["q.b"].to(F64)
    k = h @ w["k"].to(F64).T + w["k.b"].to(F64)
    v = (h @ w["v"].to(F64).T + w["v.b"].to(F64)).view(T, G, dv)
    q = (rms(q, eps) * w["q.norm"].to(F64)).view(T, H, d)
    k = (rms(k, eps) * w["k.norm"].to(F64)).view(T, G, d)
    if m.get("rot"):
        q = rotate_halves(q, positions, m["rot"]["base"], m["rot"]["dims"])
        k = rotate_halves(k, positions, m["rot"]["base"], m["rot"]["dims"])
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * float(m["scale"])
    cap = m.get("softcap")
    if cap:
        scores = float(cap) * torch.tanh(scores / float(cap))
    scores = scores.masked_fill(~window_mask(positions, (m.get("mask") or {}).get("size"))[None], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv) @ w["o"].to(F64).T


def gated_linear_attention(h, w, m, eps, state=None):
    """q = W_q h * dim^(-1/2), k = W_k h [T, H, dim], v = W_v h [T, H, vdim].  Decay per token and key channel:
    alpha = sigmoid(W_a2 (W_a1 h) + b_a2)^(1/tau) [T, H, dim].  Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T
    (S before the first token is zero, or `state`), o_t = S_t^T q_t.  Each head's o over its root mean square times
    a weight of size vdim that the heads share; heads side by side times silu(W_g h), through W_o.
    Returns (output, the state after the last token [H, dim, vdim])."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w["q"].to(F64).T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].to(F64).T).view(T, H, d)
    v = (h @ w["v"].to(F64).T).view(T, H, dv)
    z = (h @ w["a1"].to(F64).T) @ w["a2"].to(F64).T + w["a2.b"].to(F64)
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / float(m["tau"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state.to(F64).clone()
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = (rms(out, eps) * w["norm"].to(F64)).reshape(T, H * dv)
    gate = h @ w["g"].to(F64).T
    return (out * gate * torch.sigmoid(gate)) @ w["o"].to(F64).T, S


def side_by_side(h, positions, w, m, eps):
    """left_scale * capped_attention(h) + right_scale * gated_linear_attention(h); both read the same h."""
    left = capped_attention(h, positions, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right, _ = gated_linear_attention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def relu_gated_mlp(h, gate, up, down):
    """down (relu(gate h) * (up h))."""
    return (torch.relu(h @ gate.to(F64).T) * (h @ up.to(F64).T)) @ down.to(F64).T


def squared_relu_mlp(h, up, down):
    """down relu(up h)^2."""
    return (torch.relu(h @ up.to(F64).T) ** 2) @ down.to(F64).T


def route(h, w, router, fragile=None):
    """z = W_router h over experts + identity outputs; s = softmax(z).  Choice scores c = s + correction.  The outputs
    form groups.count groups of neighbours; a group's score is its largest c; outside the groups.keep best groups c
    counts as minus infinity.  The `top` largest c are chosen; their weights are s over the chosen, divided by their sum
    (+ 1e-20).  Returns (indices [T, top], weights [T, top])."""
    z = h @ w["router"].to(F64).T
    s = torch.softmax(z, dim=-1)
    c = s + w["correction"].to(F64) if "correction" in w else s.clone()
    total, top = z.shape[1], int(router["top"])
    groups = router.get("groups")
    if groups and int(groups["count"]) > 1:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = c.view(-1, count, total // count).max(dim=-1).values
        kept = torch.topk(best, keep, dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        c = c.masked_fill(~allowed.repeat_interleave(total // count, dim=1), float("-inf"))
        if fragile is not None and keep < count:
            ranked = torch.sort(best, dim=-1, descending=True).values
            fragile |= (ranked[:, keep - 1] - ranked[:, keep]) < 1e-2
    chosen = torch.topk(c, top, dim=-1).indices
    if fragile is not None:
        ranked = torch.sort(c, dim=-1, descending=True).values
        if top < total:
            margin = ranked[:, top - 1] - ranked[:, top]
            fragile |= margin < 1e-2          # (an excluded output's -inf gives an infinite margin)
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20)


def expert_mixture(h, w, mlp, fragile=None):
    """sum over the chosen outputs e of weight_e * f_e(h): f_e is the squared-ReLU expert e for e < experts and the
    identity, f_e(h) = h, for the router.identity outputs behind them; plus sigmoid(W_sg h) * shared(h) where there is
    a shared expert (same form)."""
    router = mlp["router"]
    experts = int(router["experts"])
    chosen, weights = route(h, w, router, fragile)
    out = torch.zeros(h.shape[0], h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for weight, e in zip(weights[t], chosen[t]):
            e = int(e)
            if e >= experts:
                out[t] += weight * h[t]
            else:
                out[t] += weight * squared_relu_mlp(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w["shared.sg"].to(F64).T) * squared_relu_mlp(h, w["shared.up"], w["shared.down"])
    return out


def forward(config: dict, tensors: dict, tokens, layer_outputs=None, fragile=None):
    """Logits [T, vocab] (64-bit) of one sequence from position 0.  `layer_outputs`: a list that receives the residual
    stream after every layer.  `fragile`: a boolean tensor [T] in which the rows are marked whose result rests on a
    router's close call that 16-bit rounding may turn."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = tensors["embed"].to(F64)[torch.tensor(list(tokens), dtype=torch.long)] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, tensors[p + "norm1"], tensors[p + "norm1.b"], eps)
        w = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mix.")}
        if layer["type"] == "latent_attention":
            y = latent_attention(h, positions, w, layer["mixer"], eps)
        else:
            y = side_by_side(h, positions, w, layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp:
            w = {k[len(p) + 4:]: v for k, v in tensors.items() if k.startswith(p + "mlp.")}
            if mlp["kind"] == "dense":
                y = y + relu_gated_mlp(h, w["gate"], w["up"], w["down"])
            else:
                y = y + expert_mixture(h, w, mlp, fragile)
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = layer_norm(x, tensors["final.norm"], tensors["final.norm.b"], eps)
    return (x @ tensors["head"].to(F64).T) * float(config["logit_scale"])


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
