"""Each mechanism of the Pilutar decoder alone, as its kernels or its part, against the plain functions
(tests/plain_pilutar.py): the layer norm with its bias (gathered rows too); a gate of one number per head; the gated
ReLU and the squared ReLU on a product's 32-bit rows; one RMS norm over all of q and one over all of k with biases ahead
of the rotation in halves; the cap on the scores and a window's edge in the attention kernel (one key's score made to
stand out just inside and just outside the window); gated linear attention whole, in portions cut inside, at and around
its chunks of 32 tokens down to two tokens, token by token, in mixed steps on reused slots, with channels that forget at
once beside channels that keep everything; the router (correction, groups, identity outputs, renormalised weights, ties)
and the whole mixture in both element types, with identity outputs and without."""
import numpy as np
import pytest
import torch

import plain_pilutar as pp

pytestmark = pytest.mark.gpu
F64 = torch.float64
DEV = "cuda:0"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype=None):
    return t.to("cuda", dtype=dtype) if dtype else t.to("cuda")


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device="cuda")


def runs(plan):
    """positions, slots and the device lists of a step from [(slot, first position, count)]."""
    positions, slots, segments, singles, at = [], [], [], [], 0
    for slot, start, count in plan:
        positions += list(range(start, start + count))
        slots += [slot] * count
        if count > 1:
            segments += [at, start, count]
        else:
            singles.append(at)
        at += count
    return (ints(positions), ints(slots), ints(segments) if segments else ints([0])[:0], len(segments) // 3,
            ints(singles) if singles else None, at - len(singles))


# ---- norm, gates, activations ----

@pytest.mark.parametrize("hidden,rows", [(64, 5), (50, 9), (257, 4), (1024, 33), (4100, 3)])
def test_layer_norm_with_bias(hidden, rows):
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(rows, hidden, generator=g) * 3 + 5.0          # a mean far from zero: the variance is of the deviations
    w, b = 1 + 0.3 * torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    want = pp.layer_norm(x.to(F64), w, b, 2e-5)
    for dtype, tolerance in [(torch.float32, 3e-5), (torch.bfloat16, 3e-2)]:
        out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ops.layernorm(dev(x), dev(w), dev(b), out, 2e-5)
        assert torch.allclose(out.cpu().to(F64), want, atol=tolerance, rtol=tolerance)
    index = ints([rows - 1, 0, -1, 1])
    out = torch.empty(4, hidden, device="cuda")
    ops.layernorm(dev(x), dev(w), dev(b), out, 2e-5, rows_index=index)
    assert torch.allclose(out[[0, 1, 3]].cpu().to(F64), want[[rows - 1, 0, 1]], atol=3e-5, rtol=3e-5) and float(out[2].abs().max()) == 0
    out = torch.empty(rows, hidden, device="cuda")
    ops.layernorm(dev(x), dev(w), None, out, 2e-5)
    assert torch.allclose(out.cpu().to(F64), want - b.to(F64), atol=3e-5, rtol=3e-5)


@pytest.mark.parametrize("heads,dv", [(1, 8), (3, 20), (8, 48)])
def test_one_gate_a_head(heads, dv):
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(heads)
    o, wide = torch.randn(7, heads * dv, generator=g), torch.randn(7, heads + 9, generator=g) * 3
    want = (o.to(F64).view(7, heads, dv) * torch.sigmoid(wide[:, 4:4 + heads].to(F64))[:, :, None]).view(7, -1)
    od = dev(o.clone())
    ops.gate_rows(od, dev(wide)[:, 4:4 + heads], ops.GATE_SIGMOID, span=dv)
    assert torch.allclose(od.cpu().to(F64), want, atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("width", [33, 64])
def test_gated_relu_and_squared_relu(width):
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(width)
    both = torch.randn(6, 2 * width, generator=g)
    out = torch.empty(6, width, device="cuda")
    ops.activation_rows(dev(both), out, ops.ACT_RELU, gated=True)
    assert torch.equal(out.cpu(), torch.relu(both[:, :width]) * both[:, width:])
    ops.activation_rows(dev(both)[:, :width], out, ops.ACT_RELU_SQUARED)
    assert torch.allclose(out.cpu(), torch.relu(both[:, :width]) ** 2)


# ---- the attention beside the recurrence ----

def attention_case(seed, hidden, m, T):
    g = torch.Generator().manual_seed(seed)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    bf = lambda t: t.to(torch.bfloat16)
    mat = lambda rows, cols, s=1.0: bf(torch.randn(rows, cols, generator=g) * s / cols ** 0.5)
    w = {"q": mat(H * d, hidden, 2.0), "k": mat(G * d, hidden, 2.0), "v": mat(G * dv, hidden), "o": mat(hidden, H * dv),
         "q.b": bf(0.5 * torch.randn(H * d, generator=g)), "k.b": bf(0.5 * torch.randn(G * d, generator=g)),
         "v.b": bf(0.5 * torch.randn(G * dv, generator=g)),
         "q.norm": bf(1 + 0.3 * torch.randn(H * d, generator=g)), "k.norm": bf(1 + 0.3 * torch.randn(G * d, generator=g))}
    h = bf(torch.randn(T, hidden, generator=g)).to(F64)
    return h, w


def run_mixer(kind, params, weights, h, dtype, steps, state_shape=None, page_size=8):
    """The mixer part alone over a cache manager and step runtime of its own; `steps`: [(first position, count)] of one
    request.  Returns what the part adds to a zero residual, [T, hidden] 64-bit."""
    from lia_rs_b200.cache import CacheManager
    from lia_rs_b200.engine import StepEntry, StepRuntime
    from lia_rs_b200.parts import MIXERS, Runtime
    cls = MIXERS[kind]
    rt = Runtime(DEV, TORCH[dtype])
    cache_request, state_request = cls.cache_request(params), cls.state_request(params)
    cache = CacheManager({0: cache_request} if cache_request else {}, {0: state_request} if state_request else {}, 64, 4,
                         page_size, 1024, TORCH[dtype], DEV)
    step = StepRuntime(cache, 1000, 1024, DEV)
    part = cls(params, {"L." + k: v.to(DEV) for k, v in weights.items()}, "L.", rt)
    slot = cache.admit()
    out = []
    for start, count in steps:
        assert cache.ensure(slot, start, start + count)
        ctx = step.begin([StepEntry(slot, [1] * count, start, [])])
        residual = torch.zeros(count, h.shape[1], device=DEV)
        part.forward(ctx, h[start:start + count].to(DEV).to(TORCH[dtype]), residual, 1.0,
                     kv=ctx.kv_view(0, True) if cache_request else None, state=ctx.state(0) if state_request else None)
        torch.cuda.synchronize()
        step.raise_device_errors()
        out.append(residual.cpu().to(F64))
    return torch.cat(out)


LEFT = [dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, softcap=5.0, mask={"size": 11}, rot={"base": 1000.0, "dims": 8}),
        dict(heads=3, kv_heads=3, dim=24, vdim=8, scale=0.2, softcap=None, mask=None, rot=None),
        dict(heads=8, kv_heads=1, dim=64, vdim=64, scale=0.125, softcap=30.0, mask={"size": 33}, rot={"base": 1e6, "dims": 64}),
        # three query heads a key head: the split-key kernel takes them, the tcgen05 prompt kernel does not (the kernel for
        # every size serves the portions); 32 a key head at head size 32: two groups of 16 in the split-key kernel
        dict(heads=6, kv_heads=2, dim=64, vdim=64, scale=0.125, softcap=8.0, mask={"size": 20}, rot={"base": 1e4, "dims": 32}),
        dict(heads=32, kv_heads=1, dim=32, vdim=32, scale=0.18, softcap=15.0, mask={"size": 50}, rot={"base": 1e4, "dims": 32}),
        dict(heads=4, kv_heads=4, dim=128, vdim=128, scale=0.09, softcap=50.0, mask=None, rot={"base": 5e5, "dims": 64})]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m", LEFT)
def test_capped_attention_with_whole_norms(m, dtype):
    hidden, T, eps = 72, 70, 1e-5
    h, w = attention_case(m["heads"], hidden, m, T)
    want = pp.capped_attention(h, torch.arange(T), w, m, eps)
    params = {"hidden": hidden, "heads": m["heads"], "kv_heads": m["kv_heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
              "scale": m["scale"], "softcap": m["softcap"], "window": m["mask"]["size"] if m["mask"] else None, "rot": m["rot"],
              "biases": "qkv", "qk_norm": "whole", "norm_eps": eps}
    tolerance = 2e-5 if dtype == "float32" else 4e-2
    for steps in ([(0, T)], [(0, 7), (7, 2), (9, 40), (49, 1), (50, 20)], [(0, 30)] + [(t, 1) for t in range(30, T)]):
        got = run_mixer("sink_attention", params, w, h, dtype, steps)
        assert float((got - want).abs().max()) <= tolerance * max(1.0, float(want.abs().max())), steps[:2]


@pytest.mark.parametrize("softcap", [None, 4.0])
@pytest.mark.parametrize("window,page", [(5, 4), (16, 16), (17, 8), (1, 4)])
def test_a_window_s_edge_in_the_attention_kernel(window, page, softcap):
    """One key's score stands out (its query asks for exactly that key, scaled up): the output is that key's value when the
    key is the oldest one inside the window and is not when it is the first one outside; queries in a prompt portion and
    single tokens; the key at a page's border, inside a page and far back."""
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(window * 10 + page)
    T, d, dv = 64, 16, 8
    k = torch.randn(T, 1, d, generator=g)
    v = torch.randn(T, 1, dv, generator=g)
    pages = T // page
    k_pages, v_pages = dev(k.view(pages, page, 1, d).contiguous()), dev(v.view(pages, page, 1, dv).contiguous())
    table = ints(range(pages)).view(1, pages)
    for target in (0, page - 1, page, 37):
        for distance in (window - 1, window):
            t = target + distance
            if t >= T:
                continue
            q = torch.zeros(T, 1, d)
            q[t, 0] = 30.0 * k[target, 0] / k[target, 0].norm() ** 2 * 4.0
            out = torch.zeros(T, dv, device="cuda")
            ops.attention_general(dev(q.view(T, d)), (d, d), None, None, k_pages, None, v_pages, dv, dv, ints(range(T)),
                                  ints([0] * T), table, out, (dv, dv), T, 1, 1, window, 1.0, rows=ints([t]), softcap=softcap)
            torch.cuda.synchronize()
            positions = torch.arange(T)
            scores = (q[t, 0].to(F64) @ k[:, 0].to(F64).T)
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            visible = (positions <= t) & (t - positions < window)
            p = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1)
            want = p @ v[:, 0].to(F64)
            assert torch.allclose(out[t].cpu().to(F64), want, atol=1e-5, rtol=1e-5), (target, distance)
            seen = float(p[target])
            assert (seen > 0.2) if distance == window - 1 and not softcap else True
            assert seen == 0.0 if distance == window else True


# ---- gated linear attention ----

def gla_case(seed, hidden, H, d, dv, rank, tau, T):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.to(torch.bfloat16)
    mat = lambda rows, cols, s=1.0: bf(torch.randn(rows, cols, generator=g) * s / cols ** 0.5)
    w = {"q": mat(H * d, hidden, 2.0), "k": mat(H * d, hidden, 2.0), "v": mat(H * dv, hidden), "g": mat(H * dv, hidden, 2.0),
         "o": mat(hidden, H * dv), "norm": bf(1 + 0.3 * torch.randn(dv, generator=g)), "a1": mat(rank, hidden, 2.0),
         "a2": mat(H * d, rank, 3.0), "a2.b": bf(1.0 + 3.0 * torch.randn(H * d, generator=g))}
    h = bf(torch.randn(T, hidden, generator=g)).to(F64)
    m = {"heads": H, "dim": d, "vdim": dv, "tau": tau}
    return h, w, m


def gla_params(hidden, m, rank, eps):
    return {"hidden": hidden, "heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"], "tau": m["tau"],
            "norm_eps": eps, "decay_rank": rank}


@pytest.mark.parametrize("H,d,dv,rank,tau", [(2, 12, 20, 6, 4.0), (1, 32, 32, 1, 1.0), (3, 10, 6, 5, 16.0), (4, 64, 48, 16, 8.0),
                                             (1, 256, 128, 3, 2.0)])
def test_gated_linear_attention_whole_in_portions_and_token_by_token(H, d, dv, rank, tau):
    hidden, T, eps = 56, 101, 1e-5
    h, w, m = gla_case(H * 7 + d, hidden, H, d, dv, rank, tau, T)
    want, _ = pp.gated_linear_attention(h, w, m, eps)
    params = gla_params(hidden, m, rank, eps)
    scale = max(1.0, float(want.abs().max()))
    whole = run_mixer("gated_linear_attention", params, w, h, "float32", [(0, T)])
    assert float((whole - want).abs().max()) <= 1e-4 * scale
    # portions cut inside, at and around the chunks of 32 tokens, down to two tokens, single tokens in between
    cuts, at, steps = [31, 2, 1, 30, 1, 33, 3], 0, []
    for count in cuts:
        steps.append((at, count))
        at += count
    assert at == T
    portions = run_mixer("gated_linear_attention", params, w, h, "float32", steps)
    assert float((portions - want).abs().max()) <= 1e-4 * scale
    single = run_mixer("gated_linear_attention", params, w, h, "float32", [(t, 1) for t in range(40)])
    assert float((single - want[:40]).abs().max()) <= 1e-4 * scale
    rounded = run_mixer("gated_linear_attention", params, w, h, "bfloat16", [(0, 50), (50, 1), (51, 50)])
    assert float((rounded - want).abs().max()) <= 5e-2 * scale


def test_channels_that_forget_at_once_beside_channels_that_keep_everything():
    """The decay's bias puts half of the key channels at alpha ~ 0 (sigmoid(-30)) and half at alpha ~ 1 (sigmoid(+30)):
    the powers of the first underflow inside a chunk, the second carry the first token to the last one.  Nothing may
    overflow or turn into NaN, and a token 150 positions back still decides through the channels that keep."""
    hidden, H, d, dv, rank, T, eps = 40, 2, 16, 16, 4, 150, 1e-6
    h, w, m = gla_case(5, hidden, H, d, dv, rank, 1.0, T)
    bias = torch.full((H * d,), 30.0)
    bias[::2] = -30.0
    w["a2.b"] = bias.to(torch.bfloat16)
    w["a2"] = torch.zeros_like(w["a2"])
    want, state = pp.gated_linear_attention(h, w, m, eps)
    without, _ = pp.gated_linear_attention(torch.cat([torch.zeros(1, hidden, dtype=F64), h[1:]]), w, m, eps)
    assert float((want[-1] - without[-1]).abs().max()) > 1e-3 * float(want.abs().max())
    params = gla_params(hidden, m, rank, eps)
    for steps in ([(0, T)], [(0, 120)] + [(t, 1) for t in range(120, T)], [(0, 33), (33, 64), (97, 53)]):
        got = run_mixer("gated_linear_attention", params, w, h, "float32", steps)
        assert torch.isfinite(got).all()
        assert float((got - want).abs().max()) <= 1e-4 * max(1.0, float(want.abs().max()))


def test_gated_linear_attention_mixed_steps_on_reused_slots():
    """The kernels alone over two slots: portions beside single tokens, a request that takes over a slot whose state
    another request left (zeroed at admission, as the cache manager does)."""
    from lia_rs_b200.kernels import ops
    hidden, H, d, dv, rank, eps, tau = 48, 2, 12, 20, 3, 2e-6, 4.0
    cases = {name: gla_case(seed, hidden, H, d, dv, rank, tau, T) for name, seed, T in [("a", 1, 70), ("b", 2, 45), ("c", 3, 9)]}
    w = cases["a"][1]
    m = cases["a"][2]
    width = 2 * H * (d + dv) + rank
    rows = {}
    for name, (h, _, _) in cases.items():
        parts = [h @ w[key].to(F64).T for key in ("q", "k", "v", "g", "a1")]
        rows[name] = torch.cat(parts, dim=1).to(torch.float32)
    state = torch.zeros(2, H, d, dv, device="cuda")
    got = {name: torch.zeros(h.shape[0], H * dv) for name, (h, _, _) in cases.items()}
    steps = [[("a", 0, 0, 37), ("b", 1, 0, 2)],
             [("a", 0, 37, 1), ("b", 1, 2, 40)],
             [("b", 1, 42, 1), ("a", 0, 38, 32)],
             [("b", 1, 43, 2)],
             [("c", 1, 0, 9)]]                                              # b is gone: its slot starts over for c
    for step in steps:
        if step[0][0] == "c":
            state[1].zero_()
        positions, slots, segments, n_segments, singles, portion_tokens = runs([(slot, start, count) for _, slot, start, count in step])
        batch = dev(torch.cat([rows[name][start:start + count] for name, _, start, count in step]).contiguous())
        n = batch.shape[0]
        log_decay = torch.empty(n, H * d, device="cuda")
        ops.gla_encode(batch, dev(w["a2"]), dev(w["a2.b"].float()), log_decay, slots, H, d, dv, d ** -0.5, tau)
        chunks = ops.retention_chunks(portion_tokens, n_segments) if n_segments else 0
        scratch = torch.empty(max(1, ops.gla_scratch_floats(chunks, H, d, dv)), device="cuda") if chunks else None
        out = torch.zeros(n, H * dv, device="cuda")
        ops.gla(batch, log_decay, state, segments, n_segments, chunks, singles, slots, dev(w["norm"].float()), out, H, d, dv, eps,
                scratch=scratch)
        torch.cuda.synchronize()
        at = 0
        for name, _, start, count in step:
            got[name][start:start + count] = out[at:at + count].cpu()
            at += count
    for name, (h, _, _) in cases.items():
        ww = dict(w)
        ww["o"] = torch.eye(H * dv)                                          # the kernel's output, ahead of W_o
        want, _ = pp.gated_linear_attention(h, {**ww, "o": torch.eye(H * dv)}, m, eps)
        assert torch.allclose(got[name].to(F64), want, atol=2e-4, rtol=2e-4), name


# ---- the mixture of experts ----

def mixture_case(seed, hidden, experts, top, ff, shared_ff, identity, groups):
    from lia_rs_b200.parts import FEED_FORWARDS
    params = {"hidden": hidden, "experts": experts, "top": top, "router_scale": 1.0, "intermediate": ff,
              "expert_form": "relu_squared", "identity": identity, "correction": True,
              "groups": {"count": groups[0], "keep": groups[1]} if groups else None, "renormalise": True,
              "shared": {"intermediate": shared_ff} if shared_ff else None}
    cls = FEED_FORWARDS["expert_mixture"]
    g = torch.Generator().manual_seed(seed)
    weights = {}
    for spec in cls.tensor_specs(params, "L.mlp."):
        if spec.name.endswith("correction"):
            weights[spec.name] = (0.15 * torch.randn(spec.shape, generator=g)).to(torch.bfloat16)
            continue
        spread = 3.0 if spec.name.endswith("router") else 1.5
        weights[spec.name] = (torch.randn(spec.shape, generator=g) * spread / spec.shape[-1] ** 0.5).to(torch.bfloat16)
    router = {"experts": experts, "top": top, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"router": router, "shared": {"ff": shared_ff} if shared_ff else None}
    return cls, params, weights, mlp


def run_mixture(cls, params, weights, x, dtype, alpha=1.0, base=None, store=False):
    from lia_rs_b200.cache import CacheManager
    from lia_rs_b200.engine import StepEntry, StepRuntime
    from lia_rs_b200.parts import Runtime
    rt = Runtime(DEV, TORCH[dtype])
    cache = CacheManager({}, {}, 64, 4, 2, 512, TORCH[dtype], DEV)
    step = StepRuntime(cache, 1000, 512, DEV)
    part = cls(params, {k: v.to(DEV) for k, v in weights.items()}, "L.mlp.", rt)
    n = x.shape[0]
    residual = (torch.zeros(n, x.shape[1]) if base is None else base.clone()).to(DEV)
    slot = cache.admit()
    assert cache.ensure(slot, 0, n)
    ctx = step.begin([StepEntry(slot, [1] * n, 0, [])])
    part.forward(ctx, x.to(DEV).to(TORCH[dtype]), residual, alpha, store=store)
    torch.cuda.synchronize()
    step.raise_device_errors()
    return residual.cpu().to(F64)


@pytest.mark.parametrize("experts,identity,top,groups", [(5, 1, 2, (3, 2)), (8, 4, 4, (2, 1)), (4, 0, 3, None), (1, 0, 1, None),
                                                        (6, 3, 9, (3, 3)), (2, 2, 1, (2, 1)), (9, 0, 2, (3, 1)), (1, 3, 2, (4, 2))])
def test_router_choice_and_weights(experts, identity, top, groups):
    from lia_rs_b200.kernels import ops
    hidden, n = 48, 64
    outputs = experts + identity
    g = torch.Generator().manual_seed(experts * 10 + identity)
    x = torch.randn(n, hidden, generator=g)
    w = {"router": torch.randn(outputs, hidden, generator=g) * 0.5, "correction": 0.2 * torch.randn(outputs, generator=g)}
    router = {"experts": experts, "top": top, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    fragile = torch.zeros(n, dtype=torch.bool)
    chosen, weights = pp.route(x.to(F64), w, router, fragile)
    ids = torch.empty(n, top, dtype=torch.int32, device="cuda")
    got = torch.empty(n, top, device="cuda")
    ops.moe_route(dev(x), dev(w["router"]), top, 1.0, ids, got, correction=dev(w["correction"]),
                  groups=groups[0] if groups else 0, keep=groups[1] if groups else 0, renormalise=True)
    sound = ~fragile
    assert sound.sum() > n // 2
    assert torch.equal(ids.cpu().long()[sound], chosen[sound])           # the same outputs in the same order
    assert torch.allclose(got.cpu().to(F64)[sound], weights[sound], atol=1e-5, rtol=1e-5)
    assert torch.allclose(got.sum(dim=-1).cpu(), torch.ones(n), atol=1e-5)
    # a negative correction larger than any score: choice scores below zero are still ranked, never taken for "out"
    low = dev(w["correction"] - 5.0)
    ops.moe_route(dev(x), dev(w["router"]), top, 1.0, ids, got, correction=low, groups=groups[0] if groups else 0,
                  keep=groups[1] if groups else 0, renormalise=True)
    assert torch.equal(ids.cpu().long()[sound], chosen[sound])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,experts,top,ff,shared_ff,identity,groups,n",
                         [(64, 5, 2, 40, 24, 1, (3, 2), 37), (128, 8, 4, 64, 96, 4, (2, 1), 150), (50, 3, 3, 30, None, 0, None, 9),
                          (96, 2, 2, 48, 16, 2, (2, 2), 1), (64, 16, 2, 32, None, 0, (4, 2), 300)])
def test_mixture_with_identity_outputs(hidden, experts, top, ff, shared_ff, identity, groups, n, dtype):
    cls, params, weights, mlp = mixture_case(hidden + experts, hidden, experts, top, ff, shared_ff, identity, groups)
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, hidden, generator=g).to(torch.bfloat16)
    plain = {k[len("L.mlp."):]: v for k, v in weights.items()}
    fragile = torch.zeros(n, dtype=torch.bool)
    want = pp.expert_mixture(x.to(F64), plain, mlp, fragile)
    got = run_mixture(cls, params, weights, x.float(), dtype)
    sound = ~fragile
    tolerance = 2e-5 if dtype == "float32" else 3e-2
    scale = max(1.0, float(want.abs().max()))
    assert float((got[sound] - want[sound]).abs().max()) <= tolerance * scale
    base = torch.randn(n, hidden, generator=g)
    added = run_mixture(cls, params, weights, x.float(), dtype, alpha=0.5, base=base)
    assert float((added[sound] - (base.to(F64) + 0.5 * want)[sound]).abs().max()) <= tolerance * scale
    # a token alone gives what it gives in the batch
    alone = run_mixture(cls, params, weights, x[n // 2:n // 2 + 1].float(), dtype)
    assert float((alone[0] - got[n // 2]).abs().max()) <= (1e-6 if dtype == "float32" else 2e-2) * scale
