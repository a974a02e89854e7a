"""Each mechanism of the Zipelix decoder alone, as its kernels, against the plain functions (tests/plain_zipelix.py):
several residual streams (the token's row of copies, a sublayer's read with its norm, its write-back through the mixing
matrix, both in one pass, gathered rows), the row-wise gates and the logits' cap; rotation in interleaved pairs with
the latent's norm and the append to the pages, and a reader of another layer's pages that appends nothing; retention
(rotation in halves, the key's scale, the recurrence whole, in portions cut anywhere around its chunks of 32 tokens,
token by token, in mixed steps on reused slots, with one far token that alone decides under a decay of exactly 1 and
one that must have faded under a small decay); the mixture of experts (scores, the choice with ties, weights that are
not renormalised, the shared expert's gate, every expert's products over the grouped rows, the weighted sum in the
order of the choices, a token alone against the same token in a batch)."""
import numpy as np
import pytest
import torch

import plain_zipelix as pz

pytestmark = pytest.mark.gpu
F64 = torch.float64


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


# ---- several residual streams ----

@pytest.mark.parametrize("streams,hidden,rows", [(1, 64, 5), (2, 50, 9), (3, 257, 4), (4, 320, 33), (8, 96, 7)])
def test_streams_read_norm_and_write_back(streams, hidden, rows):
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(streams * 100 + hidden)
    x = torch.randn(rows, streams, hidden, generator=g) * 2
    hc = {"in": torch.randn(streams, generator=g), "mix": torch.eye(streams) + 0.3 * torch.randn(streams, streams, generator=g),
          "out": torch.randn(streams, generator=g)}
    w = 1 + 0.3 * torch.randn(hidden, generator=g)
    y = torch.randn(rows, hidden, generator=g)
    eps = 3e-6
    # the read: u = sum_s in[s] x_s and its norm
    u_want = torch.einsum("s,tsw->tw", hc["in"].to(F64), x.to(F64))
    for dtype, tolerance in [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)]:
        xd = dev(x.reshape(rows, streams * hidden).contiguous())
        u = torch.empty(rows, hidden, device="cuda")
        normed = torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ops.hyper_step(xd, streams, in_weights=dev(hc["in"]), u=u, norm_weight=dev(w), normed=normed, eps=eps)
        assert torch.allclose(u.cpu().to(F64), u_want, atol=2e-5, rtol=1e-5)
        assert torch.allclose(normed.float().cpu().to(F64), pz.norm(u_want, w, eps), atol=tolerance, rtol=tolerance)
        assert torch.equal(xd.cpu(), x.reshape(rows, -1))                 # a read leaves the streams as they were
    # the write-back alone, from the old streams all at once (mix is indexed [from, to])
    want = torch.einsum("sr,tsw->trw", hc["mix"].to(F64), x.to(F64)) + hc["out"].to(F64)[None, :, None] * y.to(F64)[:, None, :]
    xd = dev(x.reshape(rows, -1).contiguous())
    ops.hyper_step(xd, streams, y=dev(y), mix=dev(hc["mix"]), out_weights=dev(hc["out"]))
    assert torch.allclose(xd.cpu().to(F64).view(rows, streams, hidden), want, atol=3e-5, rtol=1e-5)
    # write-back and the next sublayer's read in one pass
    in2, w2 = torch.randn(streams, generator=g), 1 + 0.3 * torch.randn(hidden, generator=g)
    xd = dev(x.reshape(rows, -1).contiguous())
    u, normed = torch.empty(rows, hidden, device="cuda"), torch.empty(rows, hidden, device="cuda")
    ops.hyper_step(xd, streams, y=dev(y), mix=dev(hc["mix"]), out_weights=dev(hc["out"]), in_weights=dev(in2), u=u,
                   norm_weight=dev(w2), normed=normed, eps=eps)
    u2 = torch.einsum("s,tsw->tw", in2.to(F64), want)
    assert torch.allclose(xd.cpu().to(F64).view(rows, streams, hidden), want, atol=3e-5, rtol=1e-5)
    assert torch.allclose(u.cpu().to(F64), u2, atol=5e-5, rtol=1e-5)
    assert torch.allclose(normed.cpu().to(F64), pz.norm(u2, w2, eps), atol=5e-5, rtol=2e-5)
    # the plain sum of the streams of chosen rows (what the model's norm reads at the end)
    pick = [rows - 1, 0, rows // 2]
    total = torch.empty(len(pick), hidden, device="cuda")
    ops.hyper_step(dev(x.reshape(rows, -1).contiguous()), streams, rows_index=ints(pick), u=total)
    assert torch.allclose(total.cpu().to(F64), x.to(F64).sum(dim=1)[pick], atol=2e-5, rtol=1e-5)


def test_streams_start_as_copies_of_the_embedding():
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    for dtype in (torch.float32, torch.bfloat16):
        table = torch.randn(19, 50, generator=g).to(dtype)
        tokens = [3, 18, 0, 3, 7]
        for streams in (1, 3, 5):
            out = torch.zeros(len(tokens), streams * 50, device="cuda")
            ops.embedding_streams(ints(tokens), dev(table), out, streams)
            want = table.float()[tokens][:, None, :].expand(-1, streams, -1).reshape(len(tokens), -1)
            assert torch.equal(out.cpu(), want)


def test_gates_and_the_cap():
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    wide = torch.randn(13, 90, generator=g) * 3
    o = torch.randn(13, 37, generator=g)
    for act, plain in [(ops.GATE_SIGMOID, torch.sigmoid), (ops.GATE_SILU, pz.silu)]:
        for dtype, tolerance in [(torch.float32, 2e-6), (torch.bfloat16, 2e-2)]:
            od = dev(o, dtype)
            ops.gate_rows(od, dev(wide)[:, 11:48], act)                  # the gate: columns of wider rows
            want = o.to(dtype).to(F64) * plain(wide[:, 11:48].to(F64))
            assert torch.allclose(od.float().cpu().to(F64), want, atol=tolerance, rtol=tolerance)
    z = torch.randn(7, 61, generator=g) * 40
    for cap in (4.0, 15.0, 50.0):
        zd = dev(z.clone())
        ops.softcap_rows(zd, cap)
        assert torch.allclose(zd.cpu().to(F64), cap * torch.tanh(z.to(F64) / cap), atol=1e-5, rtol=2e-6)
        assert float(zd.abs().max()) <= cap


# ---- rotation in interleaved pairs, the latent and the pages ----

class Pages:
    def __init__(self, slots, max_tokens, page_size, seed=0):
        self.page_size = page_size
        self.blocks = (max_tokens + page_size - 1) // page_size
        self.num_pages = slots * self.blocks + 2
        order = torch.randperm(self.num_pages, generator=torch.Generator().manual_seed(seed))[:slots * self.blocks]
        self.table = order.view(slots, self.blocks).to(torch.int32).cuda().contiguous()

    def empty(self, dim, dtype=torch.float32):
        return torch.zeros((self.num_pages, self.page_size, 1, dim), dtype=dtype, device="cuda")

    def at(self, pages, slot, position):
        return pages[int(self.table[slot, position // self.page_size]), position % self.page_size, 0]


@pytest.mark.parametrize("H,d,dr,dims,rank", [(3, 12, 8, 8, 20), (1, 16, 16, 6, 48), (5, 8, 32, 32, 17), (2, 24, 4, 2, 64)])
def test_interleaved_pairs_latent_norm_and_append(H, d, dr, dims, rank):
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 10 + dr)
    page, base, eps = 4, 700.0, 2e-6
    cache = Pages(2, 96, page, seed=H)
    where = list(range(29, 40)) + [0, 3, 64]                               # a run across page borders, and single rows
    slots = [1] * 11 + [0, 0, 1]
    n = len(where)
    positions = torch.tensor(where)
    q_rows, shared = torch.randn(n, H * (d + dr), generator=g), torch.randn(n, rank + dr, generator=g)
    weight = 1 + 0.3 * torch.randn(rank, generator=g)
    freq = pz.frequencies(base, dims)
    q_plain, q_rot = torch.zeros(H, n, d, device="cuda"), torch.zeros(n, H * dr, device="cuda")
    latent_pages, part_pages = cache.empty(rank), cache.empty(dr)
    ops.latent_prepare(dev(q_rows), dev(shared), dev(weight), eps, dev(freq, torch.float32), dims, ints(where), ints(slots),
                       cache.table, q_plain, q_rot, latent_pages, part_pages, H, d, dr, rank, pairs=True)
    q = q_rows.to(F64).view(n, H, d + dr)
    assert torch.allclose(q_plain.cpu().to(F64).transpose(0, 1), q[:, :, :d], atol=1e-6)
    want_q = pz.rotate_interleaved(q[:, :, d:].contiguous(), positions, base, dims)
    assert torch.allclose(q_rot.cpu().to(F64).view(n, H, dr), want_q, atol=3e-5, rtol=2e-5)
    latent = pz.norm(shared.to(F64)[:, :rank], weight, eps)
    part = pz.rotate_interleaved(shared.to(F64)[:, rank:].contiguous(), positions, base, dims)
    for r in range(n):
        assert torch.allclose(cache.at(latent_pages, slots[r], where[r]).cpu().to(F64), latent[r], atol=2e-5, rtol=2e-5)
        assert torch.allclose(cache.at(part_pages, slots[r], where[r]).cpu().to(F64), part[r], atol=3e-5, rtol=2e-5)
    if dims < dr:                                                          # what lies behind rot.dims passes unchanged
        assert torch.allclose(q_rot.cpu().view(n, H, dr)[:, :, dims:].to(F64), q[:, :, d + dims:], atol=1e-6)
    # a layer that reads another layer's pages: its queries are prepared, the pages stay as they are
    before = (latent_pages.clone(), part_pages.clone())
    q_plain.zero_(), q_rot.zero_()
    ops.latent_prepare(dev(q_rows), None, None, eps, dev(freq, torch.float32), dims, ints(where), ints(slots), cache.table,
                       q_plain, q_rot, latent_pages, part_pages, H, d, dr, rank, pairs=True)
    assert torch.allclose(q_rot.cpu().to(F64).view(n, H, dr), want_q, atol=3e-5, rtol=2e-5)
    assert torch.equal(latent_pages, before[0]) and torch.equal(part_pages, before[1])


# ---- retention ----

def retention_case(seed, H, d, dv, T, rot, decays, width=24):
    """Random inputs and projections of one sequence, the plain result (W_o = identity), and the 32-bit rows [q | k | v | g]."""
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(T, width, generator=g, dtype=F64)
    w = {"q": torch.randn(H * d, width, generator=g, dtype=F64), "k": torch.randn(H * d, width, generator=g, dtype=F64),
         "v": torch.randn(H * dv, width, generator=g, dtype=F64), "g": torch.randn(H * dv, width, generator=g, dtype=F64) * 0.3,
         "o": torch.eye(H * dv, dtype=F64)}
    m = {"heads": H, "dim": d, "vdim": dv, "decay": decays}
    if rot:
        m["rot"] = rot
    return h, w, m


def retention_rows(h, w):
    return torch.cat([h @ w["q"].T, h @ w["k"].T, h @ w["v"].T, h @ w["g"].T], dim=1).to(torch.float32)


def retention_steps(rows_of, m, eps, steps, n_slots=4):
    """Runs `steps` (each a list of (sequence, slot, first position, count); a slot's state is zeroed when a sequence
    begins in it, as the cache manager does at admission) through the encode and recurrence kernels; returns
    {sequence: [T, H dv] 32-bit}."""
    from lia_rs_b200.kernels import ops
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    rot = m.get("rot")
    dims = rot["dims"] if rot else 0
    freq = dev(pz.frequencies(rot["base"], dims), torch.float32) if rot else torch.zeros(1, device="cuda")
    state = torch.full((n_slots, H, d, dv), 7.0, device="cuda")            # what an earlier request left in the slot
    decay = torch.tensor(m["decay"], dtype=torch.float32, device="cuda")
    out = {name: torch.zeros(r.shape[0], H * dv) for name, r in rows_of.items()}
    for step in steps:
        plan = [(slot, start, count) for _, slot, start, count in step]
        for slot, start, _ in plan:
            if start == 0:
                state[slot].zero_()
        positions, slots, segments, n_segments, singles, portion_tokens = runs(plan)
        rows = torch.cat([rows_of[name][start:start + count] for name, _, start, count in step]).to("cuda").contiguous()
        ops.retention_encode(rows, freq, dims, positions, slots, H, d, float(d) ** -0.5)
        chunks = ops.retention_chunks(portion_tokens, n_segments) if n_segments else 0
        scratch = torch.empty(max(1, ops.retention_scratch_floats(chunks, H, d, dv)), device="cuda") if chunks else None
        o = torch.zeros(rows.shape[0], H * dv, device="cuda")
        ops.retention(rows, decay, state, segments, n_segments, chunks, singles, slots, o, H, d, dv, eps, scratch=scratch)
        at = 0
        for name, _, start, count in step:
            out[name][start:start + count] = o[at:at + count].cpu()
            at += count
    return out


def plain_retention_output(h, w, m, eps):
    """The plain mixer with W_o = identity and the gate divided out: each head's o over its root mean square, times silu(g)."""
    return pz.retention(h, torch.arange(h.shape[0]), w, m, eps)


@pytest.mark.parametrize("H,d,dv,rot,decays", [
    (2, 16, 16, {"base": 100.0, "dims": 16}, [0.9, 1.0]),
    (3, 10, 6, {"base": 300.0, "dims": 6}, [0.5, 0.97, 0.999]),
    (1, 32, 40, None, [0.96]),
    (4, 24, 12, {"base": 1e4, "dims": 24}, [1.0, 1.0, 0.8, 0.99])])
def test_retention_whole_in_portions_and_token_by_token(H, d, dv, rot, decays):
    eps, T = 1e-5, 101
    h, w, m = retention_case(H * 7 + d, H, d, dv, T, rot, decays)
    want = plain_retention_output(h, w, m, eps)
    rows = {"a": retention_rows(h, w)}
    whole = retention_steps(rows, m, eps, [[("a", 1, 0, T)]])["a"]
    assert torch.allclose(whole.to(F64), want, atol=2e-4, rtol=2e-4)
    # portions cut inside, at and around the chunks of 32 tokens, down to two tokens, single tokens in between
    cuts, at, steps = [31, 2, 1, 30, 1, 33, 3], 0, []
    for count in cuts:
        steps.append([("a", 2, at, count)])
        at += count
    assert at == T
    portions = retention_steps(rows, m, eps, steps)["a"]
    assert torch.allclose(portions.to(F64), want, atol=2e-4, rtol=2e-4)
    single = retention_steps({"a": rows["a"][:40]}, m, eps, [[("a", 0, t, 1)] for t in range(40)])["a"]
    assert torch.allclose(single.to(F64), want[:40], atol=2e-4, rtol=2e-4)


def test_retention_mixed_steps_on_reused_slots():
    eps, H, d, dv = 2e-6, 2, 12, 20
    rot, decays = {"base": 50.0, "dims": 8}, [0.93, 1.0]
    cases = {name: retention_case(seed, H, d, dv, T, rot, decays) for name, seed, T in [("a", 1, 70), ("b", 2, 45), ("c", 3, 9)]}
    m = cases["a"][2]
    rows = {name: retention_rows(h, w_) for name, (h, w_, _) in cases.items()}
    # (the projections differ per sequence only to make the inputs differ: the kernel sees rows)
    steps = [[("a", 0, 0, 37), ("b", 1, 0, 2)],
             [("a", 0, 37, 1), ("b", 1, 2, 40)],
             [("b", 1, 42, 1), ("a", 0, 38, 32)],
             [("b", 1, 43, 2)],
             [("c", 1, 0, 9)]]                                              # b is gone: its slot starts over for c
    got = retention_steps(rows, m, eps, steps, n_slots=2)
    for name, (h, w_, _) in cases.items():
        want = plain_retention_output(h, w_, m, eps)
        upto = {"a": 70, "b": 45, "c": 9}[name]
        assert torch.allclose(got[name][:upto].to(F64), want[:upto], atol=2e-4, rtol=2e-4), name


def test_retention_keeps_a_far_token_under_decay_one_and_forgets_it_under_a_small_one():
    eps, H, d, dv, T = 1e-6, 2, 16, 16, 150
    h, w, m = retention_case(11, H, d, dv, T, None, [1.0, 0.5])
    rows = retention_rows(h, w).view(T, -1).clone()
    q, k, v = rows[:, :H * d].view(T, H, d), rows[:, H * d:2 * H * d].view(T, H, d), rows[:, 2 * H * d:2 * H * d + H * dv].view(T, H, dv)
    k[0] *= 40.0                                                            # one key that the last query asks for
    v[0] *= 40.0
    q[T - 1] = k[0] / 40.0
    # the plain result from the same rows
    want = torch.zeros(T, H, dv, dtype=F64)
    for head, decay in enumerate(m["decay"]):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay * S + torch.outer(k[t, head].to(F64) * d ** -0.5, v[t, head].to(F64))
            want[t, head] = S.T @ q[t, head].to(F64)
    direction = lambda a, b: float((a * b).sum() / (a.norm() * b.norm()))
    assert direction(want[T - 1, 0], v[0, 0].to(F64)) > 0.95 and abs(direction(want[T - 1, 1], v[0, 1].to(F64))) < 0.6
    gate = rows[:, 2 * H * d + H * dv:].to(F64)
    want = pz.rms(want, eps).reshape(T, H * dv) * pz.silu(gate)
    for steps in ([[("a", 0, 0, T)]], [[("a", 0, 0, 120)]] + [[("a", 0, t, 1)] for t in range(120, T)]):
        got = retention_steps({"a": rows}, m, eps, steps)["a"]
        assert torch.allclose(got.to(F64), want, atol=3e-4, rtol=3e-4)


# ---- the mixture of experts ----

DEV = "cuda:0"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def mixture_case(seed, hidden, experts, top, ff, shared_ff, scale):
    from lia_rs_b200.parts import FEED_FORWARDS
    params = {"hidden": hidden, "experts": experts, "top": top, "router_scale": scale, "intermediate": ff,
              "shared": {"intermediate": shared_ff} if shared_ff else None}
    cls = FEED_FORWARDS["expert_mixture"]
    g = torch.Generator().manual_seed(seed)
    weights = {}
    for spec in cls.tensor_specs(params, "L.mlp."):
        spread = 3.0 if spec.name.endswith("router") else 1.5
        weights[spec.name] = (torch.randn(spec.shape, generator=g) * spread / spec.shape[-1] ** 0.5).to(torch.bfloat16)
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}, "shared": {"ff": shared_ff} if shared_ff else None}
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


def plain_mixture(weights, mlp, x):
    w = {k[len("L.mlp."):]: v for k, v in weights.items()}
    return pz.expert_mixture(x.to(F64), w, mlp)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hidden,experts,top,ff,shared_ff,scale,n", [
    (64, 5, 2, 40, 24, 1.7, 37),            # few rows an expert: the narrowest tiles
    (72, 2, 2, 136, None, 0.6, 9),          # all experts chosen; no shared expert; sizes that are not multiples of 128
    (128, 9, 1, 200, 64, 1.0, 300),         # one choice; hundreds of rows: wider tiles, several an expert
    (96, 16, 4, 48, 16, 2.5, 140),          # many experts, some of them possibly without a row
    (50, 3, 2, 21, 10, 1.0, 12)])           # sizes that only the 32-bit pipes take
def test_expert_mixture_against_the_plain_one(dtype, hidden, experts, top, ff, shared_ff, scale, n):
    cls, params, weights, mlp = mixture_case(hidden + experts, hidden, experts, top, ff, shared_ff, scale)
    x = torch.randn(n, hidden, generator=torch.Generator().manual_seed(n)).to(torch.bfloat16).float()
    base = torch.randn(n, hidden, generator=torch.Generator().manual_seed(n + 1))
    marks = torch.zeros(n, dtype=torch.bool)
    w = {k[len("L.mlp."):]: v for k, v in weights.items()}
    want = pz.expert_mixture(x.to(F64), w, mlp, fragile=marks)
    got = run_mixture(cls, params, weights, x, dtype, alpha=0.7, base=base)
    sound = ~marks
    limit = (2e-5 if dtype == "float32" else 1.5e-2) * max(1.0, float(want.abs().max()))
    assert float((got - (base.to(F64) + 0.7 * want))[sound].abs().max()) <= limit
    stored = run_mixture(cls, params, weights, x, dtype, alpha=0.7, base=base, store=True)
    assert float((stored - 0.7 * want)[sound].abs().max()) <= limit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_token_alone_gives_what_it_gives_in_a_batch(dtype):
    cls, params, weights, mlp = mixture_case(5, 64, 6, 3, 72, 32, 1.3)
    x = torch.randn(150, 64, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).float()
    batch = run_mixture(cls, params, weights, x, dtype)
    for t in (0, 77, 149):
        alone = run_mixture(cls, params, weights, x[t:t + 1], dtype)
        if dtype == "float32":
            assert torch.equal(alone[0], batch[t])                          # every row's sums run in one fixed order
        else:
            assert float((alone[0] - batch[t]).abs().max()) <= 2e-3 * max(1.0, float(batch[t].abs().max()))


def test_router_scores_choice_ties_and_weights():
    from lia_rs_b200.kernels import ops
    n, hidden, experts, top, scale = 23, 48, 7, 3, 1.9
    g = torch.Generator().manual_seed(3)
    x = torch.randn(n, hidden, generator=g)
    router = torch.randn(experts + 1, hidden, generator=g) * 0.2
    router[4] = router[1]                                                   # two experts of equal score: the lower index first
    ids = torch.zeros(n, top, dtype=torch.int32, device="cuda")
    weights, gate = torch.zeros(n, top, device="cuda"), torch.zeros(n, device="cuda")
    ops.moe_route(dev(x), dev(router), top, scale, ids, weights, gate)
    z = x.to(F64) @ router.to(F64).T
    s = torch.softmax(z[:, :experts], dim=-1)
    for t in range(n):
        ranked = sorted(range(experts), key=lambda e: (-float(s[t, e]) if e != 4 else -float(s[t, 1]), e))[:top]
        assert ids[t].tolist() == ranked
        assert torch.allclose(weights[t].cpu().to(F64), torch.tensor([float(s[t, e]) for e in ranked], dtype=F64) * scale, atol=1e-6)
    assert float(weights.sum(dim=1).max()) < scale                          # not renormalised: the chosen scores as they are
    assert torch.allclose(gate.cpu().to(F64), torch.sigmoid(z[:, experts]), atol=1e-6)
