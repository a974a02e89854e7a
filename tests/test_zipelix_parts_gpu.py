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
