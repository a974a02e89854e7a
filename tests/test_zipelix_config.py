"""What needs no GPU of the Zipelix decoder: its configuration and its refusals, the registry, the model description
(tensor names, parts chosen layer by layer, which layer reads whose cache, caches and states), random weights through
the loader, the plain implementation's mechanisms against hand-made cases, and the cache manager with latent pages that
several layers read beside state slots."""
import copy
import json
import random

import pytest
import torch

import plain_zipelix as pz
import zipelix_helpers as zh
from lia_rs_b200.cache import CacheManager
from lia_rs_b200.config import ConfigError, ZipelixConfig, resolve_architecture
from lia_rs_b200.parts import KVCacheRequest

F64 = torch.float64
NAMES = list(zh.ZIPELIX) + [f"random-{seed}" for seed in (201, 202, 203, 204)]


def raw_config(name):
    return zh.ZIPELIX[name]["config"] if name in zh.ZIPELIX else zh.random_configuration(int(name.split("-")[1]))


@pytest.mark.parametrize("name", NAMES)
def test_configuration_round_trip_and_registry(name):
    raw = raw_config(name)
    architecture = resolve_architecture(raw)
    assert architecture.name == "Zipelix" and architecture.config_class is ZipelixConfig
    config = ZipelixConfig.from_dict(raw)
    again = ZipelixConfig.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config and again.to_dict() == config.to_dict()
    assert [l["type"] for l in config.layers] == [l["type"] for l in raw["layers"]]
    assert config.streams == raw.get("streams") and config.logit_softcap == raw.get("logit_softcap")


def test_configuration_refusals():
    good = zh.ZIPELIX["zip-A"]["config"]

    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        return raw

    cases = [
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "at most"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
        (lambda r: r["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
        (lambda r: r["layers"][1].update(type="attention"), "not known"),
        (lambda r: r["layers"][1]["mlp"].update(kind="experts"), "not known"),
        (lambda r: r["layers"][1]["mlp"]["router"].update(top=6), "exceeds"),
        (lambda r: r["layers"][1]["mlp"]["router"].pop("scale"), "router.scale"),
        (lambda r: r["layers"][1]["mixer"].update(decay=[0.9, 0.9]), "one number per head"),
        (lambda r: r["layers"][1]["mixer"].update(decay=[0.9, 1.5, 0.9]), r"\(0, 1\]"),
        (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
        (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "latent-attention layer"),
        (lambda r: r["layers"][4]["mixer"].update(kv_from=2), "cache of its own"),
        (lambda r: r["layers"][2]["mixer"].update(kv_rank=16), "must equal"),
        (lambda r: r["layers"][2]["mixer"]["rot"].update(base=5.0), "must equal"),
        (lambda r: r.pop("width"), "width"),
        (lambda r: r["norm"].pop("eps"), "norm.eps"),
        (lambda r: r.update(streams=0), "streams"),
        (lambda r: r.update(logit_softcap=-1.0), "logit_softcap"),
        (lambda r: r.update(layers=[]), "non-empty"),
    ]
    for change, words in cases:
        with pytest.raises(ConfigError, match=words):
            ZipelixConfig.from_dict(broken(change))
    # sizes beyond the kernels are refused when the model is described, before any tensor is read
    architecture = resolve_architecture(good)
    for change, words in [(lambda r: r.update(streams=9), "streams"),
                          (lambda r: r["layers"][3]["mixer"].update(dim=300, rot={"base": 50.0, "dims": 24}), "head_dim"),
                          (lambda r: r["layers"][1]["mlp"]["router"].update(experts=2000), "experts")]:
        with pytest.raises(ValueError, match=words):
            architecture.build(ZipelixConfig.from_dict(broken(change))).check()


@pytest.mark.parametrize("name", NAMES)
def test_model_description(name):
    raw = raw_config(name)
    config = ZipelixConfig.from_dict(raw)
    spec = resolve_architecture(raw).build(config)
    assert spec.max_positions is None and spec.position_table_name is None and spec.head_name is None
    assert spec.streams == (raw.get("streams") or 1) and spec.logit_softcap == raw.get("logit_softcap")
    assert [l.mixer.kind for l in spec.layers] == [l["type"] for l in raw["layers"]]
    assert all(l.arrangement == "hyper" for l in spec.layers)
    names = {s.name: tuple(s.shape) for s in spec.tensor_specs() if not s.optional}
    width, s = raw["width"], raw.get("streams")
    assert names["embed"] == (raw["vocab"], width) and names["final.norm"] == (width,) and "head" not in names
    caches, states = spec.cache_requests(), spec.state_requests()
    for i, layer in enumerate(raw["layers"]):
        m, mlp, p = layer["mixer"], layer["mlp"], f"l{i}."
        entry = spec.schedule[i]
        assert names[p + "norm1"] == (width,) and (p + "norm2" in names) == (mlp is not None)
        for q, present in (("hc1.", True), ("hc2.", mlp is not None)):
            assert (p + q + "mix" in names) == (present and s is not None)
            if present and s is not None:
                assert names[p + q + "in"] == (s,) and names[p + q + "out"] == (s,) and names[p + q + "mix"] == (s, s)
        if layer["type"] == "latent_attention":
            H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            assert names[p + "mix.q"] == (H * (d + dr), width) and names[p + "mix.g"] == (H * dv, width)
            assert names[p + "mix.uk"] == (H * d, rank) and names[p + "mix.uv"] == (H * dv, rank) and names[p + "mix.o"] == (width, H * dv)
            own = m.get("kv_from") is None
            assert (p + "mix.dkv" in names) == own == (p + "mix.dkv.norm" in names) == (i in caches) == entry.writes
            assert entry.cache == (i if own else m["kv_from"])
            if own:
                assert names[p + "mix.dkv"] == (rank + dr, width) and names[p + "mix.dkv.norm"] == (rank,)
                assert caches[i] == KVCacheRequest(1, rank, None, v_head_dim=dr)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            assert names[p + "mix.q"] == (H * d, width) == names[p + "mix.k"] and names[p + "mix.v"] == (H * dv, width) == names[p + "mix.g"]
            assert names[p + "mix.o"] == (width, H * dv)
            assert entry.cache is None and i not in caches and states[i].shape == (H, d, dv) and states[i].dtype == torch.float32
        if mlp and mlp["kind"] == "dense":
            assert names[p + "mlp.gate"] == (mlp["ff"], width) == names[p + "mlp.up"] and names[p + "mlp.down"] == (width, mlp["ff"])
        elif mlp:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            assert names[p + "mlp.router"] == (E, width) and p + f"mlp.e{E}.up" not in names
            assert all(names[p + f"mlp.e{e}.gate"] == (ff, width) and names[p + f"mlp.e{e}.down"] == (width, ff) for e in range(E))
            assert (p + "mlp.shared.sg" in names) == bool(mlp.get("shared"))
            if mlp.get("shared"):
                assert names[p + "mlp.shared.sg"] == (1, width) and names[p + "mlp.shared.up"] == (mlp["shared"]["ff"], width)


@pytest.mark.parametrize("name", ["zip-A", "zip-D"])
def test_random_weights_pass_the_loader(tmp_path, name):
    from lia_rs_b200.weights import load_weights, write_random_model
    raw = zh.ZIPELIX[name]["config"]
    config = ZipelixConfig.from_dict(raw)
    folder = write_random_model(config, str(tmp_path / "m"), seed=5)
    spec = resolve_architecture(raw).build(config)
    tensors = load_weights(folder, spec.tensor_specs())
    assert set(tensors) == {s.name for s in spec.tensor_specs() if not s.optional}
    if name == "zip-A":          # the mixing matrices start as the identity, the other coefficients as ones
        assert torch.equal(tensors["l1.hc2.mix"].float(), torch.eye(3)) and torch.equal(tensors["l0.hc1.in"].float(), torch.ones(3))


def test_plain_mechanisms_on_cases_made_by_hand():
    """The plain implementation itself: rotations that are turns by known angles, the recurrence against its closed sum,
    the mixture's choice and weights, the streams' update with an asymmetric matrix."""
    x = torch.tensor([[1.0, 0.0, 0.0, 1.0, 5.0, 7.0]], dtype=F64)
    quarter = torch.tensor([1]) * 1
    # base 1: every frequency is 1; position pi/2 is not an integer, so use base e^... instead: angle = p * f_0 = 1 rad
    out = pz.rotate_interleaved(x, quarter, 1.0, 4)
    c, s = torch.cos(torch.tensor(1.0, dtype=F64)), torch.sin(torch.tensor(1.0, dtype=F64))
    assert torch.allclose(out, torch.stack([c, s, -s, c, torch.tensor(5.0, dtype=F64), torch.tensor(7.0, dtype=F64)])[None])
    out = pz.rotate_halves(x, quarter, 1.0, 4)                  # pairs (x0, x2) and (x1, x3)
    assert torch.allclose(out[0, :4], torch.stack([c, -s, s, c]))
    f = pz.frequencies(100.0, 4)
    assert torch.allclose(f, torch.tensor([1.0, 0.1], dtype=F64))
    # retention with identity-like projections: o_t = sum_j decay^(t-j) (q_t . k_j / sqrt(d)) v_j
    g = torch.Generator().manual_seed(0)
    T, H, d, dv = 7, 2, 4, 3
    h = torch.randn(T, 6, generator=g, dtype=F64)
    w = {k: torch.randn(n, 6, generator=g, dtype=F64) for k, n in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv))}
    w["o"] = torch.eye(H * dv, dtype=F64)
    m = {"heads": H, "dim": d, "vdim": dv, "decay": [0.5, 1.0]}
    got = pz.retention(h, torch.arange(T), w, m, 1e-6)
    q, k, v = (h @ w[n].T for n in ("q", "k", "v"))
    for t in range(T):
        for head in range(H):
            o = sum(m["decay"][head] ** (t - j) * (q[t, head * d:(head + 1) * d] @ k[j, head * d:(head + 1) * d]) / 2.0
                    * v[j, head * dv:(head + 1) * dv] for j in range(t + 1))
            o = o / torch.sqrt((o * o).mean() + 1e-6) * pz.silu(h[t] @ w["g"].T)[head * dv:(head + 1) * dv]
            assert torch.allclose(got[t, head * dv:(head + 1) * dv], o, atol=1e-12)
    # the mixture: router rows that make expert 2, then 0, the largest; weights are the scores times the scale
    h = torch.tensor([[1.0, 0.0]], dtype=F64)
    w = {"router": torch.tensor([[1.0, 0.0], [-3.0, 0.0], [2.0, 0.0]], dtype=F64)}
    for e in range(3):
        w[f"e{e}.gate"] = torch.full((1, 2), 10.0, dtype=F64)      # silu(10) is 10 within 5e-4
        w[f"e{e}.up"] = torch.tensor([[float(e + 1), 0.0]], dtype=F64)
        w[f"e{e}.down"] = torch.tensor([[1.0], [0.0]], dtype=F64)
    out = pz.expert_mixture(h, w, {"router": {"experts": 3, "top": 2, "scale": 2.0}})
    scores = torch.softmax(torch.tensor([1.0, -3.0, 2.0], dtype=F64), 0)
    want = 2.0 * (scores[2] * 3.0 + scores[0] * 1.0) * pz.silu(torch.tensor(10.0, dtype=F64))
    assert torch.allclose(out[0, 0], want) and out[0, 1] == 0
    # the streams: mix is indexed [from, to]
    streams = torch.tensor([[[1.0]], [[10.0]]], dtype=F64)
    hc = {"hc1.in": torch.tensor([1.0, 0.0]), "hc1.out": torch.tensor([0.0, 1.0]), "hc1.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]])}
    new = pz.hyper_step(streams, hc, "hc1.", lambda z: 100.0 * z, torch.ones(1), 0.0)
    assert new[:, 0, 0].tolist() == [0.0, 101.0]                # stream 0 went to stream 1; y = 100 * sign(1) only there


def test_cache_manager_with_shared_latents_and_state_slots():
    """One group of latent pages that three layers read (one writes), state slots of two sizes: random admissions,
    portions and releases keep the invariants; pages and slots return and are given out again."""
    from lia_rs_b200.parts.base import StateRequest
    latent = KVCacheRequest(1, 32, None, v_head_dim=8)
    manager = CacheManager({0: latent, 3: KVCacheRequest(1, 48, None, v_head_dim=16)},
                           {1: StateRequest((2, 4, 6), torch.float32), 2: StateRequest((3, 8, 8), torch.float32)},
                           num_pages=24, page_size=8, max_slots=3, max_context=120, dtype=torch.float32)
    rng = random.Random(3)
    at, seen = {}, set()
    for _ in range(400):
        if at and rng.random() < 0.15:
            slot = rng.choice(list(at))
            manager.release(slot)
            del at[slot]
        elif len(at) < 3 and rng.random() < 0.3:
            slot = manager.admit()
            assert slot is not None and slot not in at
            seen.add(slot)
            at[slot] = 0
        elif at:
            slot = rng.choice(list(at))
            count = rng.choice([1, 1, 2, 5, 17])
            if at[slot] + count <= 120 and manager.ensure(slot, at[slot], at[slot] + count):
                at[slot] += count
        manager.check()
    assert seen == {0, 1, 2}
