"""Tiny Zipelix configurations for the tests, their model folders with random weights, and the comparison with the
plain implementation (tests/plain_zipelix.py).

The configurations differ in everything that config.json gives: widths and vocabularies; 1 to 5 streams and a model
without hyper-connections at all; the order of the two kinds of layer (each first, last and alone); latent attention
with 1 to 5 heads, ranks smaller and larger than a head, rotated parts of which all or only the first dimensions turn,
unrotated sizes that differ from the rotated and from the values', layers that read an earlier layer's latents (one
source read by two layers, two sources in one model, a reader directly behind and far behind its source); retention
with 1 to 4 heads, key and value head sizes equal and unequal and not multiples of four, decays equal to 1, close to 1
and small, rotation of all, part or none of a head; dense feed-forwards, mixtures with 2 to 9 experts of which 1 to
all are chosen, with and without a shared expert, router scales other than 1, and layers without a feed-forward; a
soft cap present and absent."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_zipelix


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, mlp, rot_dims=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
             "rot": {"base": base, "dims": rot_dims or rot_dim}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _retention(heads, dim, vdim, decay, rot, mlp):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        mixer["rot"] = rot
    return {"type": "retention", "mixer": mixer, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, scale, ff, shared):
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


ZIPELIX = {
    "zip-A": dict(
        config={"architecture": "Zipelix", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
                "streams": 3, "logit_softcap": 8.0,
                "layers": [_latent(2, 16, 8, 24, 32, 0.2, 10000.0, _dense(96)),
                           _retention(3, 16, 8, [0.9, 0.97, 1.0], {"base": 1000.0, "dims": 8}, _moe(5, 2, 1.7, 40, 24)),
                           _latent(4, 8, 8, 12, 32, 0.3, 10000.0, _moe(4, 1, 0.6, 56, None), kv_from=0),
                           _retention(2, 24, 40, [0.5, 0.99], {"base": 50.0, "dims": 24}, None),
                           _latent(3, 24, 8, 8, 32, 0.15, 10000.0, _dense(72), kv_from=0)]},
        seed=1, page_size=8, sharpen=2.0),
    "zip-B": dict(
        config={"architecture": "Zipelix", "vocab": 131, "width": 96, "norm": {"eps": 3e-6}, "initializer_range": 0.06,
                "streams": 2,
                "layers": [_retention(1, 32, 32, [0.96], None, _dense(120)),
                           _latent(1, 32, 16, 16, 48, 0.18, 2000.0, None, rot_dims=12),
                           _latent(5, 8, 16, 24, 48, 0.22, 2000.0, _moe(9, 9, 1.0, 24, 64), rot_dims=12, kv_from=1),
                           _retention(4, 10, 6, [0.8, 0.9, 0.95, 0.999], {"base": 300.0, "dims": 6}, _moe(2, 2, 2.5, 48, None))]},
        seed=2, page_size=4, sharpen=2.5),
    "zip-C": dict(          # one stream with learned coefficients; two sources of latents
        config={"architecture": "Zipelix", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "initializer_range": 0.05,
                "streams": 1, "logit_softcap": 30.0,
                "layers": [_latent(4, 64, 32, 48, 96, 0.1, 25000.0, _dense(192)),
                           _latent(2, 32, 64, 64, 160, 0.12, 1e6, _moe(6, 3, 1.2, 64, 32)),
                           _retention(2, 64, 64, [0.98, 0.995], {"base": 1e6, "dims": 64}, _dense(160)),
                           _latent(4, 16, 64, 16, 160, 0.12, 1e6, _dense(64), kv_from=1),
                           _latent(8, 32, 32, 16, 96, 0.125, 25000.0, _moe(7, 2, 1.0, 40, 80), kv_from=0)]},
        seed=3, page_size=16, sharpen=1.5),
    "zip-D": dict(          # no hyper-connections: plain residual sums; no cap
        config={"architecture": "Zipelix", "vocab": 157, "width": 80, "norm": {"eps": 2e-5}, "initializer_range": 0.07,
                "layers": [_latent(4, 24, 16, 40, 56, 0.15, 1000.0, _moe(3, 2, 1.5, 100, 36)),
                           _retention(2, 20, 28, [0.9375, 1.0], {"base": 1000.0, "dims": 10}, _dense(100)),
                           _latent(4, 24, 16, 40, 56, 0.15, 1000.0, None, kv_from=0)]},
        seed=4, page_size=16, sharpen=1.5),
    "zip-E": dict(          # retention alone: the engine runs without a page pool, on state slots alone; five streams
        config={"architecture": "Zipelix", "vocab": 83, "width": 56, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
                "streams": 5, "logit_softcap": 4.0,
                "layers": [_retention(2, 12, 20, [0.7, 0.98], {"base": 100.0, "dims": 12}, _dense(72)),
                           _retention(3, 36, 4, [0.99, 0.9, 0.999], {"base": 10000.0, "dims": 2}, _moe(4, 3, 0.8, 32, 16))]},
        seed=5, page_size=8, sharpen=1.0),
}


def random_configuration(seed: int) -> dict:
    """A configuration drawn at random: 2 to 6 layers of both kinds in any order, sizes that are and are not multiples
    of 4, 8 or 16, every optional key present or absent; latent layers read an earlier layer's cache half of the time."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 96, 128, 144])
    if seed % 3 == 0:
        width = rng.choice([50, 66, 100, 257])          # rows that no 16-byte access fits
    layers, sources = [], []
    for i in range(rng.randint(2, 6)):
        roll = rng.random()
        if roll < 0.25:
            mlp = None
        elif roll < 0.55:
            mlp = _dense(rng.choice([40, 96, 100, 200]))
        else:
            experts = rng.choice([2, 3, 5, 8, 12])
            mlp = _moe(experts, rng.randint(1, min(experts, 4)), rng.choice([0.5, 1.0, 2.0]), rng.choice([24, 40, 50, 96]),
                       rng.choice([None, 16, 72]))
        if rng.random() < 0.6:
            if sources and rng.random() < 0.5:
                j = rng.choice(sources)
                src = layers[j]["mixer"]
                layers.append(_latent(rng.choice([1, 2, 3, 4, 6]), rng.choice([8, 16, 24, 40]), src["rot_dim"], rng.choice([8, 16, 40]),
                                      src["kv_rank"], rng.uniform(0.1, 0.3), src["rot"]["base"], mlp,
                                      rot_dims=src["rot"]["dims"], kv_from=j))
            else:
                rot_dim = rng.choice([4, 8, 16, 32])
                layers.append(_latent(rng.choice([1, 2, 3, 4, 5]), rng.choice([8, 16, 24, 64]), rot_dim, rng.choice([8, 16, 40]),
                                      rng.choice([16, 32, 48, 64, 96, 128]), rng.uniform(0.1, 0.3),
                                      rng.choice([100.0, 10000.0, 500000.0]), mlp,
                                      rot_dims=rng.choice([d for d in (2, 4, 8, rot_dim) if d <= rot_dim])))
                sources.append(i)
        else:
            heads, dim = rng.choice([1, 2, 3, 5]), rng.choice([6, 8, 16, 30, 32, 64])
            rot = None
            if rng.random() < 0.8:
                rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": rng.choice([d for d in (2, 4, 6, 8, 16, dim) if d <= dim and d % 2 == 0])}
            layers.append(_retention(heads, dim, rng.choice([4, 8, 18, 32, 64]),
                                     [rng.choice([1.0, 0.999, 0.98, 0.9, 0.6]) for _ in range(heads)], rot, mlp))
    config = {"architecture": "Zipelix", "vocab": rng.choice([61, 128, 250]), "width": width,
              "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-5])}, "initializer_range": 0.07, "layers": layers}
    if rng.random() < 0.8:
        config["streams"] = rng.choice([1, 2, 3, 4, 6, 8])
    if rng.random() < 0.6:
        config["logit_softcap"] = rng.choice([5.0, 15.0, 50.0])
    return config


def make_model(folder: str, name: str) -> dict:
    """The folder through the package's random-weights mode; then the weights are moved to where a fault shows: the
    matrices that make queries and keys are scaled up (peaked attention weights: a wrong, missing or extra key changes
    the output), norm weights are spread, the hyper-connection coefficients leave 1 and the identity far behind (every
    entry of `mix` matters, `mix` is far from symmetric: a transposed index shows), the routers are scaled up (the
    scores differ between experts: a wrong choice or weight shows), the shared expert's gate is spread.
    Returns {dir, config, weights (by checkpoint name, as stored), page_size, name}."""
    from safetensors.torch import load_file, save_file

    from lia_rs_b200.config import ZipelixConfig
    from lia_rs_b200.weights import write_random_model
    if name in ZIPELIX:
        entry = ZIPELIX[name]
    else:
        seed = int(name.split("-")[1])
        entry = dict(config=random_configuration(seed), seed=seed, page_size=(4, 8, 16)[seed % 3], sharpen=2.0)
    write_random_model(ZipelixConfig.from_dict(entry["config"]), folder, seed=entry["seed"])
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    g = torch.Generator().manual_seed(entry["seed"] + 100)
    bf16 = lambda t: t.to(torch.bfloat16)
    for key in list(weights):
        shape = weights[key].shape
        tail = key.split(".", 1)[1] if "." in key else key
        if tail in ("mix.q", "mix.k", "mix.uk", "mix.dkv"):
            weights[key] = bf16(weights[key].float() * entry["sharpen"])
        elif tail == "mix.dkv.norm":
            weights[key] = bf16(1.0 + 0.3 * torch.randn(shape, generator=g))
        elif "norm" in key:
            weights[key] = bf16(1.0 + 0.3 * torch.randn(shape, generator=g))
        elif tail.endswith(".in"):
            weights[key] = bf16((0.4 + 0.8 * torch.rand(shape, generator=g)) / shape[0] ** 0.5)
        elif tail.endswith(".out"):
            weights[key] = bf16(0.5 + torch.rand(shape, generator=g))
        elif tail.endswith(".mix") and tail.startswith("hc"):
            weights[key] = bf16(0.8 * torch.eye(shape[0]) + 0.35 * torch.randn(shape, generator=g) / shape[0] ** 0.5)
        elif tail == "mlp.router":
            weights[key] = bf16(weights[key].float() * 6.0)
        elif tail == "mlp.shared.sg":
            weights[key] = bf16(weights[key].float() * 4.0)
    save_file(weights, path)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return dict(dir=folder, config=config, weights=weights, page_size=entry["page_size"], name=name)


_CACHE = {}
_MARKS = {}       # storage of a cached reference -> per row 0 (sound), 1 (behind a fragile row of its sequence), 2 (fragile)


def plain_logits(model: dict, tokens) -> torch.Tensor:
    key = (model["name"], model["dir"], tuple(tokens))
    if key not in _CACHE:
        fragile = torch.zeros(len(tokens), dtype=torch.bool)
        logits = plain_zipelix.forward(model["config"], model["weights"], list(tokens), fragile=fragile).contiguous()
        behind = (torch.cumsum(fragile.long(), 0) - fragile.long()) > 0
        _MARKS[logits.untyped_storage().data_ptr()] = torch.where(fragile, 2, behind.long())
        _CACHE[key] = logits
    return _CACHE[key]


def marks_of(reference: torch.Tensor):
    """The marks of the rows of a cached reference or of a slice of rows of one (a view of it), else None."""
    marks = _MARKS.get(reference.untyped_storage().data_ptr())
    if marks is None or reference.dim() != 2 or reference.stride(1) != 1:
        return None
    first = reference.storage_offset() // reference.stride(0)
    return marks[first:first + reference.shape[0]]


def longest_sum(config: dict) -> int:
    sizes = [config["width"]]
    for layer in config["layers"]:
        m = layer["mixer"]
        sizes.append(m["heads"] * max(m["dim"] + m.get("rot_dim", 0), m["vdim"], m.get("kv_rank", 0)))
        mlp = layer.get("mlp")
        if mlp:
            sizes.append(mlp["ff"] if mlp["kind"] == "dense" else max(mlp["expert"]["ff"], (mlp.get("shared") or {}).get("ff", 0)))
    return max(sizes)


def assert_close(actual, reference, dtype: str, what: str, config: dict):
    """Against the exact (64-bit) model.  32-bit: every logit within 8 K 2^-24 of the largest logit per layer that the
    sums pass through (K the model's longest sum; a retention layer's sums run along the sequence and count as four).
    bfloat16: every row's root-mean-square error within 2.5e-2 of the largest logit, times the root of the number of
    layers over 3 (rounding noise of a layer adds to that of the layers before), and no single logit further off than
    three times that.  A row that the plain implementation marks as resting on a close call (a router's choice between
    two experts of nearly equal score, a retention head whose output direction is a cancellation) may come out on the
    other side in 16-bit arithmetic: it only has to be finite, and the rows behind it in its sequence, which read what it
    cached, get four times the limit."""
    marks = marks_of(reference) if dtype != "float32" else None
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    reference = reference.to(torch.float64)
    assert actual.shape == reference.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(reference.shape)}"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    layers = len(config["layers"])
    weighted = layers + 3 * sum(1 for layer in config["layers"] if layer["type"] == "retention")
    scale = max(1.0, float(reference.abs().max()))
    error = (actual - reference).abs()
    if dtype == "float32":
        limit = 8.0 * longest_sum(config) * 2.0 ** -24 * scale * weighted
        worst = float(error.max())
    else:
        limit = 2.5e-2 * scale * max(1.0, (weighted / 3.0) ** 0.5)
        if marks is not None and error.dim() == 2:
            error = error * torch.tensor([1.0, 0.25, 0.0], dtype=torch.float64)[marks][:, None]
        worst = max(float((error ** 2).mean(dim=-1).sqrt().max()), float(error.max()) / 3.0)
    if worst > limit:
        row = int(error.max(dim=-1).values.argmax()) if error.dim() > 1 else 0
        raise AssertionError(f"{what}: error {worst:.3e} > {limit:.3e} (largest at wanted row {row})")
