"""Tiny Pilutar configurations for the tests, their model folders with random weights, and the comparison with the
plain implementation (tests/plain_pilutar.py).

The configurations differ in everything that config.json gives: widths and vocabularies; the order of the two kinds of
layer (each first, last and alone); latent attention with 1 to 5 heads, ranks smaller and larger than a head, rotated
parts of which all or only the first dimensions turn, windows of 1 token, of a few and of more than any test's length,
and none; side-by-side mixers whose attention has as many key heads as query heads, fewer, and one, key and value sizes
equal and unequal, partial, full and absent rotation, a cap present and absent, windows that do and do not divide the
page, and whose recurrence has 1 to 4 heads, key and value sizes that are not multiples of four, tau of 1 and larger,
decay ranks from 1 on; weights of the two sides other than 1, one of them negative; dense feed-forwards, mixtures with
1 to 9 experts, 0 to 4 identity outputs, 1 to all outputs chosen, groups present and absent with 1 to all kept, with and
without a shared expert, and layers without a feed-forward; factors on the embedding and the logits present and absent."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_pilutar


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, window, mlp, rot_dims=None, rot=True):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot:
        mixer["rot"] = {"base": base, "dims": rot_dims or rot_dim}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _left(heads, kv_heads, dim, vdim, scale, window=None, softcap=None, rot=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        left["mask"] = {"size": window}
    if softcap:
        left["softcap"] = softcap
    if rot:
        left["rot"] = rot
    return left


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, shared=None, identity=0, groups=None):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


PILUTAR = {
    "pil-A": dict(
        config={"architecture": "Pilutar", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
                "embedding": {"scale": 6.0}, "logit_scale": 0.5,
                "layers": [
                    _parallel(_left(4, 2, 16, 24, 0.25, window=11, softcap=5.0, rot={"base": 1000.0, "dims": 8}),
                              _right(2, 12, 20, 4.0, 6), 0.7, 0.4, _dense(96)),
                    _latent(3, 16, 8, 12, 32, 0.2, 10000.0, 7, _moe(5, 2, 40, shared=24, identity=1, groups=(3, 2))),
                    _parallel(_left(3, 3, 8, 8, 0.3, window=33, softcap=20.0, rot={"base": 50.0, "dims": 8}),
                              _right(3, 8, 8, 1.0, 1), 1.0, -0.5, _moe(4, 3, 56)),
                    _latent(2, 24, 8, 8, 16, 0.15, 500.0, 40, None, rot_dims=4)]},
        seed=1, page_size=8, sharpen=2.0),
    "pil-B": dict(          # no factors, no windows in two layers, no cap, nothing turns in one mixer
        config={"architecture": "Pilutar", "vocab": 131, "width": 96, "norm": {"eps": 3e-6}, "initializer_range": 0.06,
                "layers": [
                    _latent(1, 32, 16, 16, 48, 0.18, 2000.0, None, _dense(120), rot_dims=12),
                    _parallel(_left(6, 1, 16, 12, 0.2, rot={"base": 300.0, "dims": 16}), _right(1, 32, 32, 16.0, 3), 0.5, 0.5,
                              _moe(9, 9, 24, shared=64, identity=3, groups=(4, 4))),
                    _parallel(_left(2, 2, 24, 40, 0.2, window=1), _right(4, 10, 6, 2.0, 5), 0.6, 0.9,
                              _moe(2, 1, 48, identity=2, groups=(2, 1))),
                    _latent(5, 8, 16, 24, 48, 0.22, 2000.0, 1, _moe(1, 1, 24, shared=16), rot=False)]},
        seed=2, page_size=4, sharpen=2.5),
    "pil-C": dict(          # side-by-side mixers alone; sizes of real shapes' divisibility (multiples of 16 and 32)
        config={"architecture": "Pilutar", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "initializer_range": 0.05,
                "embedding": {"scale": 11.0}, "logit_scale": 0.3,
                "layers": [
                    _parallel(_left(4, 1, 64, 64, 0.125, window=48, softcap=30.0, rot={"base": 25000.0, "dims": 32}),
                              _right(2, 64, 64, 8.0, 16), 0.6, 0.5, _dense(192)),
                    _parallel(_left(8, 4, 32, 32, 0.17, window=20, softcap=10.0, rot={"base": 1e6, "dims": 32}),
                              _right(4, 32, 48, 16.0, 8), 0.8, 0.3, _moe(8, 4, 64, shared=96, identity=4, groups=(4, 2)))]},
        seed=3, page_size=16, sharpen=1.5),
    "pil-D": dict(          # latent attention alone: no recurrent state anywhere
        config={"architecture": "Pilutar", "vocab": 157, "width": 80, "norm": {"eps": 2e-5}, "initializer_range": 0.07,
                "logit_scale": 2.0,
                "layers": [
                    _latent(4, 24, 16, 40, 56, 0.15, 1000.0, 19, _moe(3, 2, 100, shared=36)),
                    _latent(2, 64, 32, 48, 96, 0.1, 25000.0, 64, _dense(100)),
                    _latent(4, 24, 16, 40, 56, 0.15, 1000.0, 5, None)]},
        seed=4, page_size=16, sharpen=1.5),
}


def random_configuration(seed: int) -> dict:
    """A configuration drawn at random: 2 to 5 layers of both kinds in any order, sizes that are and are not multiples
    of 4, 8 or 16, every optional key present or absent."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 96, 128, 144])
    if seed % 3 == 0:
        width = rng.choice([50, 66, 100, 257])          # rows that no 16-byte access fits
    layers = []
    for _ in range(rng.randint(2, 5)):
        roll = rng.random()
        if roll < 0.2:
            mlp = None
        elif roll < 0.45:
            mlp = _dense(rng.choice([40, 96, 100, 200]))
        else:
            experts, identity = rng.choice([1, 2, 3, 5, 8, 12]), rng.choice([0, 0, 1, 2, 4])
            outputs = experts + identity
            groups = None
            if rng.random() < 0.6:
                count = rng.choice([c for c in (1, 2, 3, 4, 5, 6) if outputs % c == 0])
                groups = (count, rng.randint(1, count))
            most = min(outputs if not groups else groups[1] * (outputs // groups[0]), 4)
            mlp = _moe(experts, rng.randint(1, most), rng.choice([24, 40, 50, 96]), shared=rng.choice([None, 16, 72]),
                       identity=identity, groups=groups)
        window = rng.choice([None, 1, 3, 8, 17, 32, 50, 200])
        if rng.random() < 0.4:
            rot_dim = rng.choice([4, 8, 16, 32])
            layers.append(_latent(rng.choice([1, 2, 3, 4, 5]), rng.choice([8, 16, 24, 64]), rot_dim, rng.choice([8, 16, 40]),
                                  rng.choice([16, 32, 48, 64, 96, 128]), rng.uniform(0.1, 0.3),
                                  rng.choice([100.0, 10000.0, 500000.0]), window, mlp,
                                  rot_dims=rng.choice([d for d in (2, 4, 8, rot_dim) if d <= rot_dim]), rot=rng.random() < 0.85))
        else:
            kv_heads = rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 40, 64])
            rot = None
            if rng.random() < 0.8:
                rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": rng.choice([d for d in (2, 4, 8, 16, dim) if d <= dim])}
            left = _left(kv_heads * rng.choice([1, 2, 4]), kv_heads, dim, rng.choice([8, 16, 24, 40, dim]), rng.uniform(0.1, 0.3),
                         window=window, softcap=rng.choice([None, 3.0, 15.0, 50.0]), rot=rot)
            right = _right(rng.choice([1, 2, 3, 5]), rng.choice([6, 8, 16, 30, 32, 64]), rng.choice([4, 8, 18, 32, 64]),
                           rng.choice([1.0, 2.0, 8.0, 16.0]), rng.choice([1, 2, 4, 7, 16]))
            layers.append(_parallel(left, right, rng.choice([1.0, 0.6, 0.3]), rng.choice([1.0, 0.5, -0.7]), mlp))
    config = {"architecture": "Pilutar", "vocab": rng.choice([61, 128, 250]), "width": width,
              "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-5])}, "initializer_range": 0.07, "layers": layers}
    if rng.random() < 0.7:
        config["embedding"] = {"scale": rng.choice([1.0, 4.0, 12.0])}
    if rng.random() < 0.7:
        config["logit_scale"] = rng.choice([0.25, 1.0, 3.0])
    return config


def make_model(folder: str, name: str) -> dict:
    """The folder through the package's random-weights mode; then the weights are moved to where a fault shows: the
    matrices that make queries and keys are scaled up (peaked attention weights: a wrong, missing or extra key changes
    the output), norm weights and every bias are spread, the decay's bias is spread widely (channels that forget within
    a few tokens beside channels that keep hundreds), the routers are scaled up and the corrections spread around zero
    with both signs (the scores differ between outputs: a wrong choice, group or weight shows), the shared expert's gate
    is spread.  Returns {dir, config, weights (by checkpoint name, as stored), page_size, name}."""
    from safetensors.torch import load_file, save_file

    from lia_rs_b200.config import PilutarConfig
    from lia_rs_b200.weights import write_random_model
    if name in PILUTAR:
        entry = PILUTAR[name]
    else:
        seed = int(name.split("-")[1])
        entry = dict(config=random_configuration(seed), seed=seed, page_size=(4, 8, 16)[seed % 3], sharpen=2.0)
    write_random_model(PilutarConfig.from_dict(entry["config"]), folder, seed=entry["seed"])
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    g = torch.Generator().manual_seed(entry["seed"] + 100)
    bf16 = lambda t: t.to(torch.bfloat16)
    for key in list(weights):
        shape = weights[key].shape
        tail = key.split(".", 1)[1] if "." in key else key
        if tail in ("mix.q", "mix.uk", "mix.dkv", "mix.left.q", "mix.left.k", "mix.right.q", "mix.right.k"):
            weights[key] = bf16(weights[key].float() * entry["sharpen"])
        elif tail == "mix.right.a2.b":
            weights[key] = bf16(1.0 + 3.0 * torch.randn(shape, generator=g))
        elif tail in ("mix.right.a1", "mix.right.a2"):
            weights[key] = bf16(weights[key].float() * 4.0)
        elif tail.endswith(".b"):
            weights[key] = bf16(0.3 * torch.randn(shape, generator=g))
        elif "norm" in key:
            weights[key] = bf16(1.0 + 0.3 * torch.randn(shape, generator=g))
        elif tail == "mlp.router":
            weights[key] = bf16(weights[key].float() * 6.0)
        elif tail == "mlp.correction":
            weights[key] = bf16(0.15 * torch.randn(shape, generator=g))
        elif tail in ("mlp.shared.sg", "mix.g"):
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
        logits = plain_pilutar.forward(model["config"], model["weights"], list(tokens), fragile=fragile).contiguous()
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
        for part in ([m] if layer["type"] == "latent_attention" else [m["left"], m["right"]]):
            sizes.append(part["heads"] * max(part["dim"] + part.get("rot_dim", 0), part["vdim"], part.get("kv_rank", 0)))
        mlp = layer.get("mlp")
        if mlp:
            sizes.append(mlp["ff"] if mlp["kind"] == "dense" else max(mlp["expert"]["ff"], (mlp.get("shared") or {}).get("ff", 0)))
    return max(sizes)


def assert_close(actual, reference, dtype: str, what: str, config: dict):
    """Against the exact (64-bit) model.  32-bit: every logit within 8 K 2^-24 of the largest logit per layer that the
    sums pass through (K the model's longest sum; a layer with a recurrence, whose sums run along the sequence, counts
    as four).  bfloat16: every row's root-mean-square error within 2.5e-2 of the largest logit, times the root of the
    number of layers over 3 (rounding noise of a layer adds to that of the layers before), and no single logit further
    off than three times that.  A row that the plain implementation marks as resting on a close call (a router's choice
    between two outputs or two groups of nearly equal score) may come out on the other side in 16-bit arithmetic: it
    only has to be finite, and the rows behind it in its sequence, which read what it cached, get four times the limit."""
    marks = marks_of(reference) if dtype != "float32" else None
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    reference = reference.to(torch.float64)
    assert actual.shape == reference.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(reference.shape)}"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    layers = len(config["layers"])
    weighted = layers + 3 * sum(1 for layer in config["layers"] if layer["type"] == "parallel")
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
