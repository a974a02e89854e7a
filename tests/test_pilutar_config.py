"""The Pilutar configuration, its registration and the model description that is built from it, on the CPU: the round
trip through `to_dict`, refusals with the key's path, the parts chosen layer by layer with their parameters, the tensor
names and shapes, caches and states, a size that only the stored tensor gives, and random weights through the loader."""
import copy
import json
import os

import pytest
import torch

import pilutar_helpers as ph
from lia_rs_b200.config import ConfigError, PilutarConfig, known_architectures, resolve_architecture
from lia_rs_b200.parts import KVCacheRequest

NAMES = list(ph.PILUTAR)


def raw_config(name):
    return copy.deepcopy(ph.PILUTAR[name]["config"])


@pytest.mark.parametrize("name", NAMES + ["random-7", "random-9"])
def test_round_trip_and_registry(name):
    raw = raw_config(name) if name in ph.PILUTAR else ph.random_configuration(int(name.split("-")[1]))
    config = PilutarConfig.from_dict(raw)
    again = PilutarConfig.from_dict(config.to_dict())
    assert again == config and again.layers == config.layers
    assert "Pilutar" in known_architectures() and resolve_architecture(raw).config_class is PilutarConfig
    assert config.embedding_scale == (raw.get("embedding") or {}).get("scale", 1.0) and config.logit_scale == raw.get("logit_scale", 1.0)


def test_refusals_name_the_key():
    good = raw_config("pil-A")

    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        return raw
    cases = [
        (lambda r: r["layers"][0].update(type="retention"), r"layers\[0\].type"),
        (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=7), r"left.rot.dims"),
        (lambda r: r["layers"][0]["mixer"]["left"]["mask"].update(size=0), r"left.mask.size"),
        (lambda r: r["layers"][0]["mixer"]["right"].update(tau=0.0), r"right.tau"),
        (lambda r: r["layers"][0]["mixer"].pop("right"), "'right'"),
        (lambda r: r["layers"][1]["mixer"].update(kv_rank=0), "kv_rank"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=10), r"rot.dims"),
        (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "router.top"),
        (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4), "groups"),
        (lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=1, count=6), "groups"),
        (lambda r: r["layers"][1]["mlp"]["router"].update(identity=-1), "identity"),
        (lambda r: r["layers"][1]["mlp"].update(kind="glu"), "kind"),
        (lambda r: r.pop("width"), "width"),
        (lambda r: r["norm"].pop("eps"), "norm.eps"),
        (lambda r: r.update(layers=[]), "non-empty"),
    ]
    for change, words in cases:
        with pytest.raises(ConfigError, match=words):
            PilutarConfig.from_dict(broken(change))
    # sizes beyond the kernels are refused when the model is described, before any tensor is read
    architecture = resolve_architecture(good)
    for change, words in [(lambda r: r["layers"][0]["mixer"]["right"].update(dim=300), "head_dim"),
                          (lambda r: r["layers"][1]["mixer"].update(kv_rank=600), "kv_rank"),
                          (lambda r: r["layers"][2]["mlp"]["router"].update(experts=2000, identity=0), "expert")]:
        with pytest.raises(ValueError, match=words):
            architecture.build(PilutarConfig.from_dict(broken(change)))


@pytest.mark.parametrize("name", NAMES)
def test_model_description(name):
    raw = raw_config(name)
    config = PilutarConfig.from_dict(raw)
    spec = resolve_architecture(raw).build(config)
    assert spec.max_positions is None and spec.position_table_name is None and spec.head_name == "head"
    assert spec.streams == 1 and spec.logit_softcap is None
    assert spec.embedding_scale == config.embedding_scale and spec.logit_scale == config.logit_scale
    kinds = {"latent_attention": "latent_attention", "parallel": "side_by_side"}
    assert [l.mixer.kind for l in spec.layers] == [kinds[l["type"]] for l in raw["layers"]]
    assert all(l.arrangement == "parallel" and l.norm.kind == "layernorm" for l in spec.layers)
    names = {s.name: tuple(s.shape) for s in spec.tensor_specs() if not s.optional}
    width = raw["width"]
    assert names["embed"] == (raw["vocab"], width) == names["head"]
    assert names["final.norm"] == (width,) == names["final.norm.b"]
    caches, states = spec.cache_requests(), spec.state_requests()
    for i, layer in enumerate(raw["layers"]):
        m, mlp, p = layer["mixer"], layer["mlp"], f"l{i}."
        assert names[p + "norm1"] == (width,) == names[p + "norm1.b"] and p + "norm2" not in names
        if layer["type"] == "latent_attention":
            H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            assert names[p + "mix.q"] == (H * (d + dr), width) and names[p + "mix.g"] == (H, width)
            assert names[p + "mix.uk"] == (H * d, rank) and names[p + "mix.uv"] == (H * dv, rank) and names[p + "mix.o"] == (width, H * dv)
            assert names[p + "mix.dkv"] == (rank + dr, width) and names[p + "mix.dkv.norm"] == (rank,)
            window = m["mask"]["size"] if m.get("mask") else None
            assert caches[i] == KVCacheRequest(1, rank, window, v_head_dim=dr) and i not in states
            assert spec.layers[i].mixer.params["rot_pairs"] and spec.layers[i].mixer.params["gate"] == "sigmoid_head"
        else:
            left, right = m["left"], m["right"]
            H, G, d, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            assert names[p + "mix.left.q"] == (H * d, width) and names[p + "mix.left.q.b"] == (H * d,) == names[p + "mix.left.q.norm"]
            assert names[p + "mix.left.k"] == (G * d, width) and names[p + "mix.left.k.b"] == (G * d,) == names[p + "mix.left.k.norm"]
            assert names[p + "mix.left.v"] == (G * dv, width) and names[p + "mix.left.v.b"] == (G * dv,)
            assert names[p + "mix.left.o"] == (width, H * dv) and p + "mix.left.o.b" not in names
            window = left["mask"]["size"] if left.get("mask") else None
            assert caches[i] == KVCacheRequest(G, d, window, v_head_dim=dv)
            H, d, dv, rank = right["heads"], right["dim"], right["vdim"], right["rank"]
            assert names[p + "mix.right.q"] == (H * d, width) == names[p + "mix.right.k"]
            assert names[p + "mix.right.v"] == (H * dv, width) == names[p + "mix.right.g"] and names[p + "mix.right.o"] == (width, H * dv)
            assert names[p + "mix.right.norm"] == (dv,) and names[p + "mix.right.a1"] == (rank, width)
            assert names[p + "mix.right.a2"] == (H * d, rank) and names[p + "mix.right.a2.b"] == (H * d,)
            assert states[i].shape == (H, d, dv) and states[i].dtype == torch.float32
            members = spec.layers[i].mixer.params["members"]
            assert [x["scale"] for x in members] == [m["left_scale"], m["right_scale"]]
        if mlp is None:
            assert spec.layers[i].feed_forward is None
        elif mlp["kind"] == "dense":
            assert names[p + "mlp.gate"] == (mlp["ff"], width) == names[p + "mlp.up"] and names[p + "mlp.down"] == (width, mlp["ff"])
            assert spec.layers[i].feed_forward.params["gate_activation"] == "relu"
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            outputs = E + mlp["router"].get("identity", 0)
            assert names[p + "mlp.router"] == (outputs, width) and names[p + "mlp.correction"] == (outputs,)
            assert p + f"mlp.e{E}.up" not in names and p + "mlp.e0.gate" not in names
            assert all(names[p + f"mlp.e{e}.up"] == (ff, width) and names[p + f"mlp.e{e}.down"] == (width, ff) for e in range(E))
            assert (p + "mlp.shared.sg" in names) == bool(mlp.get("shared"))
            if mlp.get("shared"):
                assert names[p + "mlp.shared.sg"] == (1, width) and names[p + "mlp.shared.up"] == (mlp["shared"]["ff"], width)
                assert p + "mlp.shared.gate" not in names


def test_a_size_that_only_the_stored_tensor_gives(tmp_path):
    """Without `right.rank` the description leaves the decay product's rank open: any stored rank loads, the two
    matrices must agree when the part is built, and the random-weights mode asks for the key."""
    from lia_rs_b200.weights import adopt_tensors, random_weights
    raw = raw_config("pil-A")
    weights = random_weights(PilutarConfig.from_dict(raw), seed=3)
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["right"].pop("rank")
    config = PilutarConfig.from_dict(raw)
    spec = resolve_architecture(raw).build(config)
    shapes = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    assert shapes["l0.mix.right.a1"] == (None, raw["width"]) and shapes["l0.mix.right.a2"][1] is None
    adopted = adopt_tensors(weights, spec.tensor_specs())
    assert adopted["l0.mix.right.a1"].shape[0] == 6 and adopted["l2.mix.right.a1"].shape[0] == 1
    with pytest.raises(ValueError, match="left to the stored tensor"):
        random_weights(config, seed=3)


@pytest.mark.parametrize("name", ["pil-A", "pil-B"])
def test_random_weights_pass_the_loader(tmp_path, name):
    from lia_rs_b200.weights import load_weights, write_random_model
    raw = raw_config(name)
    config = PilutarConfig.from_dict(raw)
    folder = write_random_model(config, str(tmp_path / name), seed=5)
    with open(os.path.join(folder, "config.json")) as f:
        assert PilutarConfig.from_dict(json.load(f)) == config
    spec = resolve_architecture(raw).build(config)
    tensors = load_weights(folder, spec.tensor_specs())
    assert set(tensors) == {s.name for s in spec.tensor_specs() if not s.optional}
    assert float(tensors["l0.norm1"].float().min()) == 1.0 and float(tensors["final.norm.b"].float().abs().max()) > 0
