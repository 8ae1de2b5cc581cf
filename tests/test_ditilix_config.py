"""The Ditilix configuration: reading, refusing, the plan it makes (which layer owns a cache
and which reads another's); the tensors a model folder must hold; the plain implementation's
own mechanisms against closed forms.  No device."""

import copy
import math

import pytest
import torch

import ditilix_tiny as tiny
from plain import ditilix_plain as plain
from thing_htn_2026_b200.config import ConfigError, config_from_dict, known_architectures
from thing_htn_2026_b200.config.ditilix import DitilixConfig
from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
from thing_htn_2026_b200.weights.loader import merge_specs


def test_architecture_is_registered_and_chosen_by_its_key():
    assert "Ditilix" in known_architectures()
    config = config_from_dict(tiny.config_json("a"))
    assert isinstance(config, DitilixConfig)
    assert config.to_dict()["layers"][2]["mixer"]["kv_from"] == 1
    assert config_from_dict(config.to_dict()) == config


@pytest.mark.parametrize("name", sorted(tiny.CONFIGS))
def test_plan_follows_the_layer_list(name):
    data = tiny.config_json(name)
    plan = config_from_dict(data).plan()
    assert len(plan.schedule) == len(plan.layers) == len(data["layers"])
    owners = [i for i, layer in enumerate(data["layers"]) if layer["mixer"].get("kv_from") is None]
    for i, (entry, layer) in enumerate(zip(plan.schedule, data["layers"])):
        source = layer["mixer"].get("kv_from")
        assert entry.layer == i
        assert entry.writes_cache == (source is None)
        assert entry.cache == owners.index(i if source is None else source)
        block = plan.layers[i].block
        assert block.kind == "parallel"
        assert block.params["mixer"].kind == "attention"
        assert block.params["mixer"].params["kv"] == ("own" if source is None else "shared")
        assert ("ffn" in block.params) == (layer["mlp"] is not None)
        if layer["mlp"] is not None:
            assert block.params["ffn"].kind == {"dense": "polynorm", "moe": "routed_clamped_experts"}[layer["mlp"]["kind"]]


def test_every_size_and_constant_of_the_file_reaches_a_part():
    data = tiny.config_json("a")
    plan = config_from_dict(data).plan()
    block = plan.layers[2].block.params
    assert block["factor"] == 0.5
    attn = block["mixer"].params
    assert (attn["n_heads"], attn["n_kv_heads"], attn["head_dim"], attn["value_dim"]) == (4, 2, 64, 64)
    assert (attn["scale"], attn["softcap"], attn["q_temp"]) == (0.25, 9.0, {"coef": 0.3, "every": 16})
    assert attn["position"] is None and attn["window"] is None
    norm = block["norm"].params
    assert (norm["eps"], norm["groups"], norm["residual"]) == (1e-5, 3, "float32")
    ffn = block["ffn"].params
    assert (ffn["n_experts"], ffn["top"], ffn["expert_ff"], ffn["limit"]) == (6, 2, 24, 1.5)
    assert (ffn["shared_ff"], ffn["shared_limit"], ffn["slope"]) == (40, 0.8, 1.702)
    dense = plan.layers[0].block.params["ffn"].params
    assert (dense["intermediate_size"], dense["eps"]) == (136, 1e-5)
    assert plan.head.params["scale"] == 2.0 and plan.final_norm.params["groups"] == 3
    assert plan.embedding.params["positions"] == {"kind": "sinusoid", "base": 10000.0}
    # what a file may leave out
    bare = config_from_dict(tiny.config_json("b"))
    assert bare.residual_mult == 1.0 and bare.logit_scale == 1.0 and bare.norm_groups == 1
    free = bare.plan().layers[2].block.params["mixer"].params
    assert free["softcap"] is None and free["q_temp"] == {"coef": 0.6, "every": 70}
    assert bare.plan().layers[0].block.params["ffn"].params["shared_ff"] == 0


def test_tensor_names_and_shapes():
    specs = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("c")).plan()))
    shapes = {name: tuple(s.shape) for name, s in specs.items()}
    assert shapes["embed"] == (333, 100) and shapes["head"] == (333, 100) and shapes["final.norm"] == (100,)
    assert shapes["l0.norm1"] == (100,)
    assert shapes["l0.mix.q"] == (27, 100) and shapes["l0.mix.k"] == (9, 100) and shapes["l0.mix.v"] == (5, 100)
    assert shapes["l0.mix.o"] == (100, 15)
    assert shapes["l0.mlp.router"] == (5, 100) and shapes["l0.mlp.e4.gate"] == (30, 100) and shapes["l0.mlp.e0.down"] == (100, 30)
    assert shapes["l0.mlp.shared.up"] == (50, 100) and shapes["l0.mlp.shared.sg"] == (1, 100)
    assert shapes["l1.mlp.up"] == (77, 100) and shapes["l1.mlp.down"] == (100, 77) and shapes["l1.mlp.act"] == (4,)
    assert shapes["l1.mix.q"] == (27, 100) and "l1.mix.k" not in shapes and "l1.mix.v" not in shapes
    assert shapes["l2.mix.v"] == (72, 100) and shapes["l2.mix.o"] == (100, 72)
    assert not any(name.startswith("l3.mlp") for name in shapes) and "l3.mix.k" not in shapes
    bare = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("b")).plan()))
    assert "l0.mlp.e3.up" in bare and not any("shared" in name for name in bare)


def broken(name, change):
    data = copy.deepcopy(tiny.config_json(name))
    change(data)
    return data


@pytest.mark.parametrize("change, word", [
    (lambda d: d.pop("vocab"), "vocab"),
    (lambda d: d.__setitem__("layers", []), "layers"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d["norm"].__setitem__("eps", 0), "eps"),
    (lambda d: d["norm"].__setitem__("groups", 5), "groups"),
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda d: d["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("softcap", -1.0), "softcap"),
    (lambda d: d["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0), "every"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("kv_from", 2), "earlier"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 2), "no keys of its own"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("dim", 32), "dim"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda d: d["layers"][0]["mlp"].pop("ff"), "ff"),
    (lambda d: d["layers"][1]["mlp"]["router"].__setitem__("top", 7), "top"),
    (lambda d: d["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d["layers"][1]["mlp"]["shared"].pop("ff"), "ff"),
])
def test_bad_files_are_refused_with_the_key_named(change, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(broken("a", change))


# ----------------------------------------------------------------------------- the plain implementation


def test_plain_positions_and_temperature():
    pe = plain.sinusoid(torch.tensor([0, 3, 1000]), 6, torch.float64)
    assert pe[0].tolist() == [0.0, 1.0, 0.0, 1.0, 0.0, 1.0]
    w = 10000.0 ** (-2.0 / 6)
    assert math.isclose(pe[1, 2], math.sin(3 * w), rel_tol=1e-12) and math.isclose(pe[1, 3], math.cos(3 * w), rel_tol=1e-12)
    assert math.isclose(pe[2, 0], math.sin(1000.0), rel_tol=1e-12)
    assert plain.sinusoid(torch.tensor([2]), 5, torch.float64).shape == (1, 5)       # an odd width ends on a sine
    t = plain.query_temperature(torch.arange(12), {"coef": 0.5, "every": 4}, torch.float64)
    assert t[:3].tolist() == [1.0, 1.0, 1.0]                                       # floor((p + 1) / 4) = 0 up to p = 2
    assert math.isclose(t[3], 1 + 0.5 * math.log(2)) and math.isclose(t[6], 1 + 0.5 * math.log(2))
    assert math.isclose(t[7], 1 + 0.5 * math.log(3)) and math.isclose(t[11], 1 + 0.5 * math.log(4))
    assert plain.query_temperature(torch.arange(3), None, torch.float64).tolist() == [1.0, 1.0, 1.0]


def test_plain_norms_and_activation():
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 1.0, 1.0]], dtype=torch.float64)
    y = plain.group_norm_rms(x, torch.full((6,), 2.0, dtype=torch.float64), 3, 1e-30)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[6 / r, 8 / r, 0.0, 0.0, 2.0, 2.0]], dtype=torch.float64))
    whole = plain.group_norm_rms(x, torch.ones(6, dtype=torch.float64), 1, 0.0)
    assert math.isclose(float((whole * whole).mean()), 1.0, rel_tol=1e-12)
    z = torch.tensor([[1.0, -2.0, 2.0]], dtype=torch.float64)
    out = plain.poly_norm(z, [1.0, 10.0, 100.0, 0.5], 0.0)
    n1, n2, n3 = math.sqrt(3.0), math.sqrt(11.0), math.sqrt(43.0)
    want = [1 / n1 + 10 / n2 + 100 / n3 + 0.5, -2 / n1 + 40 / n2 - 800 / n3 + 0.5, 2 / n1 + 40 / n2 + 800 / n3 + 0.5]
    assert torch.allclose(out, torch.tensor([want], dtype=torch.float64))
    s = torch.tensor([0.0, 1.0, 50.0, -50.0], dtype=torch.float64)
    assert torch.allclose(plain.capped(s, 2.0), 2.0 * torch.tanh(s / 2.0)) and plain.capped(s, None) is s


def test_plain_routing_and_experts():
    z = torch.tensor([[0.0, 2.0, -1.0, 1.0]], dtype=torch.float64)
    chosen, weights = plain.route(z, 2)
    assert chosen.tolist() == [[1, 3]]
    assert torch.allclose(weights, torch.sigmoid(torch.tensor([[2.0, 1.0]], dtype=torch.float64)))      # not renormalised
    ar = plain.Arithmetic(torch.float64)
    eye = torch.eye(2, dtype=torch.float64)
    t = {"e.gate": eye, "e.up": eye, "e.down": eye}
    n = torch.tensor([[5.0, -5.0]], dtype=torch.float64)
    out = plain.clamped_expert(n, t, "e.", 2.0, ar)
    g = torch.tensor([2.0, -5.0], dtype=torch.float64)            # the gate is cut from above only
    u = torch.tensor([2.0, -2.0], dtype=torch.float64)
    assert torch.allclose(out, (g * torch.sigmoid(1.702 * g) * (u + 1.0))[None])
    # the weight is on the input: with a limit that cuts, expert(w n) is not w expert(n)
    half = plain.clamped_expert(0.5 * n, t, "e.", 2.0, ar)
    assert not torch.allclose(half, 0.5 * out)


def test_written_folders_load_by_name(tmp_path):
    folder = tiny.write_model(str(tmp_path / "c"), "c")
    config, tensors = plain.read_model(folder)
    assert config["architecture"] == "Ditilix" and tensors["l1.mlp.act"].shape == (4,)
    assert "l1.mix.k" not in tensors and tensors["l0.mlp.shared.sg"].shape == (1, 100)
    logits = plain.model_logits(folder, tiny.tokens("c", 7, 0))
    assert logits.shape == (7, 333) and torch.isfinite(logits).all()
    streams = []
    plain.forward(config, tensors, tiny.tokens("c", 7, 0), torch.float64, streams)
    assert len(streams) == 4 and streams[0].shape == (7, 100)
