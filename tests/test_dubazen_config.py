"""The Dubazen configuration, its plan and tensor names, the cache entry that holds keys beside a
state, and the plain implementation against closed forms.  All on the CPU."""

import copy
import math

import pytest
import torch

import dubazen_tiny as tiny
from plain import dubazen_plain as plain

from thing_htn_2026_b200.cache.sequence_cache import KVSpec, StateSpec
from thing_htn_2026_b200.config import ConfigError, config_from_dict
from thing_htn_2026_b200.models.decoder import tensor_specs_of_plan
from thing_htn_2026_b200.weights.loader import TensorSpec, check_names, merge_specs, shape_fits


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_reading_and_writing_back(name):
    data = tiny.config_json(name)
    config = config_from_dict(data)
    assert config.architecture == "Dubazen"
    assert config.to_dict() == data
    assert config_from_dict(config.to_dict()) == config


def test_the_plan_names_blocks_mixers_and_their_constants():
    plan = config_from_dict(tiny.config_json("a")).plan()
    assert [layer.block.kind for layer in plan.layers] == ["hyper_connections"] * 4
    kinds = [layer.block.params["mixer"].kind for layer in plan.layers]
    assert kinds == ["linear_attention", "mixer_pair", "selective_scan", "mixer_pair"]
    pair = plan.layers[1].block.params["mixer"].params
    assert pair["left"].kind == "gated_attention" and pair["right"].kind == "linear_attention"
    assert pair["left_scale"] == 0.7 and pair["right_scale"] == 1.3
    assert pair["left"].params["sinks"] and pair["left"].params["biases"] and pair["left"].params["gate"] == "logistic"
    assert pair["left"].params["value_position"].params["rotary_dim"] == 10
    assert pair["left"].params["position"].params["rotary_dim"] == 8
    assert pair["right"].params["decay"]["kind"] == "constant" and pair["right"].params["norm_scope"] == "all"
    gla = plan.layers[0].block.params["mixer"].params
    assert gla["decay"] == {"kind": "gated", "rank": 5, "tau": 8.0} and gla["q_scale"] == 10 ** -0.5
    ffn = plan.layers[0].block.params["ffn"].params
    assert ffn["scoring"] == "softmax" and ffn["weight_at"] == "output" and ffn["renormalise"] == 1e-20
    assert ffn["slope"] == 1.702 and not ffn["shared_gated"] and ffn["shared_limit"] == 0.8
    assert plan.layers[2].block.params.get("ffn") is None
    assert plan.final_norm.params["gain"] == "scalar"
    assert [(e.layer, e.cache) for e in plan.schedule] == [(i, i) for i in range(4)]


def test_tensor_names_and_shapes():
    specs = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("a")).plan()))
    shape = {name: spec.shape for name, spec in specs.items()}
    assert shape["embed"] == (200, 48) and shape["head"] == (200, 48) and shape["final.norm"] == ()
    assert shape["l0.norm1"] == () and shape["l0.hc1.in"] == (3,) and shape["l0.hc2.mix"] == (3, 3)
    assert shape["l0.mix.a1"] == (5, 48) and shape["l0.mix.a2"] == (30, 5) and shape["l0.mix.a2.b"] == (30,)
    assert shape["l0.mix.norm"] == (12,)
    assert shape["l1.mix.left.q"] == (96, 48) and shape["l1.mix.left.q.b"] == (96,) and shape["l1.mix.left.v"] == (20, 48)
    assert shape["l1.mix.left.sink"] == (4,) and shape["l1.mix.left.g"] == (40, 48) and shape["l1.mix.left.o.b"] == (48,)
    assert shape["l1.mix.right.norm"] == (60,) and shape["l1.mix.right.v"] == (60, 48)
    assert shape["l2.mix.in"] == (112, 48) and shape["l2.mix.conv"] == (56, 4) and shape["l2.mix.x"] == (13, 56)
    assert shape["l2.mix.dt"] == (56, 3) and shape["l2.mix.A_log"] == (56, 5)
    assert "l2.hc2.in" not in shape and "l2.norm2" not in shape and "l2.mlp.router" not in shape
    assert shape["l1.mlp.e4.gate"] == (24, 48) and shape["l1.mlp.shared.down"] == (48, 40)
    assert "l3.mlp.shared.up" not in shape
    plain_stream = merge_specs(tensor_specs_of_plan(config_from_dict(tiny.config_json("b")).plan()))
    assert not any(".hc" in name for name in plain_stream)


def test_a_rank_that_only_the_checkpoint_gives():
    data = tiny.config_json("a")
    del data["layers"][0]["mixer"]["rank"]
    specs = merge_specs(tensor_specs_of_plan(config_from_dict(data).plan()))
    assert specs["l0.mix.a1"].shape == (-1, 48) and specs["l0.mix.a2"].shape == (30, -1)
    assert shape_fits((7, 48), (-1, 48)) and not shape_fits((7, 47), (-1, 48)) and not shape_fits((7,), (-1, 48))
    found = {name: spec.shape for name, spec in specs.items()}
    found["l0.mix.a1"], found["l0.mix.a2"] = (7, 48), (30, 7)
    assert check_names("x", specs, found, strict=True) == []


@pytest.mark.parametrize("change, key", [
    (lambda d: d.__setitem__("streams", 17), "streams"),
    (lambda d: d["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda d: d["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][1]["mixer"]["left"].__setitem__("vdim", 9), "vdim"),
    (lambda d: d["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 26), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"]["left"].__setitem__("mask", {"size": 8}), "mask"),
    (lambda d: d["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5]), "decay"),
    (lambda d: d["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda d: d["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda d: d["layers"][2]["mixer"].__setitem__("state", 0), "state"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 6), "top"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda d: d["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda d: d.pop("norm"), "norm"),
])
def test_what_cannot_run_is_refused_with_its_key(change, key):
    data = copy.deepcopy(tiny.config_json("a"))
    change(data)
    with pytest.raises(ConfigError) as info:
        config_from_dict(data)
    assert key in str(info.value)


def test_a_cache_entry_of_keys_beside_a_state():
    from thing_htn_2026_b200.cache.sequence_cache import SequenceCache
    needs = [(KVSpec(2, 24, None, 0, None, 10), StateSpec((3, 20, 10))), (StateSpec((56, 5)), StateSpec((4, 56), torch.bfloat16)),
             (KVSpec(2, 24, None, 0, None, 10), StateSpec((3, 20, 10)))]
    cache = SequenceCache(needs, max_tokens=256, dtype=torch.bfloat16, device="cpu", max_slots=2)
    assert cache.kv_view(0).v_dim == 10 and cache.kv_view(2).storage.data_ptr() != cache.kv_view(0).storage.data_ptr()
    assert tuple(cache.state_view(0, 0).shape) == (2, 3, 20, 10) and tuple(cache.state_view(1, 1).shape) == (2, 4, 56)
    assert cache.state_view(2, 0).data_ptr() != cache.state_view(0, 0).data_ptr()
    with pytest.raises(KeyError):
        cache.kv_view(1)
    with pytest.raises(KeyError):
        cache.state_view(0, 1)
    with pytest.raises(TypeError):
        SequenceCache([(KVSpec(1, 8), KVSpec(1, 8))], max_tokens=64, dtype=torch.float32, device="cpu")


# ----------------------------------------------------------------------------- the plain implementation against closed forms


def test_turning_values_by_their_place_and_back_leaves_the_difference():
    v = torch.randn(1, 2, 12, dtype=torch.float64)
    there = plain.rotate(v, torch.tensor([37]), 100.0, 12)
    back = plain.rotate(there, torch.tensor([40]), 100.0, 12, sign=-1.0)
    direct = plain.rotate(v, torch.tensor([-3]), 100.0, 12)
    assert torch.allclose(back, direct, atol=1e-12)
    # the pairs are (i, i + half) and pair 0 turns by the position itself
    one = torch.zeros(1, 1, 4, dtype=torch.float64)
    one[0, 0, 0] = 1.0
    turned = plain.rotate(one, torch.tensor([2]), 10000.0, 4)
    assert torch.allclose(turned[0, 0], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0], dtype=torch.float64), atol=1e-12)
    part = plain.rotate(torch.ones(1, 1, 6, dtype=torch.float64), torch.tensor([5]), 10.0, 2)
    assert torch.equal(part[0, 0, 2:], torch.ones(4, dtype=torch.float64))


def _attention_weights(m, width=16, seed=0, sink=0.5):
    g = torch.Generator().manual_seed(seed)
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": torch.randn(H * d, width, generator=g), "k": torch.randn(G * d, width, generator=g),
         "v": torch.randn(G * e, width, generator=g), "g": torch.zeros(H * e, width), "o": torch.randn(width, H * e, generator=g),
         "q.b": torch.randn(H * d, generator=g), "k.b": torch.randn(G * d, generator=g), "v.b": torch.randn(G * e, generator=g),
         "o.b": torch.zeros(width), "sink": torch.full((H,), sink)}
    return {"x." + k: v.double() for k, v in w.items()}


def test_the_sink_takes_its_share_and_a_single_token_shows_it():
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 2, "scale": 0.5, "rot": {"dims": 0, "base": 10.0}}
    w = _attention_weights(m, sink=0.5)
    ar = plain.Arithmetic(torch.float64)
    h = torch.randn(1, 16, dtype=torch.float64)
    out = plain.softmax_attention(ar, h, w, "x.", m, 1e-6, torch.arange(1))
    q = plain.rms_divide(h @ w["x.q"].t() + w["x.q.b"], 1e-6)
    k = plain.rms_divide(h @ w["x.k"].t() + w["x.k.b"], 1e-6)
    s = (q * k).sum() * 0.5
    share = torch.exp(s) / (torch.exp(s) + math.exp(0.5))
    v = h @ w["x.v"].t() + w["x.v.b"]
    assert torch.allclose(out, (share * v * 0.5) @ w["x.o"].t(), atol=1e-12)      # the gate is logistic(0) = 1/2
    far = _attention_weights(m, sink=-40.0)
    assert torch.allclose(plain.softmax_attention(ar, h, far, "x.", m, 1e-6, torch.arange(1)), (v * 0.5) @ w["x.o"].t(), atol=1e-9)


def test_linear_attention_with_a_decay_of_one_is_a_plain_sum():
    m = {"heads": 2, "dim": 3, "vdim": 4, "decay": [1.0, 0.5]}
    g = torch.Generator().manual_seed(3)
    w = {"x." + k: torch.randn(*s, generator=g).double() for k, s in
         dict(q=(6, 8), k=(6, 8), v=(8, 8), g=(8, 8), o=(8, 8), norm=(8,)).items()}
    h = torch.randn(5, 8, generator=g).double()
    ar = plain.Arithmetic(torch.float64)
    out = plain.lightning_attention(ar, h, w, "x.", m, 1e-6)
    q, k, v = (plain.silu(h @ w["x." + n].t()) for n in "qkv")
    o = torch.zeros(5, 2, 4, dtype=torch.float64)
    for t in range(5):
        for j in range(t + 1):
            for head, decay in enumerate([1.0, 0.5]):
                o[t, head] += decay ** (t - j) * (q[t, head * 3:head * 3 + 3] @ k[j, head * 3:head * 3 + 3]) * v[j, head * 4:head * 4 + 4]
    y = plain.rms_divide(o.reshape(5, 8), 1e-6) * w["x.norm"] * plain.logistic(h @ w["x.g"].t())
    assert torch.allclose(out, y @ w["x.o"].t(), atol=1e-10)


def test_the_scan_sees_zeros_before_the_start_and_its_taps_in_order():
    m = {"inner": 2, "state": 1, "dt_rank": 1, "conv": 3}
    w = {"x.in": torch.eye(4, 4).double(), "x.conv": torch.tensor([[100.0, 10.0, 1.0], [0.0, 0.0, 1.0]]).double(),
         "x.conv.b": torch.zeros(2).double(), "x.x": torch.zeros(3, 2).double(), "x.dt": torch.zeros(2, 1).double(),
         "x.dt.b": torch.zeros(2).double(), "x.A_log": torch.zeros(2, 1).double(), "x.D": torch.ones(2).double(),
         "x.o": torch.eye(2, 2).double()}
    h = torch.tensor([[1.0, 1.0, 50.0, 50.0], [2.0, 2.0, 50.0, 50.0], [3.0, 3.0, 50.0, 50.0]]).double()
    out = plain.selective_scan(plain.Arithmetic(torch.float64), h, w, "x.", m)
    # B and C are zero: y = D x; z = 50 makes silu(z) = z; channel 0 sums its taps oldest first
    conv0 = torch.tensor([1.0, 12.0, 123.0]).double()
    assert torch.allclose(out[:, 0], plain.silu(conv0) * 50.0, rtol=1e-9)
    assert torch.allclose(out[:, 1], plain.silu(torch.tensor([1.0, 2.0, 3.0]).double()) * 50.0, rtol=1e-9)


def test_identity_connections_are_the_plain_residual():
    ar = plain.Arithmetic(torch.float64)
    X = torch.randn(4, 1, 6, dtype=torch.float64)
    w = {"n": torch.tensor(1.5).double(), "hc.in": torch.ones(1).double(), "hc.mix": torch.ones(1, 1).double(),
         "hc.out": torch.ones(1).double()}
    f = lambda h: 2.0 * h
    joined = plain.hyper_sublayer(ar, X, w, "hc.", "n", 1e-6, f)
    alone = plain.hyper_sublayer(ar, X, {"n": w["n"]}, "hc.", "n", 1e-6, f)
    assert torch.allclose(joined, alone) and torch.allclose(alone, X + 3.0 * plain.rms_divide(X, 1e-6))
    # mix is indexed [from, to]
    X2 = torch.randn(1, 2, 3, dtype=torch.float64)
    w2 = {"n": torch.tensor(1.0).double(), "hc.in": torch.tensor([1.0, 0.0]).double(),
          "hc.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]]).double(), "hc.out": torch.zeros(2).double()}
    moved = plain.hyper_sublayer(ar, X2, w2, "hc.", "n", 1e-6, f)
    assert torch.allclose(moved[0, 1], X2[0, 0]) and torch.allclose(moved[0, 0], torch.zeros(3, dtype=torch.float64))


def test_routing_weights_sum_to_one_and_the_weight_is_on_the_output():
    ar = plain.Arithmetic(torch.float64)
    g = torch.Generator().manual_seed(5)
    w = {"m.router": torch.randn(4, 6, generator=g).double()}
    for e in range(4):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = torch.randn(3, 6, generator=g).double(), torch.randn(3, 6, generator=g).double()
        w[f"m.e{e}.down"] = torch.randn(6, 3, generator=g).double()
    h = torch.randn(2, 6, generator=g).double()
    chosen, weight, z = plain.route(ar, h, w, "m.", 2)
    assert torch.allclose(weight.sum(-1), torch.ones(2, dtype=torch.float64))
    assert set(chosen[0].tolist()) == set(torch.topk(z[0], 2).indices.tolist())
    mlp = {"router": {"experts": 4, "top": 2}, "expert": {"ff": 3, "limit": 0.3}}
    out = plain.mixture(ar, h, w, "m.", mlp)
    by_hand = sum(c * plain.clamped_expert(ar, h[:1], w, f"m.e{e}.", 0.3)[0] for e, c in zip(chosen[0].tolist(), weight[0]))
    assert torch.allclose(out[0], by_hand)
    # the limit cuts: doubling a token that is far over the limit changes nothing in the gate
    big = clamped = plain.clamped_expert(ar, 100.0 * h[:1], w, "m.e0.", 0.3)
    assert torch.isfinite(big).all() and (clamped.abs() <= (0.3 * 1.3) * w["m.e0.down"].abs().sum(1) + 1e-9).all()
