"""Small Ditilix configurations of the tests' own, each unlike the others in every size and
option, and model folders with random weights for them.  Sizes visit the corners: head sizes
that take the tensor-core kernels (32, 64, 128) and ones that do not (9, 20), values larger and
smaller than keys, one kv head for many heads and one per head, norm groups of 1 to 5, layers
that read an earlier layer's keys (the layer just before, and one three layers back), a layer
without a feed-forward, dense and routed feed-forwards in every order, one expert per token,
several and all, with and without a shared expert, with and without a score cap and a query
temperature (periods of 1, 16 and 70 positions, a negative coefficient), factors on the residual
and on the logits that are absent, 1, smaller and larger than 1."""

import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # heads of 64 (tensor-core kernels in bfloat16); three norm groups; a cap that the scores reach;
    # a temperature that steps every 16 positions; two experts of six per token with a shared one
    # whose limit differs; layer 2 reads layer 1's keys, layer 3 (no feed-forward) layer 0's
    "a": dict(vocab=200, width=96, eps=1e-5, groups=3, mult=0.5, logit_scale=2.0, seed=31, layers=[
        layer(attention(4, 2, 64, 64, 0.5, softcap=4.0, temp=(0.3, 16)), dense(136)),
        layer(attention(4, 2, 64, 64, 0.5, softcap=4.0, temp=(0.3, 16)), moe(6, 2, 24, 1.5, shared=(40, 0.8))),
        layer(attention(4, 2, 64, 64, 0.25, softcap=9.0, temp=(0.3, 16), kv_from=1), moe(6, 2, 24, 1.5, shared=(40, 0.8))),
        layer(attention(4, 2, 64, 64, 0.5, softcap=4.0, kv_from=0), None),
    ]),
    # heads of 128 (the tcgen05 prompt kernel in bfloat16) and of 32 with eight heads on one kv head;
    # one norm group; a temperature period longer than a page; one expert of four per token, no
    # shared expert; no factor on the residual or the logits in the file
    "b": dict(vocab=300, width=72, eps=3e-6, groups=1, mult=None, logit_scale=None, seed=32, layers=[
        layer(attention(2, 1, 128, 128, 0.3, softcap=5.0, temp=(1.0, 70)), moe(4, 1, 48, 2.5)),
        layer(attention(2, 1, 128, 128, 0.2, softcap=7.0, temp=(1.0, 70), kv_from=0), dense(80)),
        layer(attention(8, 1, 32, 32, 0.4, temp=(0.6, 70)), moe(4, 1, 48, 2.5)),
    ]),
    # nothing a multiple of eight: width 100 in five groups, heads of 9 with values of 5, every expert
    # chosen, a shared expert wider than the routed ones; a layer without a cap and one without a
    # temperature; a temperature that changes at every position
    "c": dict(vocab=333, width=100, eps=2e-5, groups=5, mult=1.0, logit_scale=0.3, seed=33, layers=[
        layer(attention(3, 1, 9, 5, 0.9, temp=(0.2, 1)), moe(5, 5, 30, 0.7, shared=(50, 3.0))),
        layer(attention(3, 1, 9, 5, 0.9, softcap=2.0, kv_from=0), dense(77)),
        layer(attention(2, 2, 20, 36, 0.6, softcap=3.0, temp=(0.2, 1)), moe(5, 5, 30, 0.7, shared=(50, 3.0))),
        layer(attention(2, 2, 20, 36, 0.3, kv_from=2), None),
    ]),
    # values smaller than keys of a tensor-core size (48 and 32), one kv head per head; two groups; a
    # negative temperature coefficient; three experts of seven, no shared one; a dense layer last
    "d": dict(vocab=97, width=40, eps=1e-6, groups=2, mult=0.2, logit_scale=1.0, seed=34, layers=[
        layer(attention(6, 6, 48, 32, 0.35, softcap=6.0, temp=(-0.05, 3)), moe(7, 3, 16, 1.2)),
        layer(attention(6, 6, 48, 32, 0.35, softcap=6.0, temp=(-0.05, 3), kv_from=0), moe(7, 3, 16, 1.2)),
        layer(attention(2, 1, 48, 48, 0.35, softcap=6.0, temp=(0.4, 40)), dense(64)),
    ]),
}


def config_json(name):
    c = CONFIGS[name]
    data = {"architecture": "Ditilix", "vocab": c["vocab"], "width": c["width"],
            "norm": {"eps": c["eps"], "groups": c["groups"]}, "layers": c["layers"]}
    if c["mult"] is not None:
        data["residual_mult"] = c["mult"]
    if c["logit_scale"] is not None:
        data["logit_scale"] = c["logit_scale"]
    return data


def write_model(folder, name, dtype=torch.bfloat16):
    """Random weights through the library's random-weights mode (stored in bfloat16, as served
    models are), with matrices wide enough that attention weights are far from uniform and scores
    reach their cap.  Router matrices are three times wider still: the scores of the experts lie
    far apart, so that a rounding seldom decides which expert is chosen."""
    from thing_htn_2026_b200.config import config_from_dict
    from thing_htn_2026_b200.weights import random_tensors_cpu
    from thing_htn_2026_b200.weights.safetensors_io import write_safetensors
    config = config_from_dict(config_json(name))
    tensors = random_tensors_cpu(config, CONFIGS[name]["seed"], dtype, matrix_std=0.12, gain_std=0.1)
    for key in tensors:
        if key.endswith(".mlp.router"):
            tensors[key] = (tensors[key].float() * 3.0).to(dtype)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as handle:
        json.dump(config_json(name), handle, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors, metadata={"format": "pt"})
    return folder


def tokens(name, length, seed):
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (length,), generator=g).tolist()
