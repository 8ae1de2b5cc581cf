"""Small Dubazen configurations of the tests' own, each unlike the others in every size and option,
and model folders with random weights for them.  Sizes visit the corners: one, three, four and
five copies of the stream and a model with one plain stream (no hyper-connection tensors); every
order of the three mixers; attention heads whose values are smaller than, equal to and larger than
their keys, with an even and an odd number of value pairs, one kv head for several heads and one per
head, no, partial and full rotation; linear attention with keys of 6 to 130 and a single head; decays
of exactly 1 and near 0; a scan with 1 to 5 taps, states of 3 to 40 and a step-size rank of 1 to 16;
one, several and all experts per token, with and without a shared expert; a layer without a
feed-forward; widths and vocabularies that are no multiple of eight."""

import json
import os

import torch


def softmax_half(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"base": base, "dims": rot_dims}}


def lightning_half(heads, dim, vdim, decay):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}


def parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale}, "mlp": mlp}


def gla(heads, dim, vdim, tau, rank, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}, "mlp": mlp}


def mamba(inner, state, dt_rank, conv, mlp):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def moe(experts, top, ff, limit, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


CONFIGS = {
    # three copies of the stream; values smaller than keys with an odd number of pairs; partial rotation;
    # two kv heads for four heads; a decay of exactly 1 beside one near 0; a scan layer without a feed-forward
    "a": dict(vocab=200, width=48, eps=1e-5, scale=6.0, streams=3, seed=41, layers=[
        gla(3, 10, 12, 8.0, 5, moe(5, 2, 24, 1.5, shared=(40, 0.8))),
        parallel(softmax_half(4, 2, 24, 10, 0.3, 8), lightning_half(3, 10, 20, [1.0, 0.9, 0.05]), 0.7, 1.3,
                 moe(5, 2, 24, 1.5, shared=(40, 0.8))),
        mamba(56, 5, 3, 4, None),
        parallel(softmax_half(4, 2, 24, 10, 0.3, 8), lightning_half(3, 10, 20, [0.5, 0.99, 0.999]), 1.0, 0.4,
                 moe(5, 2, 24, 1.5)),
    ]),
    # one plain stream (no hyper-connection tensors); values as large as keys of a tensor-core size, one kv
    # head per head, full rotation with another base; every expert chosen, no shared one; two taps; one head
    "b": dict(vocab=300, width=72, eps=3e-6, scale=1.0, streams=None, seed=42, layers=[
        mamba(80, 16, 16, 2, moe(4, 4, 48, 2.5)),
        parallel(softmax_half(2, 2, 64, 64, 0.2, 64, base=500.0), lightning_half(1, 64, 32, [0.97]), 0.5, 0.5,
                 moe(4, 4, 48, 2.5)),
        gla(1, 64, 8, 16.0, 8, None),
    ]),
    # one copy of the stream with its connection numbers; nothing a multiple of eight; no rotation of keys;
    # values larger than keys; keys of 130 in the linear half; one tap (no convolution to speak of); one
    # expert per token; a rank of one
    "c": dict(vocab=333, width=100, eps=2e-5, scale=12.0, streams=1, seed=43, layers=[
        parallel(softmax_half(3, 1, 18, 26, 0.25, 0), lightning_half(2, 130, 6, [0.8, 0.93]), 0.6, 0.9,
                 moe(7, 1, 30, 0.7, shared=(50, 3.0))),
        mamba(30, 40, 1, 1, moe(7, 1, 30, 0.7, shared=(50, 3.0))),
        gla(2, 6, 34, 2.0, 1, moe(7, 1, 30, 0.7)),
    ]),
    # five copies of the stream; heads of 128 on one kv head with values of 32; five taps; a state of 3
    "d": dict(vocab=97, width=40, eps=1e-6, scale=3.0, streams=5, seed=44, layers=[
        mamba(48, 3, 2, 5, moe(3, 2, 16, 1.2)),
        gla(2, 16, 16, 4.0, 4, moe(3, 2, 16, 1.2)),
        parallel(softmax_half(4, 1, 128, 32, 0.09, 32), lightning_half(2, 16, 24, [0.6, 0.9]), 0.6, 0.9, None),
    ]),
}


def config_json(name):
    c = CONFIGS[name]
    data = {"architecture": "Dubazen", "vocab": c["vocab"], "width": c["width"], "embedding": {"scale": c["scale"]},
            "norm": {"eps": c["eps"]}, "layers": c["layers"]}
    if c["streams"] is not None:
        data["streams"] = c["streams"]
    return data


def write_model(folder, name, dtype=torch.bfloat16):
    """Random weights through the library's random-weights mode (stored in bfloat16, as served models
    are), with matrices wide enough that attention weights are far from uniform and experts reach
    their limits.  Router matrices are wider still, so that a rounding seldom decides which expert is
    chosen; output projections are narrower, so that the stream stays of the order of the embedding."""
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
    g = torch.Generator().manual_seed(9000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (length,), generator=g).tolist()
