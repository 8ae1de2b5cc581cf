"""A plain, slow implementation of the Ditilix decoder, one function per mechanism, written
from the design's equations with torch on the CPU.  It shares no code with the library: it
reads a model folder with its own safetensors reader, builds every mask as a full matrix,
visits experts one by one and keeps no cache.

Notation.  ``x[t]`` is the residual stream at token t (width ``W``), ``p`` a token's position
in its sequence, counted from 0.  The stream starts as ``embed[token] + pe(p)`` with
``pe(p)[2i] = sin(p w_i)``, ``pe(p)[2i+1] = cos(p w_i)``, ``w_i = 10000^(-2i/W)``.  A layer is

    n = gnorm(x) ;  x <- x + r * (mix(n) + ff(n))           (ff absent in a layer without one)

with one norm per layer that both sublayers read, ``r`` the model's residual multiplier and
``gnorm`` an RMS norm in ``groups`` equal consecutive parts, each divided by its own
``sqrt(mean(part^2) + eps)``, the whole times a gain.  The model ends with ``gnorm`` and
``logits = head(x) * logit_scale``.

``precision`` is ``torch.float32`` or ``torch.float64`` for exact arithmetic, or
``torch.bfloat16`` for an emulation of serving precision: operands and results of matrix
products are rounded to bfloat16, everything else stays in float32.
"""

import json
import math
import os
import struct

import numpy as np
import torch


# ----------------------------------------------------------------------------- reading


def read_safetensors(path):
    with open(path, "rb") as handle:
        (n,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(n).decode("utf-8"))
        data = handle.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8)
        if meta["dtype"] == "BF16":
            t = torch.from_numpy((raw.view("<u2").astype(np.uint32) << 16).view(np.float32).copy())
        elif meta["dtype"] == "F32":
            t = torch.from_numpy(raw.view("<f4").copy())
        elif meta["dtype"] == "I32":
            t = torch.from_numpy(raw.view("<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = t.reshape(meta["shape"])
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


# ----------------------------------------------------------------------------- precision


class Arithmetic:
    """``work``: the type everything is computed in; ``round_products``: whether operands and
    results of matrix products pass through bfloat16."""

    def __init__(self, precision):
        self.round_products = precision == torch.bfloat16
        self.work = torch.float32 if self.round_products else precision

    def rb(self, t):
        return t.to(torch.bfloat16).to(self.work) if self.round_products else t

    def linear(self, x, w, keep=False):
        """``x @ w.T`` for a weight matrix of shape [outputs, inputs]; ``keep``: the result is not rounded."""
        y = self.rb(x) @ self.rb(w.to(self.work)).t()
        return y if keep else self.rb(y)


# ----------------------------------------------------------------------------- small pieces


def sinusoid(positions, width, work):
    """[T, width]: sin of ``p w_i`` at the even entries, cos of the same at the odd ones."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * (10000.0 ** (-2.0 * i / width))[None, :]
    out = torch.zeros(positions.shape[0], 2 * i.shape[0], dtype=torch.float64)
    out[:, 0::2] = torch.sin(angle)
    out[:, 1::2] = torch.cos(angle)
    return out[:, :width].to(work)


def group_norm_rms(x, gain, groups, eps):
    T, W = x.shape
    parts = x.view(T, groups, W // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(T, W) * gain


def over_rms(y, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def query_temperature(positions, q_temp, work):
    """[T]: ``1 + coef * ln(floor((p + 1) / every) + 1)``; 1 without the option."""
    if not q_temp:
        return torch.ones(positions.shape[0], dtype=work)
    steps = torch.div(positions + 1, int(q_temp["every"]), rounding_mode="floor")
    return (1.0 + float(q_temp["coef"]) * torch.log(steps.to(torch.float64) + 1.0)).to(work)


def capped(s, cap):
    return s if not cap else float(cap) * torch.tanh(s / float(cap))


def causal_mask(T):
    i = torch.arange(T)
    return i[None, :] <= i[:, None]


# ----------------------------------------------------------------------------- mixer


def project_kv(n, t, prefix, m, ar):
    """Keys [T, G, D] and values [T, G, E] of a layer that has projections of its own, as its
    cache would hold them (rounded like every product's result)."""
    T = n.shape[0]
    k = ar.linear(n, t[prefix + "k"]).view(T, m["kv_heads"], m["dim"])
    v = ar.linear(n, t[prefix + "v"]).view(T, m["kv_heads"], m["vdim"])
    return k, v


def attention_mixer(n, t, prefix, m, ar, kv):
    """Grouped-query attention without rotation: the query of position p is stretched by the
    query temperature, scores are ``q . k * scale`` passed through ``cap * tanh(. / cap)``,
    every key j <= p is visible, plain softmax.  ``kv``: (keys, values) of this layer or of the
    layer whose cache it reads."""
    T = n.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = kv
    q = ar.linear(n, t[prefix + "q"]).view(T, H, D)
    temp = query_temperature(torch.arange(T), m.get("q_temp"), ar.work)
    visible = causal_mask(T)
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].t()) * temp[:, None] * float(m["scale"])
        s = capped(s, m.get("softcap")).masked_fill(~visible, float("-inf"))
        heads.append(torch.softmax(s, dim=-1) @ v[:, g])
    a = torch.stack(heads, dim=1).reshape(T, H * E)
    return ar.linear(a, t[prefix + "o"])


# ----------------------------------------------------------------------------- feed-forward


def poly_norm(z, coefficients, eps):
    a, b, c, e = (float(x) for x in coefficients)
    return a * over_rms(z, eps) + b * over_rms(z * z, eps) + c * over_rms(z * z * z, eps) + e


def dense_ff(n, t, prefix, eps, ar):
    z = ar.linear(n, t[prefix + "up"])
    return ar.linear(poly_norm(z, t[prefix + "act"], eps), t[prefix + "down"])


def clamped_expert(n, t, prefix, limit, ar):
    """``down(g * logistic(1.702 g) * (u + 1))``, ``g = min(gate(n), limit)``, ``u = clamp(up(n), +-limit)``."""
    g = ar.linear(n, t[prefix + "gate"]).clamp(max=limit)
    u = ar.linear(n, t[prefix + "up"]).clamp(min=-limit, max=limit)
    return ar.linear(g * torch.sigmoid(1.702 * g) * (u + 1.0), t[prefix + "down"])


def route(z, top):
    """z [T, experts] router logits -> (chosen [T, top], weights [T, top]): logistic scores, the
    largest ``top``, weighted by the scores as they are."""
    s = torch.sigmoid(z)
    chosen = s.topk(top, dim=-1).indices
    return chosen, s.gather(-1, chosen)


def moe(n, t, prefix, mlp, ar, margins=None):
    """The chosen experts see the token times its routing weight; their outputs are summed as
    they are.  The shared expert sees the token itself; its output is multiplied by
    ``logistic(sg . n)``.  ``margins`` (a list) receives, per token, the distance in the router's
    logits between the last expert chosen and the first one left out."""
    router = mlp["router"]
    z = ar.linear(n, t[prefix + "router"], keep=True)
    chosen, weights = route(z, int(router["top"]))
    if margins is not None and int(router["top"]) < int(router["experts"]):
        ordered = z.sort(dim=-1, descending=True).values
        margins.append(ordered[:, int(router["top"]) - 1] - ordered[:, int(router["top"])])
    out = torch.zeros_like(n)
    limit = float(mlp["expert"]["limit"])
    for e in range(int(router["experts"])):
        for slot in range(int(router["top"])):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += clamped_expert(weights[rows, slot, None] * n[rows], t, f"{prefix}e{e}.", limit, ar)
    if mlp.get("shared"):
        gate = torch.sigmoid(ar.linear(n, t[prefix + "shared.sg"], keep=True))
        out = out + gate * clamped_expert(n, t, prefix + "shared.", float(mlp["shared"]["limit"]), ar)
    return out


def feed_forward(n, t, prefix, mlp, eps, ar, margins=None):
    if mlp["kind"] == "dense":
        return dense_ff(n, t, prefix, eps, ar)
    return moe(n, t, prefix, mlp, ar, margins)


# ----------------------------------------------------------------------------- the model


def forward(config, tensors, tokens, precision=torch.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after
    every layer, ``margins`` (a list) the routing margins [T] of every routed layer."""
    ar = Arithmetic(precision)
    w = ar.work
    t = {k: v.to(w) if v.is_floating_point() else v for k, v in tensors.items()}
    eps, groups = float(config["norm"]["eps"]), int(config["norm"].get("groups", 1))
    r = float(config.get("residual_mult", 1.0))
    T = len(tokens)
    x = t["embed"][torch.tensor(tokens, dtype=torch.long)] + sinusoid(torch.arange(T), int(config["width"]), w)
    held = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        n = group_norm_rms(x, t[p + "norm1"], groups, eps)
        if m.get("kv_from") is None:
            held[i] = project_kv(n, t, p + "mix.", m, ar)
            kv = held[i]
        else:
            kv = held[int(m["kv_from"])]
        y = attention_mixer(n, t, p + "mix.", m, ar, kv)
        if layer.get("mlp"):
            y = y + feed_forward(n, t, p + "mlp.", layer["mlp"], eps, ar, margins)
        x = x + r * y
        if layers_out is not None:
            layers_out.append(x.clone())
    x = group_norm_rms(x, t["final.norm"], groups, eps)
    return ar.linear(x, t["head"], keep=True) * float(config.get("logit_scale", 1.0))


def greedy(config, tensors, prompt, n_new, precision=torch.float64):
    out = list(prompt)
    for _ in range(n_new):
        out.append(int(forward(config, tensors, out, precision)[-1].argmax()))
    return out[len(prompt):]


def routing_margin(config, tensors, tokens):
    """[T]: per token, the smallest routing margin over the routed layers, in exact arithmetic
    (infinite where every expert is chosen)."""
    margins = []
    forward(config, tensors, tokens, torch.float64, margins=margins)
    out = torch.full((len(tokens),), float("inf"), dtype=torch.float64)
    for m in margins:
        out = torch.minimum(out, m)
    return out


_models = {}


def model_logits(folder, tokens, precision=torch.float32):
    """Logits [T, vocab] (float32) of one whole sequence through the model stored in ``folder``."""
    if folder not in _models:
        _models[folder] = read_model(folder)
    config, tensors = _models[folder]
    return forward(config, tensors, list(tokens), precision).to(torch.float32)
