"""A plain, slow implementation of the Dubazen decoder, one function per mechanism, written
from the design's equations with torch on the CPU.  It shares no code with the library: it
reads a model folder with its own safetensors reader, walks a sequence token by token where
the design has a recurrence, builds every mask as a full matrix and keeps no cache or state
between calls.

Notation.  A model keeps ``s`` residual streams ``X[t, 0..s-1]`` (width ``W``) per token, all
equal to ``embed[token] * scale`` at the start.  Sublayer ``f`` with the numbers ``a[s]``
(read), ``M[s, s]`` (mix, indexed [from, to]) and ``b[s]`` (write) does

    u = sum_j a[j] X[j];   y = f(g * u / sqrt(mean(u^2) + eps));   X'[i] = sum_j M[j, i] X[j] + b[i] y

with ``g`` one number.  A layer is its mixer as such a sublayer, then its feed-forward where it
has one.  The logits read the sum of the streams through the last norm.  ``precision`` is
``torch.float32`` or ``torch.float64`` for exact arithmetic, or ``torch.bfloat16`` for an
emulation of serving precision: operands and results of matrix products (and the short
convolution with its activation) are rounded to bfloat16, everything else stays in float32.
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

    def linear(self, x, w, bias=None, keep=False):
        """``x @ w.T (+ bias)`` for a weight of shape [outputs, inputs]; ``keep``: not rounded."""
        y = self.rb(x) @ self.rb(w.to(self.work)).t()
        if bias is not None:
            y = y + bias.to(self.work)
        return y if keep else self.rb(y)


# ----------------------------------------------------------------------------- small pieces


def logistic(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * logistic(x)


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


def rms_divide(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate(x, positions, base, dims, sign=1.0):
    """Turns the first ``dims`` entries of the last axis of ``x`` [tokens, ..., size]: entry i
    pairs with entry i + dims/2, and the pair of token t turns by ``sign * p_t * base^(-2i/dims)``."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    angle = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)       # [tokens, half]
    angle = (sign * angle).to(torch.float32 if x.dtype != torch.float64 else torch.float64)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(angle).to(x.dtype).reshape(shape), torch.sin(angle).to(x.dtype).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- mixers


def softmax_attention(ar, h, w, prefix, m, eps, positions):
    """Grouped-query attention with biases, rotation, unit-RMS queries and keys, values that
    are turned by their position and turned back at the reader's, a sink in the softmax's
    denominator and a logistic output gate."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = ar.linear(h, w[prefix + "q"], w[prefix + "q.b"]).reshape(T, H, d)
    k = ar.linear(h, w[prefix + "k"], w[prefix + "k.b"]).reshape(T, G, d)
    v = ar.linear(h, w[prefix + "v"], w[prefix + "v.b"]).reshape(T, G, e)
    q = rms_divide(rotate(q, positions, rot["base"], rot["dims"]), eps)
    k = rms_divide(rotate(k, positions, rot["base"], rot["dims"]), eps)
    v = rotate(v, positions, rot["base"], e)
    q, k, v = ar.rb(q), ar.rb(k), ar.rb(v)
    sink = w[prefix + "sink"].to(ar.work)
    visible = positions[:, None] >= positions[None, :]
    out = torch.zeros(T, H, e, dtype=ar.work)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].t()) * m["scale"]
        score = score.masked_fill(~visible, -math.inf)
        top = torch.maximum(score.max(-1, keepdim=True).values, sink[head])
        weight = torch.exp(score - top)
        total = weight.sum(-1, keepdim=True) + torch.exp(sink[head] - top)
        out[:, head] = (weight / total) @ v[:, g]
    out = rotate(out, positions, rot["base"], e, sign=-1.0)
    gate = logistic(ar.linear(h, w[prefix + "g"]))
    return ar.linear(ar.rb(out.reshape(T, H * e) * gate), w[prefix + "o"], w[prefix + "o.b"])


def lightning_attention(ar, h, w, prefix, m, eps):
    """Linear attention with one constant decay per head: S <- decay S + k v^T, o = S^T q, on
    silu'd projections; one RMS norm over all heads' read-outs, a logistic gate."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = silu(ar.linear(h, w[prefix + "q"])).reshape(T, H, d)
    k = silu(ar.linear(h, w[prefix + "k"])).reshape(T, H, d)
    v = silu(ar.linear(h, w[prefix + "v"])).reshape(T, H, e)
    decay = torch.tensor(m["decay"], dtype=ar.work)
    S = torch.zeros(H, d, e, dtype=ar.work)
    out = torch.zeros(T, H, e, dtype=ar.work)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    y = rms_divide(out.reshape(T, H * e), eps) * w[prefix + "norm"].to(ar.work)
    y = y * logistic(ar.linear(h, w[prefix + "g"]))
    return ar.linear(ar.rb(y), w[prefix + "o"])


def parallel_mixer(ar, h, w, prefix, m, eps, positions):
    left = softmax_attention(ar, h, w, prefix + "left.", m["left"], eps, positions)
    right = lightning_attention(ar, h, w, prefix + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_linear_attention(ar, h, w, prefix, m, eps):
    """S <- diag(alpha_t) S + k v^T, o = S^T q with a decay per key channel,
    alpha = logistic(z)^(1/tau); per-head RMS norm with a gain, a silu gate."""
    T = h.shape[0]
    H, d, e = m["heads"], m["dim"], m["vdim"]
    q = (ar.linear(h, w[prefix + "q"]) * d ** -0.5).reshape(T, H, d)
    k = ar.linear(h, w[prefix + "k"]).reshape(T, H, d)
    v = ar.linear(h, w[prefix + "v"]).reshape(T, H, e)
    z = ar.linear(ar.linear(h, w[prefix + "a1"]), w[prefix + "a2"], w[prefix + "a2.b"], keep=True)
    log_alpha = -softplus(-z) / m["tau"]                  # ln(logistic(z)) / tau
    alpha = torch.exp(log_alpha).reshape(T, H, d)
    S = torch.zeros(H, d, e, dtype=ar.work)
    out = torch.zeros(T, H, e, dtype=ar.work)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hde,hd->he", S, q[t])
    y = rms_divide(out, eps) * w[prefix + "norm"].to(ar.work)
    y = y.reshape(T, H * e) * silu(ar.linear(h, w[prefix + "g"]))
    return ar.linear(ar.rb(y), w[prefix + "o"])


def selective_scan(ar, h, w, prefix, m):
    """Mamba: a short causal convolution and silu on x, input-dependent step size, B and C;
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c."""
    T = h.shape[0]
    inner, N, R, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    xz = ar.linear(h, w[prefix + "in"])
    x, z = xz[:, :inner], xz[:, inner:]
    kernel, kb = w[prefix + "conv"].to(ar.work), w[prefix + "conv.b"].to(ar.work)
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=ar.work), x], dim=0)
    conv = sum(padded[j:j + T] * kernel[:, j] for j in range(taps)) + kb
    x = ar.rb(silu(conv))
    low = ar.linear(x, w[prefix + "x"])
    dt_low, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:R + 2 * N]
    dt = softplus(ar.linear(dt_low, w[prefix + "dt"], keep=True) + w[prefix + "dt.b"].to(ar.work))
    A = -torch.exp(w[prefix + "A_log"].to(ar.work))
    D = w[prefix + "D"].to(ar.work)
    S = torch.zeros(inner, N, dtype=ar.work)
    y = torch.zeros(T, inner, dtype=ar.work)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return ar.linear(ar.rb(y * silu(z)), w[prefix + "o"])


# ----------------------------------------------------------------------------- feed-forward


def clamped_expert(ar, h, w, prefix, limit):
    g = torch.clamp(ar.linear(h, w[prefix + "gate"]), max=limit)
    u = torch.clamp(ar.linear(h, w[prefix + "up"]), min=-limit, max=limit)
    return ar.linear(ar.rb(g * logistic(1.702 * g) * (u + 1.0)), w[prefix + "down"], keep=True)


def route(ar, h, w, prefix, top):
    """(chosen experts [tokens, top], their weights): softmax over all experts, the ``top``
    largest, their scores divided by their sum."""
    z = ar.linear(h, w[prefix + "router"], keep=True)
    s = torch.softmax(z, dim=-1)
    best = torch.topk(s, top, dim=-1)
    return best.indices, best.values / (best.values.sum(-1, keepdim=True) + 1e-20), z


MARGINS = None      # a list, while a caller collects per-token routing margins (routing_margin below)


def mixture(ar, h, w, prefix, mlp):
    T = h.shape[0]
    chosen, weight, z = route(ar, h, w, prefix, mlp["router"]["top"])
    if MARGINS is not None:
        top = mlp["router"]["top"]
        ordered = torch.sort(z, dim=-1, descending=True).values
        MARGINS.append(ordered[:, top - 1] - ordered[:, top] if top < z.shape[-1] else torch.full((T,), math.inf))
    out = torch.zeros(T, w[prefix + "e0.down"].shape[0], dtype=ar.work)
    for t in range(T):
        for e, c in zip(chosen[t].tolist(), weight[t]):
            out[t] += c * clamped_expert(ar, h[t:t + 1], w, f"{prefix}e{e}.", mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(ar, h, w, prefix + "shared.", mlp["shared"]["limit"])
    return ar.rb(out)


# ----------------------------------------------------------------------------- the model


def scalar_norm(u, gain, eps):
    return rms_divide(u, eps) * gain


def hyper_sublayer(ar, X, w, prefix, norm_name, eps, f):
    """One sublayer over the streams X [tokens, s, W]; without hyper-connection numbers (a model
    of one plain stream) it is x <- x + f(norm(x))."""
    gain = w[norm_name].to(ar.work)
    if prefix + "in" not in w:
        return X + f(ar.rb(scalar_norm(X[:, 0], gain, eps)))[:, None, :]
    a, M, b = (w[prefix + k].to(ar.work) for k in ("in", "mix", "out"))
    u = torch.einsum("j,tjw->tw", a, X)
    y = f(ar.rb(scalar_norm(u, gain, eps))).to(ar.work)
    return torch.einsum("ji,tjw->tiw", M, X) + b[None, :, None] * y[:, None, :]


def model_forward(folder, tokens, precision=torch.float64, model=None):
    """(logits [tokens, vocab], sums of the streams after every layer [layers, tokens, W])."""
    config, w = model if model is not None else read_model(folder)
    ar = Arithmetic(precision)
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.int64)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"].to(ar.work)[tokens] * config.get("embedding", {}).get("scale", 1.0)
    streams = int(config.get("streams") or 1)
    X = x[:, None, :].repeat(1, streams, 1)
    after = []
    for i, layer in enumerate(config["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        if kind == "parallel":
            mixer = lambda h: parallel_mixer(ar, h, w, p + "mix.", m, eps, positions)
        elif kind == "gla":
            mixer = lambda h: gated_linear_attention(ar, h, w, p + "mix.", m, eps)
        elif kind == "mamba1":
            mixer = lambda h: selective_scan(ar, h, w, p + "mix.", m)
        else:
            raise ValueError(f"layer {i}: type {kind!r}")
        X = hyper_sublayer(ar, X, w, p + "hc1.", p + "norm1", eps, mixer)
        if layer.get("mlp") is not None:
            X = hyper_sublayer(ar, X, w, p + "hc2.", p + "norm2", eps,
                               lambda h: mixture(ar, h, w, p + "mlp.", layer["mlp"]))
        after.append(X.sum(1))
    n = ar.rb(scalar_norm(X.sum(1), w["final.norm"].to(ar.work), eps))
    logits = ar.linear(n, w["head"], keep=True)
    return logits, torch.stack(after)


def model_logits(folder, tokens, precision=torch.float64, model=None):
    return model_forward(folder, tokens, precision, model)[0]


def routing_margin(folder, tokens):
    """Per token, over all routed layers, the smallest distance between the logit of the last
    expert chosen and that of the best one left out, in float64: how sure the routing is."""
    global MARGINS
    MARGINS = []
    try:
        model_forward(folder, tokens, torch.float64)
        return torch.stack(MARGINS).min(0).values if MARGINS else torch.full((len(tokens),), math.inf)
    finally:
        MARGINS = None


def greedy(folder, prompt, n_new, precision=torch.float64):
    model = read_model(folder)
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(model_forward(folder, tokens, precision, model)[0][-1].argmax()))
    return tokens[len(prompt):]
