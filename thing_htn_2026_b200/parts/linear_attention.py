"""Linear attention with a decayed matrix state: a recurrent token mixer.  Per head it keeps a
matrix ``S [key_dim, value_dim]``, zero at the start of a sequence, and for every token

    S <- diag(a) S + k v^T          o = S^T q * q_scale

with ``q, k`` (heads of ``key_dim``) and ``v`` (heads of ``value_dim``) projections of the input,
through silu where ``silu_inputs`` says so.  The decay ``a`` (``decay``) is

* ``{"kind": "constant", "values": [...]}``: one constant per head, for every key channel and
  token (lightning attention);
* ``{"kind": "gated", "rank": r, "tau": tau}``: per token and key channel
  ``a = logistic(z)^(1 / tau)`` with ``z = W_a2 (W_a1 x) + b_a2`` through ``r`` channels (gated
  linear attention); ``rank`` None leaves r to the shapes of the checkpoint's two tensors.

The read-out is divided by its root mean square, per head with a gain over ``value_dim`` shared by
the heads (``norm_scope`` "head") or over all heads together with a gain over all their entries
("all"), multiplied by ``silu`` or ``logistic`` (``gate``) of a gate projection, and projected
back.  State per sequence: ``S`` float32 ``[n_heads, value_dim, key_dim]``.  Everything that enters
the recurrence after the projections is float32.  Kernel: csrc/linear_attention.cu.  A mixer in
phases (:mod:`.fused`).
"""

from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, StateSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .fused import PhasedMixer
from .registry import register_part
from .runtime import Runtime, StepContext


def pad_rank(first: torch.Tensor, second: torch.Tensor, multiple: int = 8):
    """A product through few channels, ``second (first x)``: the channels are filled up with zeros
    to a multiple of eight, which the tensor-core products want of a row and changes no result."""
    r = first.shape[0]
    to = -(-r // multiple) * multiple
    if to == r:
        return first.contiguous(), second.contiguous()
    first = torch.cat([first, first.new_zeros((to - r, first.shape[1]))], dim=0)
    second = torch.cat([second, second.new_zeros((second.shape[0], to - r))], dim=1)
    return first.contiguous(), second.contiguous()


@register_part("mixer", "linear_attention")
class LinearAttention(PhasedMixer):
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        return int(p["hidden_size"]), int(p["n_heads"]), int(p["key_dim"]), int(p["value_dim"])

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, h, d, e = cls._sizes(spec)
        p, t = spec.params, spec.tensors
        specs = [TensorSpec(t["q"], (h * d, hidden), MATRIX), TensorSpec(t["k"], (h * d, hidden), MATRIX),
                 TensorSpec(t["v"], (h * e, hidden), MATRIX), TensorSpec(t["g"], (h * e, hidden), MATRIX),
                 TensorSpec(t["o"], (hidden, h * e), MATRIX),
                 TensorSpec(t["norm"], (h * e if p.get("norm_scope", "head") == "all" else e,), GAIN)]
        decay = p["decay"]
        if decay["kind"] == "gated":
            r = -1 if decay.get("rank") is None else int(decay["rank"])
            specs += [TensorSpec(t["a1"], (r, hidden), MATRIX), TensorSpec(t["a2"], (h * d, r), MATRIX, init="unit_normal"),
                      TensorSpec(t["a2_bias"], (h * d,), GAIN, init="gate_bias")]
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        _, self.n_heads, self.key_dim, self.value_dim = self._sizes(spec)
        h, d, e = self.n_heads, self.key_dim, self.value_dim
        self.dtype = runtime.dtype
        self.norm_eps = float(p["norm_eps"])
        self.norm_all = p.get("norm_scope", "head") == "all"
        self.gate_kind = str(p.get("gate", "silu"))
        if p.get("norm_scope", "head") not in ("head", "all") or self.gate_kind not in ops.GATE_KINDS:
            raise ValueError(f"linear_attention: norm_scope {p.get('norm_scope')!r} or gate {self.gate_kind!r} unknown")
        self.silu_inputs = bool(p.get("silu_inputs"))
        self.q_scale = float(p.get("q_scale", 1.0))
        decay = p["decay"]
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.decay = self.tau = self.w_a1 = self.w_a2 = self.a_bias = None
        if decay["kind"] == "constant":
            values = [float(v) for v in decay["values"]]
            if len(values) != h:
                raise ValueError(f"linear_attention: {len(values)} decays for {h} heads")
            self.decay = torch.tensor(values, dtype=torch.float64).to(torch.float32).to(runtime.device)
        elif decay["kind"] == "gated":
            self.tau = float(decay["tau"])
            if runtime.tensor(spec, "a1").shape[0] != runtime.tensor(spec, "a2").shape[1]:
                raise ValueError("linear_attention: the two projections of the decay do not meet in one rank")
            self.w_a1, self.w_a2 = pad_rank(runtime.tensor(spec, "a1"), runtime.tensor(spec, "a2"))
            self.a_bias = f32(runtime.tensor(spec, "a2_bias"))
        else:
            raise ValueError(f"linear_attention: decay kind {decay['kind']!r} is neither 'constant' nor 'gated'")
        self.out_gain = f32(runtime.tensor(spec, "norm"))
        self.inner_width = h * e
        self.gate_offset = 2 * h * d + h * e
        self._in = (torch.cat([runtime.tensor(spec, n) for n in ("q", "k", "v", "g")], dim=0).contiguous(), None)
        self._out = (runtime.tensor(spec, "o"), None)
        self.finish()

    def in_rows(self):
        return self._in

    def out_rows(self):
        return self._out

    def cache_need(self) -> CacheNeed:
        return StateSpec((self.n_heads, self.value_dim, self.key_dim), torch.float32)

    def inner(self, x, proj, offset, ctx: StepContext, entry: ScheduleEntry, out, out_offset, scale) -> None:
        h, d, e = self.n_heads, self.key_dim, self.value_dim
        state = ctx.cache.state_view(entry.cache, self.state_base)
        gate = None
        if self.tau is not None:
            gate = ops.linear(ops.linear(x, self.w_a1, err=ctx.err), self.w_a2, out_dtype=torch.float32, err=ctx.err)
        o = ops.linear_attention(proj, (offset, offset + h * d, offset + 2 * h * d), state, ctx.rows, h, d, e,
                                 decay=self.decay, gate=gate, gate_bias=self.a_bias, tau=self.tau or 1.0,
                                 q_scale=self.q_scale, silu_inputs=self.silu_inputs)
        if self.norm_all:
            ops.gated_head_norm(o, proj, offset + self.gate_offset, self.out_gain, self.norm_eps, 1, h * e, self.dtype,
                                self.gate_kind, scale, out, out_offset)
        else:
            ops.gated_head_norm(o, proj, offset + self.gate_offset, self.out_gain, self.norm_eps, h, e, self.dtype,
                                self.gate_kind, scale, out, out_offset)
