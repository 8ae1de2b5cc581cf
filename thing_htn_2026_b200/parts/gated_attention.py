"""Grouped-query attention with biased projections, a sink in the softmax and an output gate.

    q = W_q x + b_q,  k = W_k x + b_k,  v = W_v x + b_v       (``biases``; heads of ``head_dim``, values of ``value_dim``)
    q, k: rotation of the first ``rotary_dim`` entries of a head (``position``), then each head
          divided by its root mean square (``qk_norm_eps``; no gain)
    v:    turned by its own position over ``value_position``'s entries before it is cached; a head's
          output at position i is turned back by i (so a value enters the sum turned by j - i)
    weights of row i over j <= i: exp(s_ij) / (sum_j exp(s_ij) + exp(sink_h)),  s = (q . k) * scale
          (``sinks``: one learned number per head, without key and value)
    y = W_o (concat(heads) * logistic(W_g x)) + b_o            (``gate`` "logistic")

The rotation commutes with the division by the root mean square (a rotation keeps a head's length
and the norm has no gain), so the kernel that normalises first and then turns computes the same.
One product gives q, k, v and the gate; :func:`ops.qk_prepare` normalises, turns and writes the
cache in float32 with one rounding; the attention kernels keep scores and weights in float32 (the
tensor-core kernels, which take keys and values of one size from 32 to 128 in bfloat16, multiply
the values by the weights as two bfloat16 parts);
:func:`ops.rotate_gate` turns the read-out back and gates it.  A mixer in phases
(:mod:`.fused`), so that it can share its products with a mixer beside it.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import ops
from ..cache.sequence_cache import CacheNeed, KVSpec
from ..config.base import PartSpec, ScheduleEntry
from ..weights.loader import GAIN, MATRIX, TensorSpec
from .fused import PhasedMixer, cat_bias
from .registry import part_class, register_part
from .runtime import HostBatch, Runtime, StepContext


def _position(runtime: Runtime, spec: Optional[PartSpec]):
    if spec is None:
        return None
    key = "position:" + spec.key()
    if key not in runtime.shared:
        runtime.shared[key] = part_class("position", spec.kind)(spec, runtime)
    return runtime.shared[key]


@register_part("mixer", "gated_attention")
class GatedAttention(PhasedMixer):
    @staticmethod
    def _sizes(spec: PartSpec):
        p = spec.params
        d = int(p["head_dim"])
        return int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), d, int(p.get("value_dim") or d)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> List[TensorSpec]:
        hidden, n_q, n_kv, d, dv = cls._sizes(spec)
        p, t = spec.params, spec.tensors
        specs = [TensorSpec(t["q_proj"], (n_q * d, hidden), MATRIX), TensorSpec(t["k_proj"], (n_kv * d, hidden), MATRIX),
                 TensorSpec(t["v_proj"], (n_kv * dv, hidden), MATRIX), TensorSpec(t["o_proj"], (hidden, n_q * dv), MATRIX)]
        if p.get("biases"):
            specs += [TensorSpec(t["q_bias"], (n_q * d,), MATRIX, init="small_normal"),
                      TensorSpec(t["k_bias"], (n_kv * d,), MATRIX, init="small_normal"),
                      TensorSpec(t["v_bias"], (n_kv * dv,), MATRIX, init="small_normal"),
                      TensorSpec(t["o_bias"], (hidden,), MATRIX, init="small_normal")]
        if p.get("sinks"):
            specs.append(TensorSpec(t["sink"], (n_q,), GAIN, init="sink"))
        if p.get("gate"):
            specs.append(TensorSpec(t["g_proj"], (n_q * dv, hidden), MATRIX))
        return specs

    def __init__(self, spec: PartSpec, runtime: Runtime):
        p = spec.params
        _, self.n_q, self.n_kv, self.head_dim, self.value_dim = self._sizes(spec)
        if self.n_q % self.n_kv:
            raise ValueError(f"gated_attention: {self.n_q} heads are not a multiple of {self.n_kv} kv heads")
        if p.get("gate") != "logistic":
            raise ValueError(f"gated_attention: gate {p.get('gate')!r}; the read-out is turned back and scaled in the "
                             f"logistic gate's kernel, so the gate is 'logistic'")
        self.scale = float(p["scale"])
        self.eps = None if p.get("qk_norm_eps") is None else float(p["qk_norm_eps"])
        self.window = None if p.get("window") is None else int(p["window"])
        self.dtype = runtime.dtype
        self.position = _position(runtime, p.get("position"))
        self.value_position = _position(runtime, p.get("value_position"))
        self.gated = p.get("gate") == "logistic"
        self.biased = bool(p.get("biases"))
        self.inner_width = self.n_q * self.value_dim
        self.gate_offset = (self.n_q + self.n_kv) * self.head_dim + self.n_kv * self.value_dim
        self._spec, self._runtime_tensor = spec, lambda name: runtime.tensor(spec, name)
        self.sinks = runtime.tensor(spec, "sink").to(torch.float32).contiguous() if p.get("sinks") else None
        self.unit_gain = torch.ones(self.head_dim, dtype=torch.float32, device=runtime.device) if self.eps is not None else None
        rows = [(self._runtime_tensor(n + "_proj"), self._runtime_tensor(n + "_bias") if self.biased else None)
                for n in ("q", "k", "v")]
        if self.gated:
            rows.append((self._runtime_tensor("g_proj"), None))
        self._in = (torch.cat([w for w, _ in rows], dim=0).contiguous(), cat_bias(rows))
        self._out = (self._runtime_tensor("o_proj"), self._runtime_tensor("o_bias") if self.biased else None)
        self._runtime_tensor = None
        self.finish()

    def in_rows(self):
        return self._in

    def out_rows(self):
        return self._out

    def cache_need(self) -> CacheNeed:
        return KVSpec(self.n_kv, self.head_dim, self.window, 0, None, self.value_dim)

    def _tile(self, page_size: int) -> int:
        return ops.prompt_attention_tile(self.dtype, self.head_dim, page_size, self.n_q, self.n_kv, self.value_dim)

    def step_inputs(self, batch: HostBatch, out) -> None:
        """The row tiles of the tensor-core prompt kernel, where the sizes go to it (keys and values
        of one size that it takes); every attention that wants tiles of one size shares one list."""
        size = self._tile(batch.page_size) if batch.max_count > 1 else 0
        if size and f"row_tiles/{size}/row0" not in out:
            out[f"row_tiles/{size}/row0"], out[f"row_tiles/{size}/rows"] = ops.row_tiles_of(batch.counts, batch.held, size)

    def inner(self, x, proj, offset, ctx: StepContext, entry: ScheduleEntry, out, out_offset, scale) -> None:
        kv = ctx.cache.kv_view(entry.cache)
        tiles = None
        if ctx.rows.max_q_len > 1:
            size = self._tile(kv.page_size)
            row0 = ctx.inputs.get(f"row_tiles/{size}/row0") if size else None
            if row0 is not None:
                tiles = ops.RowTiles(row0, ctx.inputs[f"row_tiles/{size}/rows"], row0.shape[0], size)
        rotary = self.position.tables() if self.position is not None else None
        turn = self.value_position.tables() if self.value_position is not None else None
        q = ops.qk_prepare(proj, self.unit_gain, self.unit_gain, "head" if self.eps is not None else None, self.eps or 1.0,
                           rotary, ctx.rows, kv, self.n_q, False, entry.writes_cache, ctx.err, value_rotary=turn,
                           proj_offset=offset)
        a = ops.attention(q, ctx.rows, kv, self.n_q, self.scale, self.window, ctx.err, tiles, exact_weights=True,
                          sinks=self.sinks)
        ops.rotate_gate(a, proj, offset + self.gate_offset, self.n_q, self.value_dim, turn, ctx.rows, ctx.err, scale, out,
                        out_offset)
